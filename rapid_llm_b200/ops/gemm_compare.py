"""The bfloat16 product kernels against the library on a decoder layer's shapes.

    python -m rapid_llm_b200.ops.gemm_compare [--tokens 128,512,2048,4096] [--hidden 4096] [--intermediate 12288] [--qkv-rows 6144]

For every token count and each of the four shapes (q/k/v, output projection, gate/up as one plain product,
down) it first checks the pair kernel against the float32 product, then times, back to back in one process
and on rotating weights, the pair kernel (``tcgen05.mma.cta_group::2``), the library (cuBLAS through
``torch.mm``) and the streaming kernel whose tiles belong to one CTA each.  This is the measurement behind
which of them ``ops.gemm`` picks.
"""

from __future__ import annotations

import argparse

import torch

from . import kernels


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--tokens", default="128,512,2048,4096")
    parser.add_argument("--hidden", type=int, default=4096)
    parser.add_argument("--intermediate", type=int, default=12288)
    parser.add_argument("--qkv-rows", type=int, default=6144)
    parser.add_argument("--device", default="cuda:0")
    args = parser.parse_args(argv)
    device = torch.device(args.device)
    generator = torch.Generator(device=device).manual_seed(0)
    fault = torch.zeros(1, dtype=torch.int32, device=device)
    shapes = [("qkv", args.qkv_rows, args.hidden), ("o", args.hidden, args.hidden),
              ("gate_up", 2 * args.intermediate, args.hidden), ("down", args.hidden, args.intermediate)]

    def timed(run, iters=20) -> float:
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(iters):
            run()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / iters * 1e3

    for tokens in (int(t) for t in args.tokens.split(",")):
        for name, n, k in shapes:
            x = torch.randn((tokens, k), generator=generator, device=device).to(torch.bfloat16)
            weights = [(torch.randn((n, k), generator=generator, device=device) * 0.05).to(torch.bfloat16) for _ in range(3)]
            out = torch.full((tokens, n), float("nan"), dtype=torch.bfloat16, device=device)
            kernels.gemm_bf16_pair(x, weights[0], out, fault)
            want = x.float() @ weights[0].float().T
            wrong = int(((out.float() - want).abs() > 6e-3 * want.abs() + 2e-3).sum())
            turn = [0]

            def rotate():
                turn[0] += 1
                return weights[turn[0] % 3]

            pair = timed(lambda: kernels.gemm_bf16_pair(x, rotate(), out, fault))
            library = timed(lambda: torch.mm(x, rotate().t(), out=out))
            single = timed(lambda: kernels.gemm_bf16(x, rotate(), out, fault))
            flops = 2.0 * tokens * n * k
            print(f"T={tokens:5d} {name:8s} pair {pair:7.1f} us ({flops / pair / 1e6:5.0f} TFLOP/s)  library {library:7.1f} us "
                  f"({flops / library / 1e6:5.0f})  one CTA a tile {single:7.1f} us  library/pair {library / pair:.2f}  "
                  f"elements off {wrong}", flush=True)
        # the gate/up product with its activation: one kernel here, the library's product and the SiLU kernel there
        x = torch.randn((tokens, args.hidden), generator=generator, device=device).to(torch.bfloat16)
        weights = [(torch.randn((2 * args.intermediate, args.hidden), generator=generator, device=device) * 0.05).to(torch.bfloat16)
                   for _ in range(3)]
        act = torch.empty((tokens, args.intermediate), dtype=torch.bfloat16, device=device)
        wide = torch.empty((tokens, 2 * args.intermediate), dtype=torch.bfloat16, device=device)
        turn = [0]

        def rotate():
            turn[0] += 1
            return weights[turn[0] % 3]

        def library_then_silu():
            torch.mm(x, rotate().t(), out=wide)
            kernels.silu_mul(wide, act)

        fused = timed(lambda: kernels.gemm_bf16_pair(x, rotate(), act, fault, swiglu=True))
        apart = timed(library_then_silu)
        print(f"T={tokens:5d} gate_up with SiLU(gate) * up: pair, fused {fused:7.1f} us  library + activation kernel {apart:7.1f} us  "
              f"ratio {apart / fused:.2f}", flush=True)
    print("fault word", int(fault.item()))
    return 0 if int(fault.item()) == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
