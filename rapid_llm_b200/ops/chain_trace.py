"""Where a launch of the persistent product chain spends its time.

    python -m rapid_llm_b200.ops.chain_trace [--tokens 8] [--hidden 4096] [--intermediate 12288] [--qkv-rows 6144]

Runs the four products of a decoder layer (output projection with the residual add and the next norm's
weight, gate/up with the SiLU, down, the next layer's q/k/v) as one ``rl_gemm_chain`` launch on random
operands, with cold caches, and prints for every phase when the CTAs passed each of the kernel's time
stamps (minimum, median and maximum over the CTAs, microseconds from the first stamp); then the same four
products as separate launches for comparison.  The stamps are the kernel's own (``%globaltimer``).
"""

from __future__ import annotations

import argparse

import torch

from . import kernels

EVENTS = ["start barrier passed", "first accumulator complete", "last partial tile counted", "this CTA's tiles complete",
          "results stored", "last weight copy issued", "activation warp passed the start barrier", "last product committed"]


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--tokens", type=int, default=8)
    parser.add_argument("--hidden", type=int, default=4096)
    parser.add_argument("--intermediate", type=int, default=12288)
    parser.add_argument("--qkv-rows", type=int, default=6144)
    parser.add_argument("--device", default="cuda:0")
    args = parser.parse_args(argv)
    device, t, hidden, inter = torch.device(args.device), args.tokens, args.hidden, args.intermediate
    generator = torch.Generator(device=device).manual_seed(0)

    def rand(*shape):
        return (torch.randn(shape, generator=generator, device=device) * 0.03).to(torch.bfloat16)

    attended, w_o, w_gate_up = rand(t, hidden), rand(hidden, hidden), rand(2 * inter, hidden)
    w_down, w_qkv = rand(hidden, inter), rand(args.qkv_rows, hidden)
    norm = torch.ones(hidden, device=device)
    residual = torch.zeros((t, hidden), device=device)
    normed = torch.empty((t, hidden), dtype=torch.bfloat16, device=device)
    sumsq = torch.empty((t, kernels.gemm_bf16_sumsq_count(hidden)), device=device)
    act = torch.empty((t, inter), dtype=torch.bfloat16, device=device)
    qkv = torch.empty((t, args.qkv_rows), dtype=torch.bfloat16, device=device)
    fault = torch.zeros(1, dtype=torch.int32, device=device)
    products = [
        dict(x=attended, w=w_o, out=normed, residual=residual, norm_weight=norm, sumsq_out=sumsq),
        dict(x=normed, w=w_gate_up, out=act, swiglu=True, sumsq_in=sumsq, norm_eps=1e-6, norm_size=hidden),
        dict(x=act, w=w_down, out=normed, residual=residual, norm_weight=norm, sumsq_out=sumsq),
        dict(x=normed, w=w_qkv, out=qkv, sumsq_in=sumsq, norm_eps=1e-6, norm_size=hidden),
    ]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)       # larger than L2

    def one_by_one():
        for product in products:
            product = dict(product)
            kernels.gemm_bf16(product.pop("x"), product.pop("w"), product.pop("out"), fault, **product)

    def timed(run) -> float:
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        times = []
        for _ in range(13):
            flush.zero_()
            torch.cuda.synchronize()
            begin.record()
            run()
            end.record()
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end) * 1000.0)
        return sorted(times[3:])[5]

    weight_bytes = 2 * (hidden * hidden + 3 * inter * hidden + args.qkv_rows * hidden)
    print(f"{t} tokens; {weight_bytes / 1e6:.0f} MB of weights")
    print(f"one launch of the chain : {timed(lambda: kernels.gemm_chain(products, fault)):7.1f} us (CUDA events around the launch)")
    print(f"four separate launches  : {timed(one_by_one):7.1f} us")
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    trace = torch.zeros((sms, 4, 8), dtype=torch.int64, device=device)
    flush.zero_()
    torch.cuda.synchronize()
    kernels.gemm_chain(products, fault, trace=trace)
    torch.cuda.synchronize()
    stamps = trace.cpu().double()
    origin = stamps[stamps > 0].min()
    for phase, name in enumerate(("output projection", "gate/up + SiLU", "down", "q/k/v")):
        print(f"phase {phase} ({name})")
        for event, label in enumerate(EVENTS):
            column = stamps[:, phase, event]
            column = column[column > 0]
            if len(column):
                print(f"  {label:42s} min {float(column.min() - origin) / 1000:7.2f}  median {float(column.median() - origin) / 1000:7.2f}"
                      f"  max {float(column.max() - origin) / 1000:7.2f} us  ({len(column)} CTAs)")
    print("fault word", int(fault.item()))
    return 0 if int(fault.item()) == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
