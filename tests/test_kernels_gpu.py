"""Each CUDA kernel alone against a plain float32/float64 PyTorch reference of the same
operation, at sizes other than the engine tests' (widths and vocabularies that are no power
of two, head sizes 16 to 256, odd group counts, page sizes 1 to 64)."""

from __future__ import annotations

import math

import pytest
import torch
from plain_qwen3 import apply_rope, causal_attention, rms_norm, rope_angles, sample_token
from tolerances import for_dtype

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def k():
    from rapid_llm_b200.ops import kernels

    return kernels


def fault_word():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def rand(shape, dtype, scale=1.0, seed=0):
    generator = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=generator) * scale).to(dtype)


# ------------------------------------------------------------------ embedding
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,hidden", [(1000, 100), (37, 4096), (513, 72)])
def test_embedding(dtype, vocab, hidden):
    table = rand((vocab, hidden), dtype).to(DEV)
    ids = torch.randint(0, vocab, (50,), dtype=torch.int32).to(DEV)
    out = torch.empty((50, hidden), dtype=dtype, device=DEV)
    fault = fault_word()
    k().embedding(out, table, ids, fault)
    assert torch.equal(out, table[ids.long()])
    assert fault.item() == 0
    bad = ids.clone()
    bad[3] = vocab
    k().embedding(out, table, bad, fault)
    assert fault.item() == 1


# -------------------------------------------------------------------- rmsnorm
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [100, 1000, 4096, 5120])
def test_add_rmsnorm(dtype, hidden):
    rows, eps = 23, 3e-6
    x = rand((rows, hidden), dtype, seed=1).to(DEV)
    residual = rand((rows, hidden), torch.float32, seed=2).to(DEV)
    weight = (1 + 0.1 * rand((hidden,), torch.float32, seed=3)).to(DEV)
    out = torch.empty_like(x)
    tol = for_dtype(dtype)
    # first layer: residual := x
    r0 = residual.clone()
    k().add_rmsnorm(x, r0, weight, out, eps, mode=0, write_residual=True)
    torch.testing.assert_close(r0, x.float(), rtol=0, atol=0)
    torch.testing.assert_close(out.float(), rms_norm(x.float(), weight, eps), **tol)
    # later layers: residual += x
    r1 = residual.clone()
    k().add_rmsnorm(x, r1, weight, out, eps, mode=1, write_residual=True)
    want_sum = x.float() + residual
    torch.testing.assert_close(r1, want_sum, rtol=0, atol=0)
    torch.testing.assert_close(out.float(), rms_norm(want_sum, weight, eps), **tol)
    # final norm over chosen rows, residual untouched
    index = torch.tensor([5, 0, 22, 5], dtype=torch.int32, device=DEV)
    picked = torch.empty((4, hidden), dtype=dtype, device=DEV)
    r2 = residual.clone()
    k().add_rmsnorm(x, r2, weight, picked, eps, mode=1, write_residual=False, row_index=index)
    assert torch.equal(r2, residual)
    torch.testing.assert_close(picked.float(), rms_norm(want_sum, weight, eps)[index.long()], **tol)


# ------------------------------------------------------------------- silu mul
@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    rows, inter = 19, 1234
    gate_up = rand((rows, 2 * inter), dtype, scale=3.0).to(DEV)
    out = torch.empty((rows, inter), dtype=dtype, device=DEV)
    k().silu_mul(gate_up, out)
    gate, up = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    torch.testing.assert_close(out.float(), gate * torch.sigmoid(gate) * up, **for_dtype(dtype))


# -------------------------------------------------------------------- gemm f32
@pytest.mark.parametrize("m,n,k_", [(1, 53, 71), (37, 130, 64), (128, 257, 100), (200, 64, 1027), (3, 1000, 4096)])
def test_gemm_f32(m, n, k_):
    a = rand((m, k_), torch.float32, seed=4).to(DEV)
    w = rand((n, k_), torch.float32, seed=5).to(DEV)
    out = torch.empty((m, n), dtype=torch.float32, device=DEV)
    k().gemm_f32(a, w, out)
    want = (a.double() @ w.double().T).float()
    torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-5 * math.sqrt(k_))


def test_gemm_f32_rows_do_not_depend_on_the_batch():
    a = rand((70, 300), torch.float32, seed=6).to(DEV)
    w = rand((90, 300), torch.float32, seed=7).to(DEV)
    full = torch.empty((70, 90), dtype=torch.float32, device=DEV)
    k().gemm_f32(a, w, full)
    for row in (0, 33, 69):
        single = torch.empty((1, 90), dtype=torch.float32, device=DEV)
        k().gemm_f32(a[row : row + 1].contiguous(), w, single)
        assert torch.equal(single[0], full[row])


# ------------------------------------------------------------------- gemm bf16
def bf16_product(x, w, n, swiglu):
    ref = x.float() @ w.float().T
    if swiglu:
        ref = torch.nn.functional.silu(ref[:, :n]) * ref[:, n:]
    return ref


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize(
    "t,n,k_",
    [(1, 128, 64), (5, 100, 72), (8, 384, 96), (16, 256, 4096), (3, 1000, 1000), (33, 160, 208), (64, 777, 136),
     (100, 300, 200), (130, 256, 128), (300, 500, 264), (513, 130, 1024)],
)
def test_gemm_bf16(t, n, k_, swiglu):
    """The tcgen05 product at sizes that are no multiple of any tile, plain and with the fused SwiGLU."""
    x = rand((t, k_), torch.bfloat16, seed=20).to(DEV)
    w = rand(((2 if swiglu else 1) * n, k_), torch.bfloat16, scale=0.05, seed=21).to(DEV)
    out = torch.full((t, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    fault = fault_word()
    k().gemm_bf16(x, w, out, fault, swiglu=swiglu)
    assert fault.item() == 0
    want = bf16_product(x, w, n, swiglu)
    torch.testing.assert_close(out.float(), want, rtol=1e-2, atol=1e-2 * float(want.abs().max()) / 4 + 1e-3)


@pytest.mark.parametrize("t,n,k_", [(64, 12288, 520), (40, 4800, 264), (33, 3553, 136), (64, 25600, 136), (57, 12290, 72),
                                    (100, 12288, 264), (200, 17408, 136)])
def test_gemm_bf16_swiglu_tiles_that_fill_the_rounds(t, n, k_):
    """An unsplit SwiGLU product of 33 tokens and more takes weight tiles of fewer than 128 rows where 128-row tiles
    would leave its last round of one tile per multiprocessor part empty (12,288 rows: 140 tiles of 88 instead of 96
    of 128; 25,600 rows: two even rounds); the lanes past a tile's rows are never stored.  Every column against the
    float32 arithmetic, ragged widths included."""
    x = rand((t, k_), torch.bfloat16, seed=30).to(DEV)
    w = rand((2 * n, k_), torch.bfloat16, scale=0.05, seed=31).to(DEV)
    out = torch.full((t, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    fault = fault_word()
    k().gemm_bf16(x, w, out, fault, swiglu=True)
    assert fault.item() == 0
    want = bf16_product(x, w, n, True)
    assert not torch.isnan(out).any()
    torch.testing.assert_close(out.float(), want, rtol=1e-2, atol=1e-2 * float(want.abs().max()) / 4 + 1e-3)
    forced = torch.empty_like(out)
    k().gemm_bf16(x, w, forced, fault, swiglu=True, k_split=2 if t <= 64 else 1)      # 128-row tiles
    if t <= 64:
        torch.testing.assert_close(out.float(), forced.float(), rtol=1e-2, atol=1e-2 * float(want.abs().max()) / 4 + 1e-3)


@pytest.mark.parametrize("split", [2, 4, 8])
@pytest.mark.parametrize("t,n,k_,swiglu", [(8, 256, 4096, False), (33, 384, 1024, False), (64, 130, 12288, False),
                                           (7, 160, 1000, True), (60, 256, 2048, True)])
def test_gemm_bf16_inner_range_split_over_a_cluster(t, n, k_, swiglu, split):
    """Partial tiles summed through distributed shared memory equal the unsplit product's
    float32 sum up to the order of additions, and do not change from call to call."""
    x = rand((t, k_), torch.bfloat16, seed=22).to(DEV)
    w = rand(((2 if swiglu else 1) * n, k_), torch.bfloat16, scale=0.05, seed=23).to(DEV)
    fault = fault_word()
    outs = []
    for _ in range(2):
        out = torch.full((t, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        k().gemm_bf16(x, w, out, fault, swiglu=swiglu, k_split=split)
        outs.append(out)
    assert fault.item() == 0 and torch.equal(outs[0], outs[1])
    want = bf16_product(x, w, n, swiglu)
    torch.testing.assert_close(outs[0].float(), want, rtol=1e-2, atol=1e-2 * float(want.abs().max()) / 4 + 1e-3)


@pytest.mark.parametrize("split", [0, 1, 4])
@pytest.mark.parametrize("t,n,k_,swiglu", [(1, 130, 64, False), (8, 384, 1024, False), (40, 200, 520, True),
                                           (64, 256, 2048, True), (200, 300, 264, False), (300, 140, 512, True)])
def test_gemm_bf16_adds_a_bias(t, n, k_, swiglu, split):
    """A float32 bias per output column, for the fused SwiGLU per gate and per up column, added before the
    SiLU: in the direct epilogue and in the cluster's reduction."""
    if t > 64 and split > 1:
        pytest.skip("token tiles above 64 do not split the inner range")
    x = rand((t, k_), torch.bfloat16, seed=44).to(DEV)
    rows = (2 if swiglu else 1) * n
    w = rand((rows, k_), torch.bfloat16, scale=0.05, seed=45).to(DEV)
    bias = rand((rows,), torch.float32, scale=2.0, seed=46).to(DEV)
    out = torch.full((t, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    fault = fault_word()
    k().gemm_bf16(x, w, out, fault, swiglu=swiglu, k_split=split, bias=bias)
    assert fault.item() == 0
    want = x.float() @ w.float().T + bias
    if swiglu:
        want = torch.nn.functional.silu(want[:, :n]) * want[:, n:]
    torch.testing.assert_close(out.float(), want, rtol=6e-3, atol=2e-3)


@pytest.mark.parametrize("pdl", [False, True])
@pytest.mark.parametrize("t,hidden,inter,qkv_rows", [(1, 256, 384, 512), (8, 4096, 12288, 6144), (16, 520, 1000, 136),
                                                      (33, 1024, 2816, 1536), (64, 4096, 12288, 6144), (5, 128, 136, 72)])
def test_gemm_chain_runs_a_layers_products_as_one_kernel(t, hidden, inter, qkv_rows, pdl):
    """Output projection (residual add, the next norm's weight), gate/up with the SiLU (the row's scale),
    down (residual add, norm weight), q/k/v of the next layer (scale, a bias): four products in one
    persistent kernel, against float32 arithmetic and against the same products launched one by one; a
    second run on the same inputs gives the same bits (sums in segment order, counters back at zero)."""
    kernels = k()
    eps = 1e-5
    gen = lambda shape, scale, seed: device_rand(shape, scale, seed)      # noqa: E731
    attended = gen((t, hidden), 1.0, 50)
    w_o, w_gu = gen((hidden, hidden), 0.03, 51), gen((2 * inter, hidden), 0.03, 52)
    w_down, w_qkv = gen((hidden, inter), 0.03, 53), gen((qkv_rows, hidden), 0.03, 54)
    norm1 = (1.0 + 0.2 * torch.randn(hidden, generator=torch.Generator().manual_seed(55))).to(DEV)
    norm2 = (1.0 + 0.2 * torch.randn(hidden, generator=torch.Generator().manual_seed(56))).to(DEV)
    bias = torch.randn(qkv_rows, generator=torch.Generator().manual_seed(57)).to(DEV)
    residual0 = torch.randn((t, hidden), generator=torch.Generator().manual_seed(58)).to(DEV) * 2.0
    residual0[t // 2] *= 20.0                      # a scale taken from the wrong row shows

    def run(chain: bool):
        residual = residual0.clone()
        normed = torch.full((t, hidden), float("nan"), dtype=torch.bfloat16, device=DEV)
        sumsq = torch.full((t, kernels.gemm_bf16_sumsq_count(hidden)), float("nan"), dtype=torch.float32, device=DEV)
        act = torch.full((t, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
        qkv = torch.full((t, qkv_rows), float("nan"), dtype=torch.bfloat16, device=DEV)
        fault = fault_word()
        products = [
            dict(x=attended, w=w_o, out=normed, residual=residual, norm_weight=norm1, sumsq_out=sumsq),
            dict(x=normed, w=w_gu, out=act, swiglu=True, sumsq_in=sumsq, norm_eps=eps, norm_size=hidden),
            dict(x=act, w=w_down, out=normed, residual=residual, norm_weight=norm2, sumsq_out=sumsq),
            dict(x=normed, w=w_qkv, out=qkv, sumsq_in=sumsq, norm_eps=eps, norm_size=hidden, bias=bias),
        ]
        kernels.PDL = pdl
        try:
            if chain:
                kernels.gemm_chain(products, fault)
            else:
                for product in products:
                    product = dict(product)
                    kernels.gemm_bf16(product.pop("x"), product.pop("w"), product.pop("out"), fault, **product)
        finally:
            kernels.PDL = False
        assert fault.item() == 0
        return residual, act, qkv

    residual, act, qkv = run(chain=True)
    again = run(chain=True)
    assert all(torch.equal(a, b) for a, b in zip((residual, act, qkv), again))

    r1 = residual0 + attended.float() @ w_o.float().T
    x1 = rms_norm(r1, norm1, eps)
    gate_up = x1 @ w_gu.float().T
    want_act = torch.nn.functional.silu(gate_up[:, :inter]) * gate_up[:, inter:]
    r2 = r1 + want_act.to(torch.bfloat16).float() @ w_down.float().T
    want_qkv = rms_norm(r2, norm2, eps) @ w_qkv.float().T + bias
    one_by_one = run(chain=False)
    # intermediate roundings to bfloat16 differ between the float32 arithmetic and both kernels: loose against
    # the arithmetic, tight between the two ways of launching
    torch.testing.assert_close(act.float(), want_act, rtol=3e-2, atol=3e-2 * float(want_act.abs().max()) / 4)
    torch.testing.assert_close(residual, r2, rtol=2e-2, atol=2e-2 * float(r2.abs().mean()))
    torch.testing.assert_close(qkv.float(), want_qkv, rtol=3e-2, atol=3e-2 * float(want_qkv.abs().max()) / 4)
    for got, other in zip((residual, act, qkv), one_by_one):
        torch.testing.assert_close(got.float(), other.float(), rtol=1e-2, atol=1e-2 * float(other.float().abs().max()) / 4)


def device_rand(shape, scale, seed):
    """Large operands are drawn on the device: a billion normal draws take the CPU tens of seconds."""
    generator = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(shape, generator=generator, device=DEV) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("t,n,k_,swiglu", [
    (1, 151936, 4096, False), (8, 151936, 4096, False), (64, 151936, 4096, False),     # the output head: 1,187 tiles
    (33, 75000, 512, False),                       # 586 tiles of 64 tokens over fewer CTAs, short inner range
    (2048, 6144, 4096, False),                     # 48 x 8 tiles of 256 tokens, one CTA per SM
    (2048, 12288, 4096, True), (700, 9000, 1000, True),   # the fused SwiGLU's 128-token tiles, ragged edges
    (300, 40000, 520, False),
])
def test_gemm_bf16_when_a_cta_walks_several_tiles(t, n, k_, swiglu):
    """More tiles than CTAs: every CTA takes tile after tile, the accumulators alternate between two
    tensor-memory buffers and the barriers' phases flip.  Each output is compared with the float32
    product; an element's bound is the rounding of its bfloat16 store plus that of a float32 sum."""
    x = device_rand((t, k_), 1.0, seed=40)
    w = device_rand(((2 if swiglu else 1) * n, k_), 0.05, seed=41)
    out = torch.full((t, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    fault = fault_word()
    k().gemm_bf16(x, w, out, fault, swiglu=swiglu)
    assert fault.item() == 0
    step = 8192                                    # the float32 reference in slabs of output columns
    for begin in range(0, n, step):
        end = min(n, begin + step)
        want = x.float() @ w[begin:end].float().T
        if swiglu:
            want = torch.nn.functional.silu(want) * (x.float() @ w[n + begin : n + end].float().T)
        torch.testing.assert_close(out[:, begin:end].float(), want, rtol=6e-3, atol=2e-3)


@pytest.mark.parametrize("t,n,k_,bias", [
    (65, 136, 64, False), (128, 256, 128, True), (256, 256, 256, False),      # one tile, shared by as many pairs as get eight k-blocks
    (300, 520, 264, True), (100, 6144, 4096, False),                          # ragged edges; the 128-token tile
    (512, 4096, 12288, False),                                                # 32 tiles, every one shared by two or three pairs
    (1000, 1304, 1024, True),
    (2048, 6144, 4096, False),                                                # 192 tiles on 74 pairs: two whole rounds and 44 shared tiles
    (2048, 24576, 4096, False), (4096, 4096, 12288, True),
])
def test_gemm_bf16_pair_of_ctas_on_one_tile(t, n, k_, bias):
    """``tcgen05.mma.cta_group::2``: two CTAs, each with half of a 256 x 256 tile's operands, one issuing thread;
    whole rounds of tiles dealt round-robin, the left-over tiles' k-ranges shared between pairs and summed by the
    owner in run order.  Against the float32 product; a second call gives the same bits."""
    x = device_rand((t, k_), 1.0, seed=60)
    w = device_rand((n, k_), 0.05, seed=61)
    b = torch.randn(n, generator=torch.Generator().manual_seed(62)).to(DEV) if bias else None
    fault = fault_word()
    outs = []
    for _ in range(2):
        out = torch.full((t, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        k().gemm_bf16_pair(x, w, out, fault, bias=b)
        outs.append(out)
    assert fault.item() == 0 and torch.equal(outs[0], outs[1])
    step = 4096
    for begin in range(0, n, step):
        end = min(n, begin + step)
        want = x.float() @ w[begin:end].float().T
        if bias:
            want = want + b[begin:end]
        torch.testing.assert_close(outs[0][:, begin:end].float(), want, rtol=6e-3, atol=2e-3)


@pytest.mark.parametrize("t,n,k_,options", [
    (128, 256, 128, {"swiglu"}), (300, 200, 320, {"swiglu", "bias", "scale"}), (1030, 1544, 520, {"swiglu", "scale"}),
    (2048, 12288, 4096, {"swiglu", "scale"}),                                  # the gate/up product of a prompt step
    (512, 1024, 256, {"norm"}), (333, 392, 320, {"norm", "scale", "bias"}), (700, 4096, 2048, {"norm"}),
    (260, 264, 72, {"scale"}),
])
def test_gemm_bf16_pair_rows_are_the_threads_own(t, n, k_, options):
    """The tokens are the accumulator's lanes, so the scale a norm left open, a bias, SiLU(gate) * up and the norm
    that follows (residual, weight, sums of squares per 32 columns) are applied by the thread that owns the row;
    whole tiles, ragged edges and tiles whose k-range several pairs share.  Against float32 arithmetic."""
    kernels = k()
    swiglu, norm = "swiglu" in options, "norm" in options
    x = device_rand((t, k_), 0.5, seed=70)
    w = device_rand(((2 if swiglu else 1) * n, k_), 0.05, seed=71)
    want = x.float() @ w.float().T
    extra = {}
    if "scale" in options:
        sumsq = torch.rand((t, 8), generator=torch.Generator().manual_seed(72)).to(DEV) * k_ / 8
        extra.update(sumsq_in=sumsq, norm_eps=1e-5, norm_size=k_)
        want = want * torch.rsqrt(sumsq.sum(1, keepdim=True) / k_ + 1e-5)
    bias = torch.randn(w.shape[0], generator=torch.Generator().manual_seed(73)).to(DEV) if "bias" in options else None
    if bias is not None:
        want = want + bias
    if swiglu:
        want = torch.nn.functional.silu(want[:, :n]) * want[:, n:]
    if norm:
        residual = torch.randn((t, n), generator=torch.Generator().manual_seed(74)).to(DEV)
        before = residual.clone()
        weight = torch.rand(n, generator=torch.Generator().manual_seed(75)).to(DEV) + 0.5
        table = torch.full((t, kernels.gemm_bf16_sumsq_count(n)), float("nan"), device=DEV)
        extra.update(residual=residual, norm_weight=weight, sumsq_out=table)
    out = torch.full((t, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    fault = fault_word()
    kernels.gemm_bf16_pair(x, w, out, fault, bias=bias, swiglu=swiglu, **extra)
    assert fault.item() == 0
    if norm:
        after = before + want
        torch.testing.assert_close(residual, after, rtol=1e-5, atol=2e-4 * max(1.0, float(want.abs().max())))
        torch.testing.assert_close(table.sum(1), (after**2).sum(1), rtol=1e-4, atol=1e-3)
        want = after * weight
    torch.testing.assert_close(out.float(), want, rtol=8e-3, atol=2e-3 * max(1.0, float(want.abs().max())))


def test_gemm_bf16_pair_says_which_products_it_takes():
    """The router asks before it calls: a width that is no multiple of 8, or more tiles than the kernel's table
    holds (4,096: 32,768 tokens by 25,600 gated columns are 25,600), goes to the library instead."""
    kernels = k()
    assert kernels.gemm_bf16_pair_takes(2048, 12288, True) and kernels.gemm_bf16_pair_takes(8192, 25600, False)
    assert not kernels.gemm_bf16_pair_takes(2048, 12290, True)
    assert not kernels.gemm_bf16_pair_takes(32768, 25600, True)
    assert kernels.gemm_bf16_pair_takes(256 * 32, 128 * 128, True) and not kernels.gemm_bf16_pair_takes(256 * 32 + 1, 128 * 128, True)


def test_gemm_bf16_pair_refuses_a_width_that_is_no_multiple_of_8():
    kernels = k()
    with pytest.raises(kernels.KernelError):
        kernels.gemm_bf16_pair(torch.zeros((300, 64), dtype=torch.bfloat16, device=DEV), torch.zeros((130, 64), dtype=torch.bfloat16, device=DEV),
                               torch.zeros((300, 130), dtype=torch.bfloat16, device=DEV), fault_word())


@pytest.mark.parametrize("split", [0, 1, 2, 4, 8])
@pytest.mark.parametrize("t,n,k_,swiglu", [(16, 300, 1024, False), (64, 256, 4096, False), (40, 57100, 640, False),
                                           (64, 200, 4096, True), (128, 260, 2048, False), (256, 300, 1024, False)])
def test_gemm_bf16_every_block_of_the_inner_range_counts(t, n, k_, swiglu, split):
    """Row ``r`` of the input is zero outside the 64 inner elements of block ``r mod blocks``: a block that
    a CTA skips, reads twice or reads from the wrong stage changes a whole output row by its full size,
    at every edge between the ranks of a split and in the last, partial, block."""
    if t > 64 and split not in (0, 1):
        pytest.skip("token tiles above 64 do not split the inner range")
    blocks = -(-k_ // 64)
    x = rand((t, k_), torch.bfloat16, seed=42)
    keep = torch.zeros((t, k_), dtype=torch.bool)
    for row in range(t):
        block = row % blocks
        keep[row, block * 64 : (block + 1) * 64] = True
    x = torch.where(keep, x, torch.zeros_like(x)).to(DEV)
    w = device_rand(((2 if swiglu else 1) * n, k_), 0.3, seed=43)
    out = torch.full((t, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    fault = fault_word()
    k().gemm_bf16(x, w, out, fault, swiglu=swiglu, k_split=split)
    assert fault.item() == 0
    want = bf16_product(x, w, n, swiglu)
    assert float(want.abs().mean()) > 0.5          # a lost block is far outside the bound
    torch.testing.assert_close(out.float(), want, rtol=6e-3, atol=2e-3)


@pytest.mark.parametrize("t,n,k_,swiglu", [(300, 520, 1000, False), (1024, 4096, 4096, False), (1100, 1536, 2048, True),
                                           (2048, 512, 12288, False)])
def test_gemm_bf16_pair_every_block_of_the_inner_range_counts(t, n, k_, swiglu):
    """The same for the kernel on pairs of CTAs: row ``r`` of the input lives in block ``r mod blocks`` alone, so a
    k-block that a pair skips, reads twice or sums twice where the runs of two pairs meet inside a tile (the left-over
    tiles' k-ranges are shared) changes whole rows by their full size."""
    blocks = -(-k_ // 64)
    x = rand((t, k_), torch.bfloat16, seed=44)
    keep = torch.zeros((t, k_), dtype=torch.bool)
    rows = torch.arange(t)
    for block in range(blocks):
        keep[rows[rows % blocks == block], block * 64 : (block + 1) * 64] = True
    x = torch.where(keep, x, torch.zeros_like(x)).to(DEV)
    w = device_rand(((2 if swiglu else 1) * n, k_), 0.3, seed=45)
    out = torch.full((t, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    fault = fault_word()
    k().gemm_bf16_pair(x, w, out, fault, swiglu=swiglu)
    assert fault.item() == 0
    want = bf16_product(x, w, n, swiglu)
    assert float(want.abs().mean()) > (0.05 if swiglu else 0.5)          # a lost block is far outside the bound
    torch.testing.assert_close(out.float(), want, rtol=6e-3, atol=2e-3 * max(1.0, float(want.abs().max()) / 8))


def test_gemm_bf16_rows_do_not_depend_on_the_batch_beyond_rounding():
    x = rand((40, 512), torch.bfloat16, seed=24).to(DEV)
    w = rand((300, 512), torch.bfloat16, scale=0.05, seed=25).to(DEV)
    fault = fault_word()
    full = torch.empty((40, 300), dtype=torch.bfloat16, device=DEV)
    k().gemm_bf16(x, w, full, fault)
    single = torch.empty((1, 300), dtype=torch.bfloat16, device=DEV)
    k().gemm_bf16(x[17:18].contiguous(), w, single, fault)
    torch.testing.assert_close(single[0].float(), full[17].float(), rtol=1e-2, atol=2e-2)


def test_gemm_bf16_under_programmatic_dependent_launch():
    """With the early-start attribute set, a chain of products still sees its predecessor's output."""
    kernels = k()
    x = rand((8, 1024), torch.bfloat16, seed=26).to(DEV)
    w1 = rand((1024, 1024), torch.bfloat16, scale=0.03, seed=27).to(DEV)
    w2 = rand((512, 1024), torch.bfloat16, scale=0.03, seed=28).to(DEV)
    fault = fault_word()
    mid, out = torch.empty((8, 1024), dtype=torch.bfloat16, device=DEV), torch.empty((8, 512), dtype=torch.bfloat16, device=DEV)
    kernels.PDL = True
    try:
        for _ in range(20):
            kernels.gemm_bf16(x, w1, mid, fault)
            kernels.gemm_bf16(mid, w2, out, fault)
    finally:
        kernels.PDL = False
    assert fault.item() == 0
    want_mid = (x.float() @ w1.float().T).to(torch.bfloat16)
    want = want_mid.float() @ w2.float().T
    torch.testing.assert_close(mid.float(), want_mid.float(), rtol=1e-2, atol=2e-2)
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=3e-2)


@pytest.mark.parametrize("pdl", [False, True])
@pytest.mark.parametrize("split", [0, 1, 2, 8])
@pytest.mark.parametrize("swiglu_after", [False, True])
@pytest.mark.parametrize("t,k_,width,n_after", [(1, 64, 128, 128), (5, 200, 328, 136), (8, 4096, 1024, 256),
                                                (33, 1000, 520, 100), (64, 264, 96, 384)])
def test_gemm_bf16_takes_a_norm_along(t, k_, width, n_after, swiglu_after, split, pdl):
    """A product that adds to the residual, applies the norm's weight and leaves the squares, then
    a product that applies the row's scale: together ``norm(residual + x W^T) W2^T``."""
    kernels = k()
    eps = 3e-5
    x = rand((t, k_), torch.bfloat16, seed=30).to(DEV)
    w = rand((width, k_), torch.bfloat16, scale=0.05, seed=31).to(DEV)
    w_after = rand(((2 if swiglu_after else 1) * n_after, width), torch.bfloat16, scale=0.05, seed=32).to(DEV)
    residual = rand((t, width), torch.float32, scale=2.0, seed=33).to(DEV)
    norm_weight = (1.0 + rand((width,), torch.float32, scale=0.2, seed=34)).to(DEV)
    # one row far larger than the others: a scale taken from the wrong row shows
    residual[t // 2] *= 30.0
    want_residual = residual + x.float() @ w.float().T
    want_normed = rms_norm(want_residual, norm_weight, eps)
    want = bf16_product(want_normed, w_after, n_after, swiglu_after)

    fault = fault_word()
    rows = torch.full((t, width), float("nan"), dtype=torch.bfloat16, device=DEV)
    sumsq = torch.full((t, kernels.gemm_bf16_sumsq_count(width)), float("nan"), dtype=torch.float32, device=DEV)
    out = torch.full((t, n_after), float("nan"), dtype=torch.bfloat16, device=DEV)
    kernels.PDL = pdl
    try:
        kernels.gemm_bf16(x, w, rows, fault, k_split=split, residual=residual, norm_weight=norm_weight, sumsq_out=sumsq)
        kernels.gemm_bf16(rows, w_after, out, fault, swiglu=swiglu_after, k_split=split,
                          sumsq_in=sumsq, norm_eps=eps, norm_size=width)
    finally:
        kernels.PDL = False
    assert fault.item() == 0
    torch.testing.assert_close(residual, want_residual, rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(sumsq.sum(dim=1), want_residual.square().sum(dim=1), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(rows.float(), want_residual * norm_weight, rtol=1e-2, atol=1e-3)
    torch.testing.assert_close(out.float(), want, rtol=1e-2, atol=1e-2 * float(want.abs().max()) / 4 + 1e-3)


def test_gemm_bf16_norm_refusals():
    kernels = k()
    x = torch.zeros((65, 64), dtype=torch.bfloat16, device=DEV)
    w = torch.zeros((128, 64), dtype=torch.bfloat16, device=DEV)
    out = torch.zeros((65, 128), dtype=torch.bfloat16, device=DEV)
    residual = torch.zeros((65, 128), dtype=torch.float32, device=DEV)
    weight = torch.ones((128,), dtype=torch.float32, device=DEV)
    sumsq = torch.zeros((65, 4), dtype=torch.float32, device=DEV)
    with pytest.raises(kernels.KernelError, match="at most 64"):
        kernels.gemm_bf16(x, w, out, fault_word(), residual=residual, norm_weight=weight, sumsq_out=sumsq)
    with pytest.raises(kernels.KernelError, match="needs residual"):
        kernels.gemm_bf16(x[:8], w, out[:8], fault_word(), residual=residual[:8])
    with pytest.raises(kernels.KernelError, match="sumsq_in"):
        kernels.gemm_bf16(x[:8], w, out[:8], fault_word(), sumsq_in=sumsq[:8, :3].contiguous(), norm_size=64)


def test_gemm_bf16_refuses_rows_that_are_no_multiple_of_16_bytes():
    kernels = k()
    with pytest.raises(kernels.KernelError):
        kernels.gemm_bf16(torch.zeros((4, 100), dtype=torch.bfloat16, device=DEV), torch.zeros((8, 100), dtype=torch.bfloat16, device=DEV),
                          torch.zeros((4, 8), dtype=torch.bfloat16, device=DEV), fault_word())


# ---------------------------------------------------- q/k norm + rope + cache write
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,rotary,page", [(4, 2, 16, 16, 4), (6, 1, 48, 48, 8), (5, 5, 128, 64, 16), (3, 3, 256, 256, 1)])
def test_qk_norm_rope_write(dtype, hq, hkv, d, rotary, page):
    check_qk_norm_rope_write(dtype, hq, hkv, d, rotary, page, tokens=21, pages=40)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,tokens", [(6, 2, 7600), (5, 1, 11000), (32, 8, 1600), (32, 8, 300), (32, 8, 190)])
def test_qk_norm_rope_write_with_many_tokens(dtype, hq, hkv, tokens):
    """Enough tokens that a warp takes a run of heads of its token (10 heads: runs of 8 and 2; 7 heads: a query
    and a key head, a value head and none share a warp instruction; the 48 heads of the 8B shape)."""
    check_qk_norm_rope_write(dtype, hq=hq, hkv=hkv, d=128, rotary=128, page=16, tokens=tokens, pages=tokens // 16 + 30)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,d,tokens", [(6, 32, 21), (3, 128, 40), (32, 128, 320), (5, 128, 2000)])
def test_qk_norm_rope_write_of_queries_alone(dtype, hq, d, tokens):
    """A layer that reads another layer's cache has queries only: rows of ``hq`` heads, nothing written to pages
    (few tokens, and enough of them for the kernel that gives a warp a run of heads)."""
    eps, theta, max_pos = 1e-6, 10000.0, 500
    q_in = rand((tokens, hq * d), dtype, seed=18).to(DEV)
    qw = (1 + 0.1 * rand((d,), torch.float32, seed=19)).to(DEV)
    positions = torch.randint(0, max_pos, (tokens,), dtype=torch.int32)
    cos, sin = rope_angles(torch.arange(max_pos), d, theta)
    q_out = torch.empty((tokens, hq * d), dtype=dtype, device=DEV)
    fault = fault_word()
    k().qk_norm_rope_write(
        q_in, q_out, num_heads=hq, num_kv_heads=2, head_dim=d, rotary_dim=d,
        cos=cos.to(DEV).contiguous(), sin=sin.to(DEV).contiguous(), positions=positions.to(DEV), eps=eps,
        fault=fault, q_weight=qw, k_weight=None, kv_dest=None, cache=None, page_size=16,
    )
    assert fault.item() == 0
    c, s = cos[positions.long()], sin[positions.long()]
    want = apply_rope(rms_norm(q_in.float().cpu().view(tokens, hq, d), qw.cpu(), eps), c, s)
    torch.testing.assert_close(q_out.float().cpu().view(tokens, hq, d), want, **for_dtype(dtype))


def check_qk_norm_rope_write(dtype, hq, hkv, d, rotary, page, tokens, pages):
    eps, theta, max_pos = 1e-5, 50000.0, 300
    qkv = rand((tokens, (hq + 2 * hkv) * d), dtype, seed=8).to(DEV)
    qw = (1 + 0.1 * rand((d,), torch.float32, seed=9)).to(DEV)
    kw = (1 + 0.1 * rand((d,), torch.float32, seed=10)).to(DEV)
    positions = torch.randint(0, max_pos, (tokens,), dtype=torch.int32)
    cos, sin = rope_angles(torch.arange(max_pos), rotary, theta)
    dest = torch.randperm(pages * page)[:tokens].to(torch.int32)
    cache = torch.zeros((pages, 2, hkv, page, d), dtype=dtype, device=DEV)
    q_out = torch.empty((tokens, hq * d), dtype=dtype, device=DEV)
    fault = fault_word()
    k().qk_norm_rope_write(
        qkv, q_out, num_heads=hq, num_kv_heads=hkv, head_dim=d, rotary_dim=rotary,
        cos=cos.to(DEV).contiguous(), sin=sin.to(DEV).contiguous(), positions=positions.to(DEV), eps=eps,
        fault=fault, q_weight=qw, k_weight=kw, kv_dest=dest.to(DEV), cache=cache, page_size=page,
    )
    assert fault.item() == 0
    host = qkv.float().cpu()
    q = host[:, : hq * d].view(tokens, hq, d)
    key = host[:, hq * d : (hq + hkv) * d].view(tokens, hkv, d)
    value = host[:, (hq + hkv) * d :].view(tokens, hkv, d)
    c, s = cos[positions.long()], sin[positions.long()]
    want_q = apply_rope(rms_norm(q, qw.cpu(), eps), c, s)
    want_k = apply_rope(rms_norm(key, kw.cpu(), eps), c, s)
    tol = for_dtype(dtype)
    torch.testing.assert_close(q_out.float().cpu().view(tokens, hq, d), want_q, **tol)
    got = cache.float().cpu()
    page_id, offset = dest.long() // page, dest.long() % page
    torch.testing.assert_close(got[page_id, 0, :, offset], want_k, **tol)
    torch.testing.assert_close(got[page_id, 1, :, offset], value, rtol=0, atol=0)
    untouched = torch.ones(pages * page, dtype=torch.bool)
    untouched[dest.long()] = False
    flat = got.permute(0, 3, 1, 2, 4).reshape(pages * page, -1)
    assert flat[untouched].abs().max() == 0


# ------------------------------------------------------------------ attention
def paged_case(dtype, hq, hkv, d, page, lengths, new_counts, seed=0, key_scale=1.0):
    """A cache with shuffled pages holding ``lengths`` tokens per request; the last
    ``new_counts`` of each are the step's queries."""
    generator = torch.Generator().manual_seed(seed)
    slots = len(lengths) + 2
    max_pages = max(-(-n // page) for n in lengths) + 1
    total_pages = sum(-(-n // page) for n in lengths) + 3
    order = (torch.randperm(total_pages - 1, generator=generator) + 1).tolist()
    table = torch.zeros((slots, max_pages), dtype=torch.int32)
    cache = torch.zeros((total_pages, 2, hkv, page, d), dtype=torch.float32)
    keys, values, queries = [], [], []
    positions, token_slot = [], []
    slot_ids = torch.randperm(slots, generator=generator)[: len(lengths)].tolist()
    for slot, length, new in zip(slot_ids, lengths, new_counts):
        key = torch.randn((length, hkv, d), generator=generator) * key_scale
        value = torch.randn((length, hkv, d), generator=generator)
        query = torch.randn((length, hq, d), generator=generator)
        keys.append(key), values.append(value), queries.append(query)
        for index in range(-(-length // page)):
            page_id = order.pop()
            table[slot, index] = page_id
            chunk = slice(index * page, min(length, (index + 1) * page))
            count = chunk.stop - chunk.start
            cache[page_id, 0, :, :count] = key[chunk].transpose(0, 1)
            cache[page_id, 1, :, :count] = value[chunk].transpose(0, 1)
        positions.extend(range(length - new, length))
        token_slot.extend([slot] * new)
    q = torch.cat([query[length - new :] for query, length, new in zip(queries, lengths, new_counts)])
    return {
        "q": q.to(dtype), "cache": cache.to(dtype), "table": table,
        "positions": torch.tensor(positions, dtype=torch.int32),
        "token_slot": torch.tensor(token_slot, dtype=torch.int32),
        "keys": keys, "values": values, "queries": queries, "slots": slot_ids,
    }


def plain_paged(case, dtype, lengths, new_counts, scale, window):
    outs = []
    for key, value, query, length, new in zip(case["keys"], case["values"], case["queries"], lengths, new_counts):
        cast = lambda t: t.to(dtype).float()  # noqa: E731  (what the kernel reads)
        full = causal_attention(cast(query), cast(key), cast(value), scale, window)
        outs.append(full[length - new :])
    return torch.cat(outs)


def run_generic(case, hq, hkv, d, scale, window):
    q = case["q"].to(DEV).contiguous()
    out = torch.empty_like(q)
    fault = fault_word()
    k().attention_generic(
        q, case["cache"].to(DEV), out, positions=case["positions"].to(DEV),
        token_slot=case["token_slot"].to(DEV), block_table=case["table"].to(DEV),
        num_heads=hq, num_kv_heads=hkv, head_dim=d, window=window, scale=scale, fault=fault,
    )
    assert fault.item() == 0
    return out.float().cpu()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(
    "hq,hkv,d,page,window",
    [(4, 2, 16, 16, 0), (6, 1, 32, 8, 0), (7, 7, 48, 4, 0), (8, 2, 128, 16, 0), (3, 1, 256, 64, 0),
     (6, 3, 64, 16, 40), (4, 4, 80, 1, 7), (10, 2, 96, 32, 33)],
)
def test_attention_generic(dtype, hq, hkv, d, page, window):
    lengths = [1, 15, 16, 17, 129, 200, 64]
    new_counts = [1, 15, 1, 2, 129, 1, 33]
    case = paged_case(dtype, hq, hkv, d, page, lengths, new_counts, seed=d + page)
    scale = d**-0.5
    got = run_generic(case, hq, hkv, d, scale, window)
    want = plain_paged(case, dtype, lengths, new_counts, scale, window)
    torch.testing.assert_close(got, want, **for_dtype(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key_and_respects_the_window_edge(dtype):
    """One key among hundreds is made to dominate: the output must be its value, unless the
    window has just passed it."""
    hq, hkv, d, page = 4, 2, 64, 16
    length, far = 700, 13
    case = paged_case(dtype, hq, hkv, d, page, [length], [1], seed=3)
    query = case["queries"][0][-1]                       # [hq, d]
    for head in range(hkv):
        case["keys"][0][far, head] = 40.0 * query[head * (hq // hkv)] / query[head * (hq // hkv)].norm()
    page_id = int(case["table"][case["token_slot"][0], far // page])
    case["cache"][page_id, 0, :, far % page] = case["keys"][0][far].to(dtype)
    scale = d**-0.5
    for window, expect_far in [(0, True), (length - far, True), (length - far - 1, False)]:
        got = run_generic(case, hq, hkv, d, scale, window)
        want = plain_paged(case, dtype, [length], [1], scale, window)
        torch.testing.assert_close(got, want, **for_dtype(dtype))
        first_head = got.view(1, hq, d)[0, 0]
        value = case["values"][0][far, 0].to(dtype).float()
        close = (first_head - value).abs().max() < 0.15
        assert bool(close) == expect_far


def run_mma(case, lengths, new_counts, hq, hkv, d, scale, window, splits=None, decode_kernel="auto", page=0):
    """The tensor-core kernels over the same paged case, items cut by the part's own planner.

    ``page`` (the cache's page size) lets the planner cut chunk tiles for the tcgen05 kernel
    where it applies; 0 keeps the mma.sync tiles."""
    import numpy as np

    from rapid_llm_b200.parts.attention import AttentionItems
    from rapid_llm_b200.parts.base import StepShape

    starts = [length - new for length, new in zip(lengths, new_counts)]
    planner = AttentionItems(hq // hkv, hkv, d)
    shape = StepShape(np.asarray(new_counts, dtype=np.int32), np.asarray(starts, dtype=np.int32),
                      decode_only=max(new_counts) == 1, page_size=page)
    plan = planner.plan(shape)
    if splits is not None and splits != plan["splits"]:
        def respread(items):
            base = items[items[:, 2] == 0]
            out = np.repeat(base, splits, axis=0)
            out[:, 2] = np.tile(np.arange(splits, dtype=np.int32), len(base))
            return out
        plan = dict(plan, chunk_items=respread(plan["chunk_items"]), decode_items=respread(plan["decode_items"]), splits=splits)
    q = case["q"].to(DEV).reshape(-1, hq * d).contiguous()
    out = torch.full_like(q, float("nan"))
    tokens = q.shape[0]
    count = plan["splits"]
    part_out = part_lse = None
    if count > 1:
        part_out = torch.full((tokens * hq * count, d), float("nan"), dtype=torch.float32, device=DEV)
        part_lse = torch.full((tokens * hq * count,), float("nan"), dtype=torch.float32, device=DEV)
    cu = torch.tensor([0] + list(np.cumsum(new_counts)), dtype=torch.int32, device=DEV)
    fault = fault_word()
    k().attention_mma(
        q, case["cache"].to(DEV), out,
        chunk_items=torch.from_numpy(plan["chunk_items"]).to(DEV), decode_items=torch.from_numpy(plan["decode_items"]).to(DEV),
        splits=count, part_out=part_out, part_lse=part_lse, cu_seqlens=cu,
        entry_start=torch.tensor(starts, dtype=torch.int32, device=DEV),
        entry_slot=torch.tensor(case["slots"], dtype=torch.int32, device=DEV),
        block_table=case["table"].to(DEV), num_heads=hq, num_kv_heads=hkv, head_dim=d,
        window=window, scale=scale, fault=fault, decode_kernel=decode_kernel,
        decode_rows=plan.get("decode_rows", 0), chunk_rows=plan.get("chunk_rows", 64),
    )
    assert fault.item() == 0
    return out.float().cpu().view(tokens, hq, d)


@pytest.mark.parametrize(
    "hq,hkv,d,page,window,splits",
    [(8, 2, 128, 16, 0, None), (8, 2, 128, 16, 0, 3), (6, 1, 32, 8, 0, None), (7, 7, 48, 4, 0, 2),
     (4, 2, 16, 16, 0, None), (3, 1, 256, 64, 0, None), (6, 3, 64, 16, 40, None), (6, 3, 64, 16, 40, 4),
     (4, 4, 80, 1, 7, None), (10, 2, 96, 32, 33, 5), (40, 2, 64, 16, 0, None), (32, 8, 128, 16, 300, 2)],
)
def test_attention_mma(hq, hkv, d, page, window, splits):
    """Chunk tiles and decode tiles in one launch, whole and with split key ranges."""
    dtype = torch.bfloat16
    lengths = [1, 15, 16, 17, 129, 200, 64, 700, 333]
    new_counts = [1, 15, 1, 2, 129, 1, 33, 1, 70]
    case = paged_case(dtype, hq, hkv, d, page, lengths, new_counts, seed=d + page)
    scale = d**-0.5
    got = run_mma(case, lengths, new_counts, hq, hkv, d, scale, window, splits)
    want = plain_paged(case, dtype, lengths, new_counts, scale, window)
    torch.testing.assert_close(got, want, **for_dtype(dtype))


@pytest.mark.parametrize("decode_kernel", ["auto", "mma", "deep", "shallow"])
@pytest.mark.parametrize(
    "hq,hkv,page,window,splits,lengths,new_counts",
    [(32, 8, 16, 0, None, [1, 5, 128, 129, 1000, 257, 2049], [1, 1, 1, 1, 1, 1, 1]),
     (8, 2, 16, 0, 3, [700, 64, 1], [1, 1, 1]),
     (12, 3, 8, 100, None, [333, 50, 128], [1, 1, 2]),          # a window; two tokens still fit a decode tile
     (40, 2, 64, 0, 2, [400, 90], [1, 1]),                      # a group of 20 rows: two decode tiles per request
     (4, 4, 128, 0, None, [513, 127], [3, 1]),                  # pages as long as a block
     (8, 8, 256, 77, 4, [900], [5]),
     (8, 1, 16, 0, 10, [5000], [1]),                            # clusters of more than eight CTAs, and of odd sizes
     (8, 2, 16, 0, 16, [3000, 40], [1, 1]),
     (16, 4, 16, 0, 6, [2000, 700], [1, 1]),
     (8, 2, 32, 500, 5, [1500], [1])],
)
def test_attention_decode_kernels(hq, hkv, page, window, splits, lengths, new_counts, decode_kernel):
    """Decode tiles at head size 128: the tcgen05 kernel (auto; with deep rings, one CTA per multiprocessor; with
    shallow rings, two) and the mma.sync tiles give the plain result."""
    dtype, d = torch.bfloat16, 128
    case = paged_case(dtype, hq, hkv, d, page, lengths, new_counts, seed=page + hq)
    scale = d**-0.5
    got = run_mma(case, lengths, new_counts, hq, hkv, d, scale, window, splits, decode_kernel)
    want = plain_paged(case, dtype, lengths, new_counts, scale, window)
    torch.testing.assert_close(got, want, **for_dtype(dtype))


def test_attention_decode_of_more_items_than_multiprocessors():
    """Ninety requests over four kv heads are 360 CTAs: the step takes the shallow rings by itself, two CTAs per
    multiprocessor, and gives the bits of the deep rings (the same sums in the same order)."""
    dtype, d, hq, hkv, page = torch.bfloat16, 128, 8, 4, 16
    generator = torch.Generator().manual_seed(3)
    lengths = torch.randint(1, 700, (90,), generator=generator).tolist()
    new_counts = [1] * len(lengths)
    case = paged_case(dtype, hq, hkv, d, page, lengths, new_counts, seed=31)
    scale = d**-0.5
    got = {which: run_mma(case, lengths, new_counts, hq, hkv, d, scale, 0, None, which) for which in ("auto", "deep", "shallow")}
    assert torch.equal(got["auto"], got["shallow"]) and torch.equal(got["deep"], got["shallow"])
    torch.testing.assert_close(got["auto"], plain_paged(case, dtype, lengths, new_counts, scale, 0), **for_dtype(dtype))


@pytest.mark.parametrize("decode_kernel", ["auto", "mma"])
def test_attention_decode_with_more_pages_than_a_cta_keeps_in_shared_memory(decode_kernel):
    """A request of 8,300 tokens in pages of 8 has 1,038 pages: beyond the page ids a CTA copies
    into shared memory (512 and 1,024), so the kernels read the block table as they go."""
    dtype, hq, hkv, d, page = torch.bfloat16, 2, 1, 128, 8
    lengths, new_counts = [8300, 9], [1, 1]
    case = paged_case(dtype, hq, hkv, d, page, lengths, new_counts, seed=21)
    scale = d**-0.5
    got = run_mma(case, lengths, new_counts, hq, hkv, d, scale, 0, 1, decode_kernel)
    want = plain_paged(case, dtype, lengths, new_counts, scale, 0)
    torch.testing.assert_close(got, want, **for_dtype(dtype))


def test_attention_prefill_tc_with_more_pages_than_a_cta_keeps_in_shared_memory():
    dtype, hq, hkv, d, page = torch.bfloat16, 4, 1, 128, 8
    lengths, new_counts = [8300], [100]
    case = paged_case(dtype, hq, hkv, d, page, lengths, new_counts, seed=22)
    scale = d**-0.5
    got = run_mma(case, lengths, new_counts, hq, hkv, d, scale, 0, page=page)
    want = plain_paged(case, dtype, lengths, new_counts, scale, 0)
    torch.testing.assert_close(got, want, **for_dtype(dtype))


@pytest.mark.parametrize(
    "hq,hkv,page,window,lengths,new_counts",
    [(32, 8, 16, 0, [2048], [2048]),                                   # one whole prompt
     (8, 2, 16, 0, [700, 300, 64, 129, 1], [700, 150, 33, 129, 1]),     # portions at odd offsets beside a decode token
     (12, 3, 8, 100, [333, 500], [200, 37]),                            # a window, a group of four
     (6, 1, 64, 0, [900, 130], [64, 130]),                              # six heads a group: tiles straddle tokens
     (4, 4, 128, 0, [513, 260], [300, 260]),                            # one head a group, pages as long as a block
     (16, 2, 32, 300, [1500], [257])],
)
def test_attention_prefill_tc(hq, hkv, page, window, lengths, new_counts):
    """Chunk tiles of the tcgen05 kernel (head size 128) against the plain result."""
    dtype, d = torch.bfloat16, 128
    case = paged_case(dtype, hq, hkv, d, page, lengths, new_counts, seed=hq + page)
    scale = d**-0.5
    got = run_mma(case, lengths, new_counts, hq, hkv, d, scale, window, page=page)
    want = plain_paged(case, dtype, lengths, new_counts, scale, window)
    torch.testing.assert_close(got, want, **for_dtype(dtype))


def test_attention_prefill_tc_finds_a_far_key_and_respects_the_window_edge():
    dtype, hq, hkv, d, page = torch.bfloat16, 4, 2, 128, 16
    length, far, new = 700, 13, 300
    case = paged_case(dtype, hq, hkv, d, page, [length], [new], seed=3)
    query = case["queries"][0][-1]
    for head in range(hkv):
        case["keys"][0][far, head] = 40.0 * query[head * (hq // hkv)] / query[head * (hq // hkv)].norm()
    page_id = int(case["table"][case["slots"][0], far // page])
    case["cache"][page_id, 0, :, far % page] = case["keys"][0][far].to(dtype)
    scale = d**-0.5
    for window, expect_far in [(0, True), (length - far, True), (length - far - 1, False)]:
        got = run_mma(case, [length], [new], hq, hkv, d, scale, window, page=page)
        want = plain_paged(case, dtype, [length], [new], scale, window)
        torch.testing.assert_close(got, want, **for_dtype(dtype))
        value = case["values"][0][far, 0].to(dtype).float()
        close = (got[-1, 0] - value).abs().max() < 0.15
        assert bool(close) == expect_far


def test_attention_mma_decode_only_step_splits_by_entry_count():
    dtype, hq, hkv, d, page = torch.bfloat16, 8, 2, 128, 16
    lengths, new_counts = [5, 1000, 64, 257], [1, 1, 1, 1]
    case = paged_case(dtype, hq, hkv, d, page, lengths, new_counts, seed=1)
    got = run_mma(case, lengths, new_counts, hq, hkv, d, d**-0.5, 0)      # planner: 16 splits, most of them empty
    want = plain_paged(case, dtype, lengths, new_counts, d**-0.5, 0)
    torch.testing.assert_close(got, want, **for_dtype(dtype))


def test_attention_mma_finds_a_far_key_and_respects_the_window_edge():
    dtype, hq, hkv, d, page = torch.bfloat16, 4, 2, 64, 16
    length, far = 700, 13
    for new in (1, 40):
        case = paged_case(dtype, hq, hkv, d, page, [length], [new], seed=3)
        query = case["queries"][0][-1]
        for head in range(hkv):
            case["keys"][0][far, head] = 40.0 * query[head * (hq // hkv)] / query[head * (hq // hkv)].norm()
        page_id = int(case["table"][case["slots"][0], far // page])
        case["cache"][page_id, 0, :, far % page] = case["keys"][0][far].to(dtype)
        scale = d**-0.5
        for window, expect_far in [(0, True), (length - far, True), (length - far - 1, False)]:
            for splits in (None, 4):
                got = run_mma(case, [length], [new], hq, hkv, d, scale, window, splits)
                want = plain_paged(case, dtype, [length], [new], scale, window)
                torch.testing.assert_close(got, want, **for_dtype(dtype))
                value = case["values"][0][far, 0].to(dtype).float()
                close = (got[-1, 0] - value).abs().max() < 0.15
                assert bool(close) == expect_far


# -------------------------------------------------------------------- sampling
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab", [331, 8193, 151936])
def test_greedy_is_first_maximum(dtype, vocab):
    rows = 5
    logits = rand((rows, vocab), dtype, seed=11).to(DEV)
    logits[1, 7] = logits[1].max() + 1
    logits[2, vocab - 1] = logits[2].max() + 2
    logits[3, 100] = logits[3, 200] = logits[3].max() + 3   # a tie: the first index wins
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    k().sample(logits, out)
    assert out.tolist() == torch.argmax(logits.float(), dim=-1).tolist()
    assert out[3].item() == 100


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab", [1237, 151936, 400003])      # a small row; the model's; more than a cluster keeps in shared memory
def test_sampling_matches_plain(dtype, vocab):
    rows = 24
    logits = rand((rows, vocab), dtype, scale=2.0, seed=12).to(DEV)
    temperature = torch.tensor([0.0, 0.7, 1.0, 1.3] * 6, dtype=torch.float32)
    top_p = torch.tensor([1.0, 0.9, 0.5, 1.0, 0.3, 0.95] * 4, dtype=torch.float32)
    penalty = torch.tensor([1.0, 1.1, 1.0, 2.0] * 6, dtype=torch.float32)
    seeds = torch.arange(rows, dtype=torch.int64) * 7919 + 5
    counters = torch.arange(rows, dtype=torch.int32) + 3
    generated = [torch.randint(0, vocab, (row % 5 * 9,)).tolist() for row in range(rows)]
    offsets = torch.tensor([0] + [len(g) for g in generated], dtype=torch.int32).cumsum(0).to(torch.int32)
    flat = torch.tensor([t for g in generated for t in g] or [0], dtype=torch.int32)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    k().sample(
        logits, out, temperature=temperature.to(DEV), top_p=top_p.to(DEV), penalty=penalty.to(DEV),
        seeds=seeds.to(DEV), counters=counters.to(DEV), seen_tokens=flat.to(DEV), seen_offsets=offsets.to(DEV),
    )
    host = logits.float().cpu()
    want = [
        sample_token(host[row], float(temperature[row]), float(top_p[row]), float(penalty[row]),
                     generated[row], int(seeds[row]), int(counters[row]))
        for row in range(rows)
    ]
    agree = sum(int(a == b) for a, b in zip(out.tolist(), want))
    assert agree >= rows - 1, (out.tolist(), want)   # a draw on a float32 rounding edge may differ


def test_sampling_follows_the_distribution():
    vocab, rows = 50, 4000
    base = torch.linspace(-2, 2, vocab)
    logits = base.repeat(rows, 1).to(DEV)
    temperature = torch.full((rows,), 0.8)
    seeds = torch.full((rows,), 1234, dtype=torch.int64)
    counters = torch.arange(rows, dtype=torch.int32)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    k().sample(logits, out, temperature=temperature.to(DEV), seeds=seeds.to(DEV), counters=counters.to(DEV))
    counts = torch.bincount(out.long().cpu(), minlength=vocab).float() / rows
    want = torch.softmax(base / 0.8, 0)
    assert (counts - want).abs().max() < 0.02
    again = torch.empty_like(out)
    k().sample(logits, again, temperature=temperature.to(DEV), seeds=seeds.to(DEV), counters=counters.to(DEV))
    assert torch.equal(out, again)


def test_kernels_refuse_what_they_cannot_do():
    kernels = k()
    with pytest.raises(kernels.KernelError):
        kernels.attention_generic(
            torch.zeros((1, 24), device=DEV), torch.zeros((2, 2, 1, 4, 24), device=DEV), torch.zeros((1, 24), device=DEV),
            positions=torch.zeros(1, dtype=torch.int32, device=DEV), token_slot=torch.zeros(1, dtype=torch.int32, device=DEV),
            block_table=torch.zeros((1, 1), dtype=torch.int32, device=DEV), num_heads=1, num_kv_heads=1, head_dim=24,
            window=0, scale=1.0, fault=fault_word(),
        )
    with pytest.raises(kernels.KernelError):
        kernels.silu_mul(torch.zeros((2, 8)), torch.zeros((2, 4)))   # CPU tensors: no CPU path
