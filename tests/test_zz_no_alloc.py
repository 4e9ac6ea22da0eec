"""The allocation-free attention entry point, called through its exported C symbol.

``rl_attention_mma_static_scratch`` is for callers that must not create device memory while
they run (a plug-in in a process with a frozen memory pool, a real-time loop, a C host
without an allocator).  It keeps the scratch of the split key ranges in an array inside the
library instead of asking the caller for two buffers.  Here it is called twice in a row on
different inputs (the array keeps the first call's contents, so the second call shows
whether stale values leak) and compared with the ordinary entry point, which gets fresh
buffers from PyTorch; a request beyond the array must be refused without a launch.

The file's name makes pytest collect it last: should it fail, a run that stops at the first
failure has already run every other test.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import numpy as np
import pytest
import torch
from test_kernels_gpu import DEV, fault_word, paged_case, plain_paged, run_mma
from tolerances import for_dtype

pytestmark = pytest.mark.gpu
TOO_LARGE = -2


def static_scratch_entry(head_dim: int):
    """The library's C symbols, declared by hand as a C caller would."""
    from rapid_llm_b200.ops import kernels

    lib = kernels.attention_lib(head_dim)
    entry = lib.rl_attention_mma_static_scratch
    entry.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                      c_void_p, c_void_p] + [c_int] * 10 + [c_float, c_void_p, c_void_p]
    entry.restype = c_int
    lib.rl_attention_static_scratch_bytes.restype = ctypes.c_longlong
    lib.rl_attention_static_scratch_strerror.argtypes = [c_int]
    lib.rl_attention_static_scratch_strerror.restype = ctypes.c_char_p
    return lib, entry


def call_static(entry, case, lengths, new_counts, hq, hkv, d, scale, window, splits):
    from rapid_llm_b200.parts.attention import AttentionItems
    from rapid_llm_b200.parts.base import StepShape

    starts = [length - new for length, new in zip(lengths, new_counts)]
    plan = AttentionItems(hq // hkv, hkv).plan(
        StepShape(np.asarray(new_counts, dtype=np.int32), np.asarray(starts, dtype=np.int32), decode_only=max(new_counts) == 1)
    )

    def spread(items):
        base = items[items[:, 2] == 0]
        out = np.repeat(base, splits, axis=0)
        out[:, 2] = np.tile(np.arange(splits, dtype=np.int32), len(base))
        return torch.from_numpy(np.ascontiguousarray(out)).to(DEV)

    chunk, decode = spread(plan["chunk_items"]), spread(plan["decode_items"])
    q = case["q"].to(DEV).reshape(-1, hq * d).contiguous()
    out = torch.full_like(q, float("nan"))
    cache, table = case["cache"].to(DEV), case["table"].to(DEV)
    cu = torch.tensor([0] + list(np.cumsum(new_counts)), dtype=torch.int32, device=DEV)
    entry_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    entry_slot = torch.tensor(case["slots"], dtype=torch.int32, device=DEV)
    fault = fault_word()
    ptr = lambda t: c_void_p(t.data_ptr() if t.numel() else 0)  # noqa: E731
    code = entry(
        ptr(q), ptr(cache), ptr(out), ptr(chunk), chunk.shape[0], ptr(decode), decode.shape[0], ptr(cu),
        ptr(entry_start), ptr(entry_slot), ptr(table), q.shape[0], hq, hkv, d, cache.shape[3], cache.shape[0],
        table.shape[1], table.shape[0], window, splits, scale, ptr(fault),
        c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    torch.cuda.synchronize()
    return code, out.float().cpu().view(q.shape[0], hq, d), int(fault.item())


def test_static_scratch_entry_matches_the_ordinary_one_twice_in_a_row():
    dtype, hq, hkv, d, page = torch.bfloat16, 8, 2, 128, 16
    lib, entry = static_scratch_entry(d)
    assert lib.rl_attention_static_scratch_bytes() == 4 << 20
    scale = d**-0.5
    runs = [
        ([1, 15, 129, 200, 700, 333], [1, 15, 40, 1, 1, 70], 3, 0, 5),
        ([900, 64, 257, 31], [1, 1, 1, 1], 4, 300, 6),       # decode only, other sizes, a window
    ]
    for index, (lengths, new_counts, splits, window, seed) in enumerate(runs):
        case = paged_case(dtype, hq, hkv, d, page, lengths, new_counts, seed=seed)
        if index == 1:
            # what the array holds from before is not always finite: a call on cached values that are not
            # numbers leaves NaN in every part it writes, and the next call must not pick any of it up
            first = runs[0]
            poisoned = paged_case(dtype, hq, hkv, d, page, first[0], first[1], seed=first[4])
            poisoned["cache"][:, 1] = float("nan")
            code, got, _ = call_static(entry, poisoned, first[0], first[1], hq, hkv, d, scale, first[3], first[2])
            assert code == 0 and torch.isnan(got).any()
        code, got, fault = call_static(entry, case, lengths, new_counts, hq, hkv, d, scale, window, splits)
        assert code == 0, lib.rl_attention_static_scratch_strerror(code).decode()
        assert fault == 0
        ordinary = run_mma(case, lengths, new_counts, hq, hkv, d, scale, window, splits)
        torch.testing.assert_close(got, ordinary, **for_dtype(dtype))
        torch.testing.assert_close(got, plain_paged(case, dtype, lengths, new_counts, scale, window), **for_dtype(dtype))


def test_static_scratch_entry_refuses_what_does_not_fit():
    dtype, hq, hkv, d, page = torch.bfloat16, 32, 8, 128, 16
    lib, entry = static_scratch_entry(d)
    lengths, new_counts = [300], [300]
    splits = 2                         # 300 tokens * 32 heads * 2 splits * 129 floats > 4 MiB
    assert 300 * hq * splits * (d + 1) * 4 > lib.rl_attention_static_scratch_bytes()
    case = paged_case(dtype, hq, hkv, d, page, lengths, new_counts, seed=7)
    code, got, fault = call_static(entry, case, lengths, new_counts, hq, hkv, d, d**-0.5, 0, splits)
    assert code == TOO_LARGE
    assert b"exceed" in lib.rl_attention_static_scratch_strerror(code)
    assert torch.isnan(got).all() and fault == 0      # nothing was launched
