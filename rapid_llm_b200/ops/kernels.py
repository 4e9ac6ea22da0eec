"""Python entry points of the CUDA kernels: tensors in, launches on the current stream.

Each function checks shapes, dtypes and devices, then calls the ``extern "C"`` launcher
with raw pointers.  Nothing here has a CPU or library fallback: a tensor that is not on a
CUDA device, or an extension that cannot be built, raises.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import attention_library, load_library

F32, BF16 = 0, 1

# Launch every kernel of this library as a programmatic dependent of the stream's previous
# kernel: it may then start while that kernel drains, and waits inside for its results.  The
# engine switches it on for its steps; direct callers get ordinary launches.
PDL = False

FAULT_BITS = {
    1: "a token id outside the vocabulary",
    2: "a page id outside the cache pool",
    4: "a position outside the rotary table or block table",
    8: "a slot outside the block table",
    16: "a bounded wait inside a kernel ran out",
}


class KernelError(RuntimeError):
    """A launch was refused (bad size or argument) or failed."""


def dtype_tag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


def _ptr(tensor: torch.Tensor | None) -> int | None:
    """The address as ctypes takes it for a ``c_void_p`` parameter (a plain integer, ``None`` for null): every
    launcher's signature is declared, so no wrapper object is needed, and a step passes thousands of these."""
    return None if tensor is None else tensor.data_ptr()


# Called before every launch of this module: whoever has queued work that the launch may depend on
# (``ops.gemm`` queues the products of a small step for one persistent kernel) runs it first.
BEFORE_LAUNCH = None


def _stream() -> int:
    """The current stream of the current device as a raw handle (asked of torch's C layer directly: the Stream
    object of ``torch.cuda.current_stream()`` costs several microseconds, and every launch asks)."""
    if BEFORE_LAUNCH is not None:
        BEFORE_LAUNCH()
    return _raw_stream(torch.cuda.current_device())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) or (lambda device: torch.cuda.current_stream(device).cuda_stream)


def _need_cuda(*tensors: torch.Tensor | None) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError(
                "kernel arguments must live on a CUDA device; there is no CPU path "
                f"(got a tensor on {tensor.device})"
            )


def _contig(name: str, tensor: torch.Tensor | None) -> None:
    if tensor is not None and not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _expect(name: str, tensor: torch.Tensor | None, dtype: torch.dtype) -> None:
    if tensor is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")


_CUDA_ERRORS = {1: "invalid value (a size or argument the kernel refuses)"}


class LaunchCounter:
    """Counts launches of this library's kernels (library products are not counted).

    A captured graph's launches are added by whoever replays it (``add``)."""

    def __init__(self) -> None:
        self.count = 0

    def add(self, launches: int) -> None:
        self.count += launches


LAUNCHES = LaunchCounter()


def _check(code: int, what: str) -> None:
    LAUNCHES.count += 1
    if code != 0:
        detail = _CUDA_ERRORS.get(code, f"CUDA error {code}")
        raise KernelError(f"{what}: {detail}")


_SIGNATURES_SET = False


def core() -> ctypes.CDLL:
    """The core kernel library, with argument types declared once."""
    global _SIGNATURES_SET
    lib = load_library("core")
    if not _SIGNATURES_SET:
        lib.rl_embedding.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
        lib.rl_add_rmsnorm.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p]
        lib.rl_silu_mul.argtypes = [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.rl_scatter_rows.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        lib.rl_to_float.argtypes = [c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p]
        lib.rl_qk_norm_rope_write.argtypes = [
            c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
            c_float, c_void_p, c_int, c_void_p,
        ]
        lib.rl_attention_generic.argtypes = [
            c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
            c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
        ]
        lib.rl_gemm_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.rl_sample.argtypes = [
            c_int, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
        ]
        for name in (
            "rl_embedding", "rl_scatter_rows", "rl_add_rmsnorm", "rl_silu_mul", "rl_to_float",
            "rl_qk_norm_rope_write", "rl_attention_generic", "rl_gemm_f32", "rl_sample",
        ):
            getattr(lib, name).restype = c_int
        _SIGNATURES_SET = True
    return lib


# --------------------------------------------------------------------------- ops
def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, fault: torch.Tensor,
              feedback: torch.Tensor | None = None) -> torch.Tensor:
    """``out[t] = table[ids[t]]``; ``ids`` int32 ``[T]``; bad ids set the fault word.

    With ``feedback`` (int32, on the device) an id ``-(r + 1)`` is replaced by ``feedback[r]``."""
    _need_cuda(out, table, ids, fault, feedback)
    _expect("ids", ids, torch.int32), _expect("feedback", feedback, torch.int32)
    _contig("out", out), _contig("table", table), _contig("ids", ids)
    if out.dtype != table.dtype or out.shape != (ids.numel(), table.shape[1]):
        raise KernelError(f"embedding: out {tuple(out.shape)} {out.dtype} does not fit table {tuple(table.shape)} {table.dtype}")
    _check(
        core().rl_embedding(dtype_tag(table.dtype), _ptr(out), _ptr(table), _ptr(ids), _ptr(feedback),
                            0 if feedback is None else feedback.numel(), ids.numel(),
                            table.shape[1], table.shape[0], _ptr(fault), 0, _stream()),   # first kernel of a step: an ordinary launch
        "embedding",
    )
    return out


def scatter_rows(table: torch.Tensor, slots: torch.Tensor, rows: torch.Tensor, fault: torch.Tensor) -> torch.Tensor:
    """``table[slots[i]] = rows[i]`` for int32 tables; a slot outside the table sets the fault word."""
    _need_cuda(table, slots, rows, fault)
    for name, tensor in (("table", table), ("slots", slots), ("rows", rows)):
        _expect(name, tensor, torch.int32), _contig(name, tensor)
    if table.dim() != 2 or rows.numel() != slots.numel() * table.shape[1]:
        raise KernelError("scatter_rows: rows must hold one table row per slot")
    _check(
        core().rl_scatter_rows(_ptr(table), table.shape[1], table.shape[0], _ptr(slots), _ptr(rows), slots.numel(),
                               _ptr(fault), _stream()),
        "scatter_rows",
    )
    return table


def add_rmsnorm(
    x: torch.Tensor,
    residual: torch.Tensor | None,
    weight: torch.Tensor,
    out: torch.Tensor,
    eps: float,
    *,
    mode: int,
    write_residual: bool,
    row_index: torch.Tensor | None = None,
) -> torch.Tensor:
    """RMSNorm of ``x`` (mode 0 or 2) or of ``x + residual`` (mode 1), float32 math.

    ``residual`` is the float32 residual stream ``[T, H]``; with ``write_residual`` the
    sum is stored back into it.  ``row_index`` (int32) selects the input rows; ``out`` then
    has one row per index.
    """
    _need_cuda(x, residual, weight, out, row_index)
    _expect("weight", weight, torch.float32), _expect("residual", residual, torch.float32)
    _expect("row_index", row_index, torch.int32)
    _contig("x", x), _contig("residual", residual), _contig("out", out)
    hidden = x.shape[-1]
    rows = row_index.numel() if row_index is not None else x.shape[0]
    if weight.numel() != hidden or out.shape != (rows, hidden) or out.dtype != x.dtype:
        raise KernelError("add_rmsnorm: shapes of x, weight and out do not agree")
    if residual is not None and residual.shape != x.shape:
        raise KernelError("add_rmsnorm: residual must have the shape of x")
    _check(
        core().rl_add_rmsnorm(dtype_tag(x.dtype), _ptr(x), _ptr(residual), _ptr(weight), _ptr(out),
                              _ptr(row_index), rows, hidden, float(eps), mode, int(write_residual), int(PDL), _stream()),
        f"add_rmsnorm(hidden={hidden})",
    )
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = silu(gate_up[:, :I]) * gate_up[:, I:]``."""
    _need_cuda(gate_up, out)
    _contig("gate_up", gate_up), _contig("out", out)
    rows, width = gate_up.shape
    if width % 2 or out.shape != (rows, width // 2) or out.dtype != gate_up.dtype:
        raise KernelError("silu_mul: out must be [rows, width / 2] of the input's dtype")
    _check(core().rl_silu_mul(dtype_tag(gate_up.dtype), _ptr(gate_up), _ptr(out), rows, width // 2, int(PDL), _stream()), "silu_mul")
    return out


def to_float(src: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need_cuda(src, out)
    _contig("src", src), _contig("out", out)
    _expect("out", out, torch.float32)
    if out.numel() != src.numel():
        raise KernelError("to_float: sizes differ")
    _check(core().rl_to_float(dtype_tag(src.dtype), _ptr(src), _ptr(out), src.numel(), int(PDL), _stream()), "to_float")
    return out


def qk_norm_rope_write(
    qkv: torch.Tensor,
    q_out: torch.Tensor,
    *,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    rotary_dim: int,
    cos: torch.Tensor,
    sin: torch.Tensor,
    positions: torch.Tensor,
    eps: float,
    fault: torch.Tensor,
    q_weight: torch.Tensor | None = None,
    k_weight: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
    kv_dest: torch.Tensor | None = None,
    cache: torch.Tensor | None = None,
    page_size: int = 1,
) -> torch.Tensor:
    """Per-head q/k RMSNorm, rotation by position, q to ``q_out``, k and v into the pages.

    ``qkv`` is ``[T, (Hq + 2 Hkv) D]`` (or ``[T, Hq D]`` when ``kv_dest`` is ``None`` and
    only queries are produced).  ``cache`` is one layer's ``[pages, 2, Hkv, page, D]``;
    ``kv_dest[t] = page * page_size + offset``.
    """
    _need_cuda(qkv, q_out, cos, sin, positions, fault, q_weight, k_weight, bias, kv_dest, cache)
    _contig("qkv", qkv), _contig("q_out", q_out), _contig("cache", cache)
    _contig("cos", cos), _contig("sin", sin)
    for name, tensor in (("cos", cos), ("sin", sin), ("q_weight", q_weight), ("k_weight", k_weight), ("bias", bias)):
        _expect(name, tensor, torch.float32)
    _expect("positions", positions, torch.int32), _expect("kv_dest", kv_dest, torch.int32)
    tokens, row_width = qkv.shape
    heads_in = num_heads + 2 * num_kv_heads if kv_dest is not None else num_heads
    if row_width != heads_in * head_dim:
        raise KernelError(f"qk_norm_rope_write: qkv width {row_width} is not {heads_in} heads of {head_dim}")
    if q_out.numel() != tokens * num_heads * head_dim or q_out.dtype != qkv.dtype:
        raise KernelError("qk_norm_rope_write: q_out does not fit")
    if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] * 2 != rotary_dim:
        raise KernelError("qk_norm_rope_write: cos/sin must be [positions, rotary_dim / 2]")
    num_pages = 0
    if kv_dest is not None:
        if cache is None or cache.dtype != qkv.dtype or cache.shape[1:] != (2, num_kv_heads, page_size, head_dim):
            raise KernelError("qk_norm_rope_write: cache must be [pages, 2, kv_heads, page_size, head_dim] of qkv's dtype")
        num_pages = cache.shape[0]
    _check(
        core().rl_qk_norm_rope_write(
            dtype_tag(qkv.dtype), _ptr(qkv), row_width, _ptr(bias), _ptr(q_weight), _ptr(k_weight),
            _ptr(cos), _ptr(sin), _ptr(positions), _ptr(kv_dest), _ptr(q_out), _ptr(cache), tokens,
            num_heads, num_kv_heads, head_dim, rotary_dim, cos.shape[0], page_size, num_pages,
            float(eps), _ptr(fault), int(PDL), _stream(),
        ),
        f"qk_norm_rope_write(head_dim={head_dim})",
    )
    return q_out


def attention_generic(
    q: torch.Tensor,
    cache: torch.Tensor,
    out: torch.Tensor,
    *,
    positions: torch.Tensor,
    token_slot: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    window: int,
    scale: float,
    fault: torch.Tensor,
) -> torch.Tensor:
    """Causal attention of every token of the step over its request's cached keys."""
    _need_cuda(q, cache, out, positions, token_slot, block_table, fault)
    _contig("q", q), _contig("cache", cache), _contig("out", out), _contig("block_table", block_table)
    for name, tensor in (("positions", positions), ("token_slot", token_slot), ("block_table", block_table)):
        _expect(name, tensor, torch.int32)
    tokens = positions.numel()
    if q.numel() != tokens * num_heads * head_dim or out.numel() != q.numel():
        raise KernelError("attention: q/out do not hold [tokens, heads, head_dim]")
    if cache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, cache and out must share a dtype")
    if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
        raise KernelError("attention: cache must be [pages, 2, kv_heads, page_size, head_dim]")
    if head_dim % 16 or head_dim > 256:
        raise KernelError(f"attention: head_dim {head_dim} must be a multiple of 16 up to 256")
    _check(
        core().rl_attention_generic(
            dtype_tag(q.dtype), _ptr(q), _ptr(cache), _ptr(out), _ptr(positions), _ptr(token_slot),
            _ptr(block_table), tokens, num_heads, num_kv_heads, head_dim, cache.shape[3],
            cache.shape[0], block_table.shape[1], block_table.shape[0], int(window), float(scale),
            _ptr(fault), _stream(),
        ),
        f"attention_generic(head_dim={head_dim})",
    )
    return out


_ATTENTION_LIBS: dict[int, ctypes.CDLL] = {}

CHUNK_TILE_ROWS = 64       # packed rows (token, head of the group) of a chunk tile of the mma.sync kernel
CHUNK_TILE_ROWS_TC = 256   # ... of the tcgen05 kernel (head size 128, unsplit key ranges)
DECODE_TILE_ROWS = 16      # ... of a decode tile
TC_HEAD_DIM = 128
DECODE_TC_KEYS = 128      # keys per block of the tcgen05 decode kernel


def attention_tc_takes(head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 attention kernels take this head size and page size."""
    if head_dim != TC_HEAD_DIM or page_size <= 0 or page_size % 8:
        return False
    return 128 % page_size == 0 or page_size % 128 == 0


def attention_lib(head_dim: int) -> ctypes.CDLL:
    """The tensor-core attention library of one head size, built at its first use."""
    lib = _ATTENTION_LIBS.get(head_dim)
    if lib is None:
        lib = load_library(attention_library(head_dim))
        lib.rl_attention_mma.argtypes = [
            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
            c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
        ]
        lib.rl_attention_mma.restype = c_int
        lib.rl_attention_decode_max_clusters.argtypes = [c_int]
        lib.rl_attention_decode_max_clusters.restype = c_int
        if lib.rl_attention_head_dim() != head_dim:
            raise KernelError(f"the attention library for head size {head_dim} was built for another size")
        if lib.rl_attention_chunk_rows() != CHUNK_TILE_ROWS or lib.rl_attention_decode_rows() != DECODE_TILE_ROWS:
            raise KernelError("the attention library's tile sizes differ from the host's")
        if lib.rl_attention_chunk_rows_tc() != (CHUNK_TILE_ROWS_TC if head_dim == TC_HEAD_DIM else 0):
            raise KernelError("the attention library's tensor-core tile size differs from the host's")
        _ATTENTION_LIBS[head_dim] = lib
    return lib


def attention_decode_clusters(head_dim: int, device: torch.device) -> dict[int, int]:
    """``{cluster size: clusters of the tcgen05 decode kernel the GPU runs at one time}`` for the sizes it can
    launch (a cluster lives inside one GPC, so this is not the number of multiprocessors over the size).
    Empty where that kernel does not exist (other head sizes)."""
    if head_dim != TC_HEAD_DIM:
        return {}
    lib = attention_lib(head_dim)
    table = {}
    with torch.cuda.device(device):
        for size in range(1, 17):
            count = int(lib.rl_attention_decode_max_clusters(size))
            if count > 0:
                table[size] = count
    return table


def attention_mma(
    q: torch.Tensor,
    cache: torch.Tensor,
    out: torch.Tensor,
    *,
    chunk_items: torch.Tensor | None,
    decode_items: torch.Tensor | None,
    splits: int,
    part_out: torch.Tensor | None,
    part_lse: torch.Tensor | None,
    cu_seqlens: torch.Tensor,
    entry_start: torch.Tensor,
    entry_slot: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    window: int,
    scale: float,
    fault: torch.Tensor,
    decode_kernel: str = "auto",
    decode_rows: int = 0,
    chunk_rows: int = CHUNK_TILE_ROWS,
    decode_splits: int = 0,
) -> torch.Tensor:
    """bfloat16 paged causal attention over work items the host cut the step into.

    Decode tiles run on the tcgen05 kernel where it applies (head size 128, pages of 8 to 64 or
    a multiple of 128 tokens) unless ``decode_kernel`` is ``"mma"``; ``decode_rows`` is the most
    packed rows any decode tile has (0 = not known), which lets that kernel unroll over fewer rows.
    ``chunk_rows`` says how the chunk items were cut: :data:`CHUNK_TILE_ROWS` for the mma.sync
    tiles, :data:`CHUNK_TILE_ROWS_TC` for the tcgen05 kernel (``splits`` must then be 1).

    ``chunk_items`` / ``decode_items`` are int32 ``[n, 4]`` rows ``(entry, first packed row,
    split, 0)`` for tiles of :data:`CHUNK_TILE_ROWS` / :data:`DECODE_TILE_ROWS` packed rows
    (row ``p`` of an entry is token ``p // group``, head ``p % group`` of each kv head).
    With ``splits > 1`` every item exists once per split and ``part_out`` ``[T * Hq * splits,
    D]`` / ``part_lse`` ``[T * Hq * splits]`` (float32) are scratch.  ``decode_splits`` (0 = as ``splits``) gives
    the decode items a split count of their own, merged inside the tcgen05 decode kernel's clusters: only with
    ``splits == 1``, where that kernel applies, up to 16.
    """
    _need_cuda(q, cache, out, chunk_items, decode_items, part_out, part_lse, cu_seqlens, entry_start,
               entry_slot, block_table, fault)
    for name, tensor in (("q", q), ("cache", cache), ("out", out)):
        _expect(name, tensor, torch.bfloat16), _contig(name, tensor)
    for name, tensor in (("chunk_items", chunk_items), ("decode_items", decode_items), ("cu_seqlens", cu_seqlens),
                         ("entry_start", entry_start), ("entry_slot", entry_slot), ("block_table", block_table)):
        _expect(name, tensor, torch.int32), _contig(name, tensor)
    _expect("part_out", part_out, torch.float32), _expect("part_lse", part_lse, torch.float32)
    width = num_heads * head_dim
    if q.dim() != 2 or q.shape[1] != width or out.shape != q.shape:
        raise KernelError("attention: q and out must be [tokens, heads * head_dim]")
    tokens = q.shape[0]
    if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
        raise KernelError("attention: cache must be [pages, 2, kv_heads, page_size, head_dim]")
    if num_heads % num_kv_heads:
        raise KernelError("attention: heads must be a multiple of kv heads")
    n_chunk = 0 if chunk_items is None else chunk_items.shape[0]
    n_decode = 0 if decode_items is None else decode_items.shape[0]
    if splits > 1:
        need = tokens * num_heads * splits
        if part_out is None or part_lse is None or part_out.numel() < need * head_dim or part_lse.numel() < need:
            raise KernelError("attention: scratch for the split key ranges is missing or too small")
    _check(
        attention_lib(head_dim).rl_attention_mma(
            _ptr(q), _ptr(cache), _ptr(out), _ptr(part_out), _ptr(part_lse), _ptr(chunk_items), n_chunk,
            _ptr(decode_items), n_decode, _ptr(cu_seqlens), _ptr(entry_start), _ptr(entry_slot),
            _ptr(block_table), tokens, num_heads, num_kv_heads, head_dim, cache.shape[3], cache.shape[0],
            block_table.shape[1], block_table.shape[0], int(window), int(splits), float(scale),
            _ptr(fault), int(PDL), {"auto": 0, "mma": 1, "deep": 2, "shallow": 3}[decode_kernel], int(decode_rows), int(chunk_rows),
            int(decode_splits), _stream(),
        ),
        f"attention_mma(head_dim={head_dim})",
    )
    LAUNCHES.count += (1 if n_chunk and n_decode else 0) + (1 if splits > 1 else 0)
    return out


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``out[M, N] = a[M, K] @ w[N, K]^T`` in true float32."""
    _need_cuda(a, w, out, bias)
    for name, tensor in (("a", a), ("w", w), ("out", out), ("bias", bias)):
        _expect(name, tensor, torch.float32)
    _contig("w", w)
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1] or out.shape != (a.shape[0], w.shape[0]):
        raise KernelError(f"gemm_f32: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
    if a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_f32: rows of a and out must be contiguous")
    _check(
        core().rl_gemm_f32(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), a.shape[0], w.shape[0], a.shape[1],
                           a.stride(0), out.stride(0), _stream()),
        "gemm_f32",
    )
    return out


_GEMM_LIB: ctypes.CDLL | None = None


def gemm_lib() -> ctypes.CDLL:
    global _GEMM_LIB
    if _GEMM_LIB is None:
        lib = load_library("gemm")
        lib.rl_gemm_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_void_p, c_void_p]
        lib.rl_gemm_bf16.restype = c_int
        lib.rl_gemm_bf16_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_void_p, c_void_p, c_void_p, c_void_p, c_int, ctypes.c_float, c_int,
                                          c_void_p, c_void_p, c_void_p]
        lib.rl_gemm_bf16_norm.restype = c_int
        lib.rl_gemm_bf16_sumsq_count.argtypes = [c_int]
        lib.rl_gemm_bf16_sumsq_count.restype = c_int
        _GEMM_LIB = lib
    return _GEMM_LIB


def gemm_bf16_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core product takes these operands (TMA wants 16-byte rows)."""
    return x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


GEMM_NORM_MAX_TOKENS = 64   # most rows of a product that carries a norm's add or a norm's open scale


def gemm_bf16_sumsq_count(n_out: int) -> int:
    """Columns of the table of partial sums of squares that a product of ``n_out`` columns writes."""
    return int(gemm_lib().rl_gemm_bf16_sumsq_count(int(n_out)))


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, fault: torch.Tensor, *, swiglu: bool = False,
              k_split: int = 0, residual: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None,
              sumsq_out: torch.Tensor | None = None, sumsq_in: torch.Tensor | None = None,
              norm_eps: float = 0.0, norm_size: int = 0, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``out[T, N] = x[T, K] @ w[N, K]^T`` in bfloat16 on the tcgen05 tensor cores.

    With ``swiglu``, ``w`` is ``[2 N, K]`` (gate rows, then up rows) and
    ``out = silu(x @ gate^T) * (x @ up^T)`` without the ``[T, 2 N]`` intermediate.
    ``k_split`` forces how many CTAs share a tile's inner range (0 = the kernel chooses).

    A norm between two products rides on them (at most :data:`GEMM_NORM_MAX_TOKENS` rows).
    With ``residual`` (float32 ``[T, N]``), ``norm_weight`` (float32 ``[N]``) and ``sumsq_out``
    (float32 ``[T, gemm_bf16_sumsq_count(N)]``) the product is added to ``residual`` in place,
    ``out = residual * norm_weight`` and ``sumsq_out`` receives partial sums of the new
    residual's squares.  With ``sumsq_in`` (such a table), ``norm_eps`` and ``norm_size``, row
    ``t`` of the product is multiplied by ``rsqrt(sum(sumsq_in[t]) / norm_size + norm_eps)``
    (before the SiLU): the scale that the norm before ``x`` left open.  ``bias`` (float32 ``[N]``, with
    ``swiglu`` ``[2 N]``) is added to every row after that scale.
    """
    _need_cuda(x, w, out, fault, residual, norm_weight, sumsq_out, sumsq_in, bias)
    if bias is not None:
        _expect("bias", bias, torch.float32), _contig("bias", bias)
        if bias.shape != (w.shape[0],):
            raise KernelError(f"gemm_bf16: bias of shape {tuple(bias.shape)} for a weight of {w.shape[0]} rows")
    for name, tensor in (("x", x), ("w", w), ("out", out)):
        _expect(name, tensor, torch.bfloat16), _contig(name, tensor)
    tokens, k = x.shape
    n_out = out.shape[1]
    if w.shape != ((2 if swiglu else 1) * n_out, k) or out.shape[0] != tokens:
        raise KernelError(f"gemm_bf16: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
    if not gemm_bf16_supports(x, w):
        raise KernelError("gemm_bf16: the inner size must be a multiple of 8 and the operands 16-byte aligned")
    norm_follows = residual is not None or norm_weight is not None or sumsq_out is not None
    if norm_follows:
        if residual is None or norm_weight is None or sumsq_out is None or swiglu:
            raise KernelError("gemm_bf16: a following norm needs residual, norm_weight and sumsq_out, and no swiglu")
        for name, tensor in (("residual", residual), ("norm_weight", norm_weight), ("sumsq_out", sumsq_out)):
            _expect(name, tensor, torch.float32), _contig(name, tensor)
        if (residual.shape != (tokens, n_out) or norm_weight.shape != (n_out,)
                or sumsq_out.shape != (tokens, gemm_bf16_sumsq_count(n_out))):
            raise KernelError("gemm_bf16: residual, norm_weight or sumsq_out do not have the product's shape")
    if sumsq_in is not None:
        _expect("sumsq_in", sumsq_in, torch.float32), _contig("sumsq_in", sumsq_in)
        if sumsq_in.dim() != 2 or sumsq_in.shape[0] != tokens or sumsq_in.shape[1] % 4 or norm_size <= 0:
            raise KernelError("gemm_bf16: sumsq_in must be [tokens, a multiple of 4] and norm_size positive")
    if (norm_follows or sumsq_in is not None) and tokens > GEMM_NORM_MAX_TOKENS:
        raise KernelError(f"gemm_bf16: a norm rides on products of at most {GEMM_NORM_MAX_TOKENS} rows, got {tokens}")
    if tokens == 0:
        return out
    _check(
        gemm_lib().rl_gemm_bf16_norm(
            _ptr(x), _ptr(w), _ptr(out), tokens, n_out, k, int(swiglu), int(PDL), int(k_split),
            _ptr(residual), _ptr(norm_weight), _ptr(sumsq_out),
            _ptr(sumsq_in), 0 if sumsq_in is None else sumsq_in.shape[1], float(norm_eps), int(norm_size),
            _ptr(bias), _ptr(fault), _stream(),
        ),
        f"gemm_bf16({tokens}x{k} by {n_out})",
    )
    return out


def gemm_bf16_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, fault: torch.Tensor,
                   bias: torch.Tensor | None = None, *, swiglu: bool = False,
                   residual: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None,
                   sumsq_out: torch.Tensor | None = None, sumsq_in: torch.Tensor | None = None,
                   norm_eps: float = 0.0, norm_size: int = 0) -> torch.Tensor:
    """``out[T, N] = x[T, K] @ w[N, K]^T (+ bias)`` in bfloat16 for steps of many tokens: pairs of CTAs on
    256 x 256 tiles (``tcgen05.mma.cta_group::2``), persistent over the tiles, the tokens on the accumulator's lanes.

    The options are those of :func:`gemm_bf16` and mean the same (``swiglu``: ``w`` is ``[2 N, K]``, gate rows
    first; ``residual``, ``norm_weight``, ``sumsq_out``: the norm that follows rides, with a slot of
    ``sumsq_out[T, gemm_bf16_sumsq_count(N)]`` per 32 columns; ``sumsq_in``, ``norm_eps``, ``norm_size``: the scale
    a norm before the product left open), at any number of tokens.  ``N`` must be a multiple of 8."""
    _need_cuda(x, w, out, fault, bias, residual, norm_weight, sumsq_out, sumsq_in)
    for name, tensor in (("x", x), ("w", w), ("out", out)):
        _expect(name, tensor, torch.bfloat16), _contig(name, tensor)
    tokens, k = x.shape
    n_out = out.shape[1]
    if w.shape != ((2 if swiglu else 1) * n_out, k) or out.shape[0] != tokens:
        raise KernelError(f"gemm_bf16_pair: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
    if not gemm_bf16_supports(x, w) or n_out % 8:
        raise KernelError("gemm_bf16_pair: the inner size and the result's width must be multiples of 8 and the operands 16-byte aligned")
    if bias is not None:
        _expect("bias", bias, torch.float32), _contig("bias", bias)
        if bias.shape != (w.shape[0],):
            raise KernelError("gemm_bf16_pair: the bias does not have the weight's rows")
    norm_follows = residual is not None or norm_weight is not None or sumsq_out is not None
    if norm_follows:
        if residual is None or norm_weight is None or sumsq_out is None or swiglu:
            raise KernelError("gemm_bf16_pair: a following norm needs residual, norm_weight and sumsq_out, and no swiglu")
        for name, tensor in (("residual", residual), ("norm_weight", norm_weight), ("sumsq_out", sumsq_out)):
            _expect(name, tensor, torch.float32), _contig(name, tensor)
        if (residual.shape != (tokens, n_out) or norm_weight.shape != (n_out,)
                or sumsq_out.shape != (tokens, gemm_bf16_sumsq_count(n_out))):
            raise KernelError("gemm_bf16_pair: residual, norm_weight or sumsq_out do not have the product's shape")
    if sumsq_in is not None:
        _expect("sumsq_in", sumsq_in, torch.float32), _contig("sumsq_in", sumsq_in)
        if sumsq_in.dim() != 2 or sumsq_in.shape[0] != tokens or sumsq_in.shape[1] % 4 or norm_size <= 0:
            raise KernelError("gemm_bf16_pair: sumsq_in must be [tokens, a multiple of 4] and norm_size positive")
    if tokens == 0:
        return out
    lib = gemm_lib()
    if not getattr(lib, "_pair_declared", False):
        lib.rl_gemm_bf16_pair.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                          c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_float, c_int, c_void_p,
                                          c_void_p, c_void_p, c_void_p, c_void_p]
        lib.rl_gemm_bf16_pair.restype = c_int
        lib.rl_gemm_bf16_pair_scratch_floats.restype = c_longlong
        lib.rl_gemm_bf16_pair_counter_words.restype = c_int
        lib._pair_declared = True
    state = _PAIR_STATE.get(fault.device)
    if state is None:        # partial tiles of the pairs' first segments, and the tiles' counters (the kernel keeps them zero)
        state = (torch.empty(lib.rl_gemm_bf16_pair_scratch_floats(), dtype=torch.float32, device=fault.device),
                 torch.zeros(lib.rl_gemm_bf16_pair_counter_words(), dtype=torch.int32, device=fault.device))
        _PAIR_STATE[fault.device] = state
    _check(lib.rl_gemm_bf16_pair(_ptr(x), _ptr(w), _ptr(out), tokens, n_out, k, int(swiglu), int(PDL),
                                 _ptr(residual), _ptr(norm_weight), _ptr(sumsq_out),
                                 0 if sumsq_out is None else sumsq_out.shape[1],
                                 _ptr(sumsq_in), 0 if sumsq_in is None else sumsq_in.shape[1], float(norm_eps), int(norm_size),
                                 _ptr(bias), _ptr(state[0]), _ptr(state[1]), _ptr(fault), _stream()),
           f"gemm_bf16_pair({tokens}x{k} by {n_out})")
    return out


_PAIR_STATE: dict[torch.device, tuple[torch.Tensor, torch.Tensor]] = {}


def gemm_bf16_pair_takes(tokens: int, n_out: int, swiglu: bool) -> bool:
    """Whether a product of this size is within the pair kernel's table of tiles (256 tokens by 256 columns of the
    result, 128 with ``swiglu``); larger products are the library's."""
    lib = gemm_lib()
    lib.rl_gemm_bf16_pair_counter_words.restype = c_int
    tiles = -(-int(tokens) // 256) * -(-int(n_out) // (128 if swiglu else 256))
    return n_out % 8 == 0 and tiles <= lib.rl_gemm_bf16_pair_counter_words() // 2


class _ChainPhase(ctypes.Structure):
    """``RlChainPhase`` of ``csrc/gemm_chain.cu``."""

    _fields_ = [
        ("x", c_void_p), ("w", c_void_p), ("out", c_void_p), ("n_out", c_int), ("k", c_int), ("swiglu", c_int),
        ("residual", c_void_p), ("norm_weight", c_void_p), ("sumsq_out", c_void_p), ("sumsq_in", c_void_p),
        ("sumsq_count", c_int), ("norm_eps", c_float), ("norm_size", c_int), ("bias", c_void_p),
    ]


GEMM_CHAIN_MAX_PHASES = 4
GEMM_CHAIN_MAX_TOKENS = 64
_CHAIN_STATE: dict[torch.device, dict] = {}


def _chain_lib() -> ctypes.CDLL:
    lib = gemm_lib()
    if not getattr(lib, "_chain_declared", False):
        lib.rl_gemm_chain.argtypes = [c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        lib.rl_gemm_chain_scratch_floats.argtypes = [c_void_p, c_int, c_int]
        lib.rl_gemm_chain_scratch_floats.restype = c_longlong
        lib.rl_gemm_chain.restype = c_int
        lib.rl_gemm_chain_counter_words.restype = c_int
        lib._chain_declared = True
    return lib


def gemm_chain_reset(device=None) -> None:
    """Zero the chain kernel's counters (after a fault: the kernel keeps them zero only when it ends well)."""
    for key, state in _CHAIN_STATE.items():
        if device is None or key == torch.device(device):
            state["counters"].zero_()
    for key, state in _PAIR_STATE.items():
        if device is None or key == torch.device(device):
            state[1].zero_()


def gemm_chain(products: list[dict], fault: torch.Tensor, trace: torch.Tensor | None = None) -> None:
    """Two to four bfloat16 products of the same (at most 64) tokens as one persistent kernel, each reading
    what earlier ones wrote.  A product is the keyword arguments of :func:`gemm_bf16` (``x``, ``w``, ``out``,
    ``swiglu``, ``residual``, ``norm_weight``, ``sumsq_out``, ``sumsq_in``, ``norm_eps``, ``norm_size``,
    ``bias``); the results are those of calling it once per product, up to the order of float32 additions.
    Scratch for partial tiles and the kernel's counters are kept per device and grow on demand.  ``trace``
    (int64 ``[multiprocessors, 4, 8]``) receives the kernel's time stamps per CTA, phase and event."""
    count = len(products)
    if not 1 <= count <= GEMM_CHAIN_MAX_PHASES:
        raise KernelError(f"gemm_chain: takes 1 to {GEMM_CHAIN_MAX_PHASES} products, got {count}")
    tokens = products[0]["x"].shape[0]
    if not 0 < tokens <= GEMM_CHAIN_MAX_TOKENS:
        raise KernelError(f"gemm_chain: takes 1 to {GEMM_CHAIN_MAX_TOKENS} tokens, got {tokens}")
    array = (_ChainPhase * count)()
    for slot, product in zip(array, products):
        x, w, out = product["x"], product["w"], product["out"]
        swiglu = bool(product.get("swiglu", False))
        extras = [product.get(name) for name in ("residual", "norm_weight", "sumsq_out", "sumsq_in", "bias")]
        _need_cuda(x, w, out, fault, *extras)
        for name, tensor in (("x", x), ("w", w), ("out", out)):
            _expect(name, tensor, torch.bfloat16), _contig(name, tensor)
        for name, tensor in zip(("residual", "norm_weight", "sumsq_out", "sumsq_in", "bias"), extras):
            _expect(name, tensor, torch.float32), _contig(name, tensor)
        n_out = out.shape[1]
        if x.shape[0] != tokens or out.shape[0] != tokens or w.shape != ((2 if swiglu else 1) * n_out, x.shape[1]):
            raise KernelError(f"gemm_chain: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
        if not gemm_bf16_supports(x, w):
            raise KernelError("gemm_chain: the inner size must be a multiple of 8 and the operands 16-byte aligned")
        residual, norm_weight, sumsq_out, sumsq_in, bias = extras
        if any(t is not None for t in (residual, norm_weight, sumsq_out)):
            if residual is None or norm_weight is None or sumsq_out is None or swiglu:
                raise KernelError("gemm_chain: a following norm needs residual, norm_weight and sumsq_out, and no swiglu")
            if (residual.shape != (tokens, n_out) or norm_weight.shape != (n_out,)
                    or sumsq_out.shape != (tokens, gemm_bf16_sumsq_count(n_out))):
                raise KernelError("gemm_chain: residual, norm_weight or sumsq_out do not have the product's shape")
        if sumsq_in is not None and (sumsq_in.dim() != 2 or sumsq_in.shape[0] != tokens or sumsq_in.shape[1] % 4
                                     or product.get("norm_size", 0) <= 0):
            raise KernelError("gemm_chain: sumsq_in must be [tokens, a multiple of 4] and norm_size positive")
        if bias is not None and bias.shape != (w.shape[0],):
            raise KernelError("gemm_chain: the bias does not have the weight's rows")
        slot.x, slot.w, slot.out = x.data_ptr(), w.data_ptr(), out.data_ptr()
        slot.n_out, slot.k, slot.swiglu = n_out, x.shape[1], int(swiglu)
        slot.residual = None if residual is None else residual.data_ptr()
        slot.norm_weight = None if norm_weight is None else norm_weight.data_ptr()
        slot.sumsq_out = None if sumsq_out is None else sumsq_out.data_ptr()
        slot.sumsq_in = None if sumsq_in is None else sumsq_in.data_ptr()
        slot.sumsq_count = 0 if sumsq_in is None else sumsq_in.shape[1]
        slot.norm_eps, slot.norm_size = float(product.get("norm_eps", 0.0)), int(product.get("norm_size", 0))
        slot.bias = None if bias is None else bias.data_ptr()
    lib = _chain_lib()
    device = fault.device
    state = _CHAIN_STATE.get(device)
    if state is None:
        state = {"counters": torch.zeros(lib.rl_gemm_chain_counter_words(), dtype=torch.int32, device=device),
                 "scratch": torch.empty(1 << 20, dtype=torch.float32, device=device), "retired": []}
        _CHAIN_STATE[device] = state
    need = int(lib.rl_gemm_chain_scratch_floats(ctypes.byref(array), count, tokens))
    if need > state["scratch"].numel():
        state["retired"].append(state["scratch"])          # a captured graph may still hold its address
        state["scratch"] = torch.empty(need, dtype=torch.float32, device=device)
    stream = _stream()
    _check(
        lib.rl_gemm_chain(ctypes.byref(array), count, tokens, _ptr(state["scratch"]), state["scratch"].numel(),
                          _ptr(state["counters"]), _ptr(trace), int(PDL), _ptr(fault), stream),
        f"gemm_chain({count} products of {tokens} tokens)",
    )


def sample(
    logits: torch.Tensor,
    out: torch.Tensor,
    *,
    temperature: torch.Tensor | None = None,
    top_p: torch.Tensor | None = None,
    penalty: torch.Tensor | None = None,
    seeds: torch.Tensor | None = None,
    counters: torch.Tensor | None = None,
    seen_tokens: torch.Tensor | None = None,
    seen_offsets: torch.Tensor | None = None,
) -> torch.Tensor:
    """One token per row of ``logits`` into ``out`` (int32); no ``temperature`` = greedy."""
    _need_cuda(logits, out, temperature, top_p, penalty, seeds, counters, seen_tokens, seen_offsets)
    _expect("out", out, torch.int32)
    for name, tensor in (("temperature", temperature), ("top_p", top_p), ("penalty", penalty)):
        _expect(name, tensor, torch.float32)
    _expect("seeds", seeds, torch.int64), _expect("counters", counters, torch.int32)
    _expect("seen_tokens", seen_tokens, torch.int32), _expect("seen_offsets", seen_offsets, torch.int32)
    if logits.dim() != 2 or logits.stride(1) != 1 or out.numel() != logits.shape[0]:
        raise KernelError("sample: logits must be [rows, vocab] with contiguous rows and out [rows]")
    _check(
        core().rl_sample(
            dtype_tag(logits.dtype), _ptr(logits), logits.shape[0], logits.shape[1], logits.stride(0),
            _ptr(temperature), _ptr(top_p), _ptr(penalty), _ptr(seeds), _ptr(counters),
            _ptr(seen_tokens), _ptr(seen_offsets), _ptr(out), int(PDL), _stream(),
        ),
        f"sample(vocab={logits.shape[1]})",
    )
    return out


def describe_fault(word: int) -> str:
    parts = [text for bit, text in FAULT_BITS.items() if word & bit]
    return "; ".join(parts) if parts else "no fault"
