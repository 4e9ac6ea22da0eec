"""Grouped-query attention over the paged cache.

Order of operations is the reference's (``rapid_llm/models/base.py:121-165``): one fused
QKV product with columns ``[q | k | v]`` (``rapid_llm/modules/linear.py:236-271``), per-head
RMSNorm of q and k over the head dimension before the rotation (``:134-137``), rotation of q
and k, K/V written to the cache (``rapid_llm/modules/attention.py:126-138``), attention of
every query over its request's cached keys with ``kv_head = q_head // group`` and scale
``head_dim ** -0.5`` (``:62``), output projection without bias.

Every size is a constructor parameter; the window (0 = all keys) and whether q/k are
normed differ per layer if the specification says so, and so does ``qkv_bias`` (a bias on the
q, k and v projections, which this architecture does not have and its predecessor has; added in
float32 in the product's epilogue).  A layer that reads another entry's
cache (``cache.writes`` false) projects queries only.
"""

from __future__ import annotations

import numpy as np
import torch

from ..config.model_spec import PartSpec
from ..ops import gemm, kernels
from .base import (
    MATRIX, MIXERS, POSITION_ENCODINGS, VECTOR, CacheNeed, Mixer, StepPlanner, StepShape, TensorSpec,
)

DEFAULT_SMS = 148         # a B200's; planning on the host without a device (tests) assumes it
MAX_SPLITS = 16
CLUSTER_SPLITS = 16       # the largest thread-block cluster (beyond 8 the kernel asks for it)
TC_CHUNK_MIN_CTAS = 32    # measured: from here on the unsplit tcgen05 chunk kernel beats the split mma.sync tiles
TC_CHUNK_SHORT_CONTEXT = 1024   # ... and below this context it does so with any number of CTAs
MIN_KEYS_PER_SPLIT = 256
PADDING_FREE_BLOCKS = 32  # blocks of 128 keys from which a decode bucket's padding rows stop counting as clusters


# Clusters of the tcgen05 decode kernel a B200 runs at one time, by cluster size (one CTA per multiprocessor, a
# cluster inside one GPC); what planning on the host without a device assumes.
DEFAULT_DECODE_CLUSTERS = {1: 148, 2: 74, 3: 45, 4: 33, 5: 26, 6: 22, 7: 15, 8: 15, 9: 15, 10: 11,
                           11: 7, 12: 7, 13: 7, 14: 7, 15: 7, 16: 7}


def cluster_splits(tiles: int, clusters: dict[int, int]) -> int:
    """Key ranges per tile of a decode-only step on the tcgen05 decode kernel, which merges them inside one
    thread-block cluster: the largest cluster size of which ``tiles`` clusters still run at one time.  (Two
    requests of 8 kv heads are 16 tiles: 16 clusters of 8 would fill 128 multiprocessors, but only 15 such
    clusters fit the GPCs, so the sixteenth would wait for a whole round; 16 clusters of 6 run together.)"""
    best = 1
    for size, count in clusters.items():
        if size > best and size <= CLUSTER_SPLITS and count >= tiles:
            best = size
    return best


class AttentionItems(StepPlanner):
    """Cuts a step into the work items of the tensor-core attention kernels.

    Every entry's packed rows (token, head of the group) are tiled: entries of one token, or
    of at most 16 packed rows, into decode tiles of 16 rows; the others into chunk tiles.  When
    the tiles are too few to fill the GPU, each tile's key range is split into ``splits`` parts
    (the same number for the whole step): in a decode-only step a function of the number of entries and
    of a coarse class of the longest context, so that a captured decode graph replays the same launches at nearly every
    context length (where the tcgen05 decode kernel merges the parts inside a thread-block cluster: the
    largest cluster of which that many run at one time); bounded by the longest context otherwise.  Chunk tiles have 256 rows
    for the tcgen05 kernel, which takes head size 128, the usual page sizes and unsplit key
    ranges, and 64 rows for the mma.sync kernel otherwise.  The tcgen05 kernel is several times
    faster per key, so it also runs, unsplit, where a split would have been wanted, unless its
    CTAs are few and the context long (a few dozen prompt tokens behind thousands of cached ones).
    The longest tiles come first in the list, and the kernels' grids start them in that order.
    The reference picks its split size per launch in the same spirit
    (``rapid_llm/kernels/ops/attention/flashdecoding.py:43-112``).
    """

    def __init__(self, group: int, num_kv_heads: int, head_dim: int = 0, sms: int = DEFAULT_SMS,
                 decode_clusters: dict[int, int] | None = None) -> None:
        self.group, self.num_kv_heads, self.head_dim = int(group), int(num_kv_heads), int(head_dim)
        self.decode_clusters = dict(decode_clusters or DEFAULT_DECODE_CLUSTERS)
        # work items the kernels want in flight: two CTAs per multiprocessor, one in a decode-only
        # step, whose kernel keeps a whole multiprocessor's shared memory busy
        self.target_ctas, self.decode_target_ctas = 2 * int(sms), int(sms)
        self.key = ("attention_items", self.group, self.num_kv_heads, self.head_dim, int(sms),
                    tuple(sorted(self.decode_clusters.items())))

    def capacity(self, max_tokens: int, max_entries: int) -> int:
        chunk_tiles = -(-max_tokens * self.group // kernels.CHUNK_TILE_ROWS) + max_entries
        decode_tiles = max_entries * -(-self.group // kernels.DECODE_TILE_ROWS)
        return 4 * (chunk_tiles + decode_tiles + 2 * self.target_ctas)

    def plan(self, shape: StepShape) -> dict:
        lengths = np.asarray(shape.lengths, dtype=np.int64)
        starts = np.asarray(shape.starts, dtype=np.int64)
        rows = lengths * self.group
        is_decode = (lengths == 1) | (rows <= kernels.DECODE_TILE_ROWS)
        tensor_core = kernels.attention_tc_takes(self.head_dim, shape.page_size)
        for chunk_rows in ((kernels.CHUNK_TILE_ROWS_TC, kernels.CHUNK_TILE_ROWS) if tensor_core else (kernels.CHUNK_TILE_ROWS,)):
            tile_rows = np.where(is_decode, kernels.DECODE_TILE_ROWS, chunk_rows)
            tiles = -(-rows // tile_rows)
            ctas = int(tiles.sum()) * self.num_kv_heads
            target = self.decode_target_ctas if shape.decode_only else self.target_ctas
            splits = max(1, min(MAX_SPLITS, target // max(ctas, 1)))
            if not shape.decode_only:
                longest = int((starts + lengths).max())
                splits = max(1, min(splits, longest // MIN_KEYS_PER_SPLIT))
            elif tensor_core:
                # ... and no more key ranges than the longest context has blocks of keys, rounded down to a power
                # of two: a step's launch constants then change at a handful of context lengths only (the runner
                # keeps a captured graph per set of constants)
                blocks = max(1, -(-int((starts + lengths).max()) // kernels.DECODE_TC_KEYS))
                # On long contexts the padding rows of a decode bucket do not count: their clusters come last in the
                # grid, see one key each, and the round they add (a few microseconds) costs less than the real rows
                # gain from more CTAs (measured at batch 5 of a bucket of 8: 5 % slower at 1,024 tokens, 10 % faster at 32,000).
                counted = ctas
                if blocks >= PADDING_FREE_BLOCKS:
                    real = len(lengths) - int(shape.padding)
                    counted = max(1, int(tiles[:real].sum()) * self.num_kv_heads)
                splits = min(cluster_splits(counted, self.decode_clusters), 1 << (blocks.bit_length() - 1))
            if splits == 1 or chunk_rows == kernels.CHUNK_TILE_ROWS or bool(is_decode.all()):
                break
            # The tcgen05 chunk kernel does not split key ranges, but it is several times faster per
            # key than the mma.sync tiles: it runs unsplit unless it would leave most of the GPU
            # idle on a long context (a few dozen prompt tokens behind thousands of cached ones).
            chunk_ctas = int(tiles[~is_decode].sum()) * self.num_kv_heads
            if chunk_ctas >= TC_CHUNK_MIN_CTAS or longest <= TC_CHUNK_SHORT_CONTEXT:
                splits = 1
                break
        # Single tokens beside prompt portions that the tcgen05 kernel takes unsplit: their tiles get key ranges of
        # their own (merged inside that kernel's clusters), or a request far into its context would be walked by one
        # CTA per kv head while the step waits.
        decode_splits = splits
        if (tensor_core and not shape.decode_only and splits == 1 and chunk_rows == kernels.CHUNK_TILE_ROWS_TC
                and bool(is_decode.any()) and not bool(is_decode.all())):
            decode_ctas = int(tiles[is_decode].sum()) * self.num_kv_heads
            blocks = max(1, -(-int((starts + lengths)[is_decode].max()) // kernels.DECODE_TC_KEYS))
            decode_splits = min(cluster_splits(decode_ctas, self.decode_clusters), 1 << (blocks.bit_length() - 1))
        entry = np.repeat(np.arange(len(lengths), dtype=np.int64), tiles)
        first = np.concatenate(([0], np.cumsum(tiles)[:-1]))
        tile_index = np.arange(int(tiles.sum()), dtype=np.int64) - np.repeat(first, tiles)
        row0 = tile_index * np.repeat(tile_rows, tiles)
        decode_tile = np.repeat(is_decode, tiles)
        # keys a tile has to walk: the tiles with the most go first, so that the last wave is short
        keys = np.repeat(starts, tiles) + (row0 + np.repeat(tile_rows, tiles)) // self.group

        def items(mask: np.ndarray, ranges: int) -> np.ndarray:
            order = np.flatnonzero(mask)
            order = order[np.argsort(-keys[order], kind="stable")]
            count = len(order)
            out = np.zeros((count * ranges, 4), dtype=np.int32)
            out[:, 0] = np.repeat(entry[order], ranges)
            out[:, 1] = np.repeat(row0[order], ranges)
            out[:, 2] = np.tile(np.arange(ranges, dtype=np.int32), count)
            return out

        decode_rows = int(np.minimum(rows[is_decode], kernels.DECODE_TILE_ROWS).max()) if is_decode.any() else 0
        return {"chunk_items": items(~decode_tile, splits), "decode_items": items(decode_tile, decode_splits),
                "splits": splits, "decode_splits": int(decode_splits), "decode_rows": decode_rows,
                "chunk_rows": int(chunk_rows)}


@MIXERS.register("gqa_attention")
class GQAAttention(Mixer):
    rides_norms = True

    def __init__(
        self,
        *,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        position: PartSpec,
        qk_norm: bool = False,
        qk_norm_eps: float = 1e-6,
        window: int = 0,
        scale: float | None = None,
        shares_cache: bool = False,
        qkv_bias: bool = False,
        dtype,
        device,
    ) -> None:
        super().__init__(dtype=dtype, device=device)
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({num_kv_heads})")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim ({head_dim}) must be a multiple of 16 up to 256")
        self.hidden = int(hidden_size)
        self.hq, self.hkv, self.d = int(num_heads), int(num_kv_heads), int(head_dim)
        self.qk_norm, self.eps = bool(qk_norm), float(qk_norm_eps)
        self.window = int(window)
        self.scale = float(scale) if scale is not None else self.d**-0.5
        self.shares_cache = bool(shares_cache)
        device = torch.device(device)
        sms = torch.cuda.get_device_properties(device).multi_processor_count if device.type == "cuda" else DEFAULT_SMS
        clusters = None
        if device.type == "cuda" and dtype == torch.bfloat16:
            clusters = kernels.attention_decode_clusters(self.d, device) or None
        self._items = AttentionItems(self.hq // self.hkv, self.hkv, self.d, sms, clusters)
        self.position = POSITION_ENCODINGS.build(position, dtype=dtype, device=device)
        self.rotary_dim = int(position.params.get("rotary_dim", self.d))

        kv_rows = 0 if self.shares_cache else 2 * self.hkv * self.d
        self.qkv = self.new_storage((self.hq * self.d + kv_rows, self.hidden), MATRIX)
        self.o = self.new_storage((self.hidden, self.hq * self.d), MATRIX)
        self.qkv_bias = self.new_storage((self.qkv.shape[0],), VECTOR) if qkv_bias else None
        self.q_norm = self.new_storage((self.d,), VECTOR) if self.qk_norm else None
        self.k_norm = self.new_storage((self.d,), VECTOR) if self.qk_norm and not self.shares_cache else None

    # -- needs ----------------------------------------------------------------- #
    def cache_need(self) -> CacheNeed | None:
        kind = "window" if self.window > 0 else "full"
        return CacheNeed(kind, self.hkv, self.d, self.window)

    def step_planner(self) -> StepPlanner | None:
        if self.dtype != torch.bfloat16:
            return None      # the float32 path runs the one-warp-per-row kernel: no work list
        return self._items

    # -- weights --------------------------------------------------------------- #
    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {
            "q_proj.weight": TensorSpec((self.hq * self.d, self.hidden)),
            "o_proj.weight": TensorSpec((self.hidden, self.hq * self.d)),
        }
        if not self.shares_cache:
            specs["k_proj.weight"] = TensorSpec((self.hkv * self.d, self.hidden))
            specs["v_proj.weight"] = TensorSpec((self.hkv * self.d, self.hidden))
        if self.qkv_bias is not None:
            for name in ("q_proj", "k_proj", "v_proj")[: 1 if self.shares_cache else 3]:
                specs[f"{name}.bias"] = TensorSpec((specs[f"{name}.weight"].shape[0],), VECTOR)
        if self.qk_norm:
            specs["q_norm.weight"] = TensorSpec((self.d,), VECTOR, init="ones_normal")
            if not self.shares_cache:
                specs["k_norm.weight"] = TensorSpec((self.d,), VECTOR, init="ones_normal")
        return specs

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        q_rows, kv_rows = self.hq * self.d, self.hkv * self.d
        if name == "q_proj.weight":
            self.qkv[:q_rows].copy_(tensor)
        elif name == "k_proj.weight":
            self.qkv[q_rows : q_rows + kv_rows].copy_(tensor)
        elif name == "v_proj.weight":
            self.qkv[q_rows + kv_rows :].copy_(tensor)
        elif name == "o_proj.weight":
            self.o.copy_(tensor)
        elif name == "q_proj.bias":
            self.qkv_bias[:q_rows].copy_(tensor.to(torch.float32))
        elif name == "k_proj.bias":
            self.qkv_bias[q_rows : q_rows + kv_rows].copy_(tensor.to(torch.float32))
        elif name == "v_proj.bias":
            self.qkv_bias[q_rows + kv_rows :].copy_(tensor.to(torch.float32))
        elif name == "q_norm.weight":
            self.q_norm.copy_(tensor.to(torch.float32))
        elif name == "k_norm.weight":
            self.k_norm.copy_(tensor.to(torch.float32))
        else:
            raise KeyError(name)

    def parameter_bytes(self) -> int:
        total = (self.qkv.numel() + self.o.numel()) * self.qkv.element_size()
        for vector in (self.q_norm, self.k_norm, self.qkv_bias):
            if vector is not None:
                total += vector.numel() * 4
        return total

    def workspace_elements_per_token(self) -> int:
        return self.qkv.shape[0] + 2 * self.hq * self.d + self.hidden      # qkv, q, attended, projected

    # -- forward --------------------------------------------------------------- #
    def forward(self, x, batch, cache, then_norm=None):
        if cache.group is None or cache.pages is None:
            raise ValueError("attention needs a cache group; the engine did not give this layer one")
        if cache.writes == self.shares_cache:
            raise ValueError("the layer's cache role in the run order does not match shares_cache")
        group = batch.groups[cache.group]
        rows = x.shape[0]
        qkv = batch.workspace.get("attn_qkv", rows, self.qkv.shape[0], x.dtype)
        gemm.linear(x, self.qkv, qkv, batch.fault, bias=self.qkv_bias, defer=batch.defer_products)
        q = batch.workspace.get("attn_q", rows, self.hq * self.d, x.dtype)
        cos, sin = self.position.tables()
        kernels.qk_norm_rope_write(
            qkv, q,
            num_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.d, rotary_dim=self.rotary_dim,
            cos=cos, sin=sin, positions=batch.positions, eps=self.eps, fault=batch.fault,
            q_weight=self.q_norm, k_weight=self.k_norm,
            kv_dest=group.kv_dest if cache.writes else None,
            cache=cache.pages if cache.writes else None,
            page_size=group.page_size,
        )
        attended = batch.workspace.get("attn_out", rows, self.hq * self.d, x.dtype)
        self.attend(q, cache.pages, attended, batch, group)
        out = batch.workspace.get("attn_proj", rows, self.hidden, x.dtype)
        return gemm.linear(attended, self.o, out, batch.fault, then_norm=then_norm, defer=batch.defer_products)

    def attend(self, q, pages, out, batch, group) -> None:
        if q.dtype == torch.bfloat16:
            plan = batch.extras[self._items.key]
            splits = plan["splits"]
            part_out = part_lse = None
            if splits > 1:
                rows = q.shape[0] * self.hq * splits
                part_out = batch.workspace.get("attn_part_out", rows, self.d, torch.float32, min_rows=rows)
                part_lse = batch.workspace.get("attn_part_lse", rows, 1, torch.float32, min_rows=rows)
            kernels.attention_mma(
                q, pages, out,
                chunk_items=plan["chunk_items"], decode_items=plan["decode_items"], splits=splits,
                part_out=part_out, part_lse=part_lse,
                cu_seqlens=batch.cu_seqlens, entry_start=batch.entry_start, entry_slot=batch.entry_slot,
                block_table=group.block_table, num_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.d,
                window=self.window, scale=self.scale, fault=batch.fault, decode_rows=plan.get("decode_rows", 0),
                chunk_rows=plan.get("chunk_rows", kernels.CHUNK_TILE_ROWS),
                decode_splits=plan.get("decode_splits", 0),
            )
            return
        kernels.attention_generic(
            q, pages, out,
            positions=batch.positions, token_slot=batch.token_slot, block_table=group.block_table,
            num_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.d,
            window=self.window, scale=self.scale, fault=batch.fault,
        )
