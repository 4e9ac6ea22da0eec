"""Grouped-query attention over the paged cache.

Order of operations is the reference's (``rapid_llm/models/base.py:121-165``): one fused
QKV product with columns ``[q | k | v]`` (``rapid_llm/modules/linear.py:236-271``), per-head
RMSNorm of q and k over the head dimension before the rotation (``:134-137``), rotation of q
and k, K/V written to the cache (``rapid_llm/modules/attention.py:126-138``), attention of
every query over its request's cached keys with ``kv_head = q_head // group`` and scale
``head_dim ** -0.5`` (``:62``), output projection without bias.

Every size is a constructor parameter; the window (0 = all keys) and whether q/k are
normed differ per layer if the specification says so.  A layer that reads another entry's
cache (``cache.writes`` false) projects queries only.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import gemm, kernels
from .base import MATRIX, MIXERS, POSITION_ENCODINGS, VECTOR, CacheNeed, Mixer, TensorSpec


@MIXERS.register("gqa_attention")
class GQAAttention(Mixer):
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
        self.position = POSITION_ENCODINGS.build(position, dtype=dtype, device=device)
        self.rotary_dim = int(position.params.get("rotary_dim", self.d))

        kv_rows = 0 if self.shares_cache else 2 * self.hkv * self.d
        self.qkv = self.new_storage((self.hq * self.d + kv_rows, self.hidden), MATRIX)
        self.o = self.new_storage((self.hidden, self.hq * self.d), MATRIX)
        self.q_norm = self.new_storage((self.d,), VECTOR) if self.qk_norm else None
        self.k_norm = self.new_storage((self.d,), VECTOR) if self.qk_norm and not self.shares_cache else None

    # -- needs ----------------------------------------------------------------- #
    def cache_need(self) -> CacheNeed | None:
        kind = "window" if self.window > 0 else "full"
        return CacheNeed(kind, self.hkv, self.d, self.window)

    # -- weights --------------------------------------------------------------- #
    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {
            "q_proj.weight": TensorSpec((self.hq * self.d, self.hidden)),
            "o_proj.weight": TensorSpec((self.hidden, self.hq * self.d)),
        }
        if not self.shares_cache:
            specs["k_proj.weight"] = TensorSpec((self.hkv * self.d, self.hidden))
            specs["v_proj.weight"] = TensorSpec((self.hkv * self.d, self.hidden))
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
        elif name == "q_norm.weight":
            self.q_norm.copy_(tensor.to(torch.float32))
        elif name == "k_norm.weight":
            self.k_norm.copy_(tensor.to(torch.float32))
        else:
            raise KeyError(name)

    def parameter_bytes(self) -> int:
        total = (self.qkv.numel() + self.o.numel()) * self.qkv.element_size()
        for vector in (self.q_norm, self.k_norm):
            if vector is not None:
                total += vector.numel() * 4
        return total

    # -- forward --------------------------------------------------------------- #
    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        if cache.group is None or cache.pages is None:
            raise ValueError("attention needs a cache group; the engine did not give this layer one")
        if cache.writes == self.shares_cache:
            raise ValueError("the layer's cache role in the run order does not match shares_cache")
        group = batch.groups[cache.group]
        rows = x.shape[0]
        qkv = batch.workspace.get("attn_qkv", rows, self.qkv.shape[0], x.dtype)
        gemm.linear(x, self.qkv, qkv)
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
        return gemm.linear(attended, self.o, out)

    def attend(self, q, pages, out, batch, group) -> None:
        kernels.attention_generic(
            q, pages, out,
            positions=batch.positions, token_slot=batch.token_slot, block_table=group.block_table,
            num_heads=self.hq, num_kv_heads=self.hkv, head_dim=self.d,
            window=self.window, scale=self.scale, fault=batch.fault,
        )
