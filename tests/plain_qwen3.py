"""A plain, slow Qwen3 dense decoder: the oracle every engine path is compared with.

Whole sequences, no cache, float32 (or float64) on the CPU, one function per part, written
from the formulas of harleyszhang/rapid_llm; each function cites the file and lines it
follows.  It shares no code with ``rapid_llm_b200``: it parses ``config.json`` and reads
``model.safetensors`` itself.  ``tests/golden/`` holds logits that rapid_llm's own model
code produced on the CPU for two tiny random models, and ``tests/test_plain_vs_golden.py``
compares this file with them.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

_NP_DTYPES = {"F32": np.float32, "F16": np.float16, "F64": np.float64, "I32": np.int32, "I64": np.int64}


def read_safetensors(path: str | Path) -> dict[str, torch.Tensor]:
    """All tensors of one file as float32 (integers stay integers)."""
    blob = Path(path).read_bytes()
    (header_len,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8 : 8 + header_len])
    header.pop("__metadata__", None)
    base = 8 + header_len
    tensors = {}
    for name, entry in header.items():
        begin, end = entry["data_offsets"]
        raw = blob[base + begin : base + end]
        if entry["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            values = torch.from_numpy(bits.view(np.float32).copy())
        else:
            values = torch.from_numpy(np.frombuffer(raw, dtype=_NP_DTYPES[entry["dtype"]]).copy())
            if values.is_floating_point():
                values = values.to(torch.float32)
        tensors[name] = values.reshape(entry["shape"])
    return tensors


def load_model_dir(model_dir: str | Path) -> tuple[dict, dict[str, torch.Tensor]]:
    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    weights: dict[str, torch.Tensor] = {}
    for path in sorted(model_dir.glob("*.safetensors")):
        weights.update(read_safetensors(path))
    return config, weights


# --------------------------------------------------------------------------- parts
def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x_t = E[id_t], no scaling (rapid_llm/models/base.py:589-591, rapid_llm/modules/vocab_parallel.py:101-103)."""
    return table[ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, weight multiplies as w (rapid_llm/kernels/backend/cpu.py:18-29,
    rapid_llm/kernels/ops/layernorm/skip_rmsnorm.py:41-48)."""
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(variance + eps) * weight


def rope_angles(positions: torch.Tensor, rotary_dim: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """inv_freq_i = theta^(-2i/R), angle = p * inv_freq, computed in float32
    (rapid_llm/modules/rotary_embedding.py:30-37,194-202)."""
    exponents = torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim
    inv_freq = 1.0 / (torch.tensor(theta, dtype=torch.float32) ** exponents)
    angles = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(angles), torch.sin(angles)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split rotation, pairs (i, i + R/2): out = [x1*c - x2*s, x2*c + x1*s]; dims past R pass
    through (rapid_llm/kernels/ops/rope/rope_emb.py:47-81, rapid_llm/kernels/backend/cpu.py:45-56).
    x is [T, heads, D]; cos/sin are [T, R/2]."""
    half = cos.shape[-1]
    c, s = cos[:, None, :].to(x.dtype), sin[:, None, :].to(x.dtype)
    x1, x2, rest = x[..., :half], x[..., half : 2 * half], x[..., 2 * half :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, rest), dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0) -> torch.Tensor:
    """Scores (q_i . k_j) * scale over j <= i (and j > i - window when a window is set, the query's own
    position included: rapid_llm/engine/kv_cache_spec.py:204,221-224); softmax over j; o = P v.
    kv head = q head // group (rapid_llm/kernels/ops/attention/flashattention2_nopad.py:85; repeat_interleave
    semantics, rapid_llm/kernels/backend/cpu.py:95-101).  q is [T, Hq, D]; k, v are [T, Hkv, D]."""
    tokens, heads, _ = q.shape
    group = heads // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    i = torch.arange(tokens)[:, None]
    j = torch.arange(tokens)[None, :]
    allowed = j <= i
    if window > 0:
        allowed = allowed & (j > i - window)
    scores = scores.masked_fill(~allowed[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hij,jhd->ihd", probs, v)


def attention_block(x, weights, prefix, cfg, positions, window):
    """q/k/v projections without bias, per-head RMSNorm of q and k before the rotation, rotation, causal
    attention, output projection (rapid_llm/models/base.py:121-165; Qwen3 flags rapid_llm/models/qwen3.py:16-18)."""
    heads, kv_heads, dim = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    tokens = x.shape[0]
    q = (x @ weights[prefix + "self_attn.q_proj.weight"].T).view(tokens, heads, dim)
    k = (x @ weights[prefix + "self_attn.k_proj.weight"].T).view(tokens, kv_heads, dim)
    v = (x @ weights[prefix + "self_attn.v_proj.weight"].T).view(tokens, kv_heads, dim)
    q = rms_norm(q, weights[prefix + "self_attn.q_norm.weight"], cfg["eps"])
    k = rms_norm(k, weights[prefix + "self_attn.k_norm.weight"], cfg["eps"])
    cos, sin = rope_angles(positions, cfg["rotary_dim"], cfg["theta"])
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    out = causal_attention(q, k, v, dim**-0.5, window)
    return out.reshape(tokens, heads * dim) @ weights[prefix + "self_attn.o_proj.weight"].T


def swiglu(x, weights, prefix):
    """down(silu(gate(x)) * up(x)), silu(z) = z * sigmoid(z), no biases (rapid_llm/modules/mlp.py:52-68,
    rapid_llm/kernels/ops/activation/swiglu.py:91-121, rapid_llm/kernels/ops/activation/activations.py:55-57)."""
    gate = x @ weights[prefix + "mlp.gate_proj.weight"].T
    up = x @ weights[prefix + "mlp.up_proj.weight"].T
    return (gate * torch.sigmoid(gate) * up) @ weights[prefix + "mlp.down_proj.weight"].T


def decoder_layer(h, weights, prefix, cfg, positions, window):
    """h' = h + Attn(Norm(h)); h'' = h' + MLP(Norm(h')) (rapid_llm/models/base.py:231-266, with the
    residual adds written out instead of deferred into the next norm)."""
    h = h + attention_block(rms_norm(h, weights[prefix + "input_layernorm.weight"], cfg["eps"]), weights, prefix, cfg, positions, window)
    h = h + swiglu(rms_norm(h, weights[prefix + "post_attention_layernorm.weight"], cfg["eps"]), weights, prefix)
    return h


def layer_windows(config: dict) -> list[int]:
    """Window per layer from the architecture's own keys; 0 = attend to everything.  No windows unless
    ``use_sliding_window`` is on and ``sliding_window`` gives a size; then on the layers that ``layer_types``
    calls ``sliding_attention``, or without that key on the layers from ``max_window_layers`` up."""
    layers = config["num_hidden_layers"]
    window = config.get("sliding_window") or 0
    if not config.get("use_sliding_window") or not window:
        return [0] * layers
    if config.get("layer_types"):
        return [window if kind == "sliding_attention" else 0 for kind in config["layer_types"]]
    first = config.get("max_window_layers") or 0
    return [window if index >= first else 0 for index in range(layers)]


def geometry(config: dict) -> dict:
    heads = config["num_attention_heads"]
    head_dim = config.get("head_dim") or config["hidden_size"] // heads
    return {
        "heads": heads,
        "kv_heads": config.get("num_key_value_heads") or heads,
        "head_dim": head_dim,
        "rotary_dim": int(head_dim * config.get("partial_rotary_factor", 1.0)),
        "eps": config["rms_norm_eps"],
        "theta": float(config.get("rope_theta", 10000.0)),
    }


@torch.no_grad()
def forward_hidden(config: dict, weights: dict[str, torch.Tensor], token_ids, dtype=torch.float32) -> torch.Tensor:
    """The residual stream [T, H] of one whole sequence after the last layer, before the final norm:
    embed, then the layers in order (rapid_llm/models/base.py:556-631)."""
    cfg = geometry(config)
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.numel())
    h = embed(ids, weights["model.embed_tokens.weight"]).to(dtype)
    for index, window in enumerate(layer_windows(config)):
        prefix = f"model.layers.{index}."
        layer = {name: value.to(dtype) for name, value in weights.items() if name.startswith(prefix)}
        h = decoder_layer(h, layer, prefix, cfg, positions, window)
    return h


@torch.no_grad()
def head_logits(config: dict, weights: dict[str, torch.Tensor], hidden: torch.Tensor) -> torch.Tensor:
    """Final norm and output head over the given rows of the residual stream; a tied head uses the embedding
    matrix unless ``lm_head.weight`` is shipped (rapid_llm/models/base.py:619-631, rapid_llm/models/weights.py:197-214)."""
    h = rms_norm(hidden, weights["model.norm.weight"].to(hidden.dtype), config["rms_norm_eps"])
    head = weights.get("lm_head.weight")
    if head is None:
        if not config.get("tie_word_embeddings", False):
            raise KeyError("lm_head.weight is absent and the embeddings are not tied")
        head = weights["model.embed_tokens.weight"]
    return h @ head.to(hidden.dtype).T


def forward_logits(config: dict, weights: dict[str, torch.Tensor], token_ids, dtype=torch.float32, rows=None) -> torch.Tensor:
    """Logits [T, V] of one whole sequence, or of its positions ``rows`` only."""
    hidden = forward_hidden(config, weights, token_ids, dtype)
    return head_logits(config, weights, hidden if rows is None else hidden[list(rows)])


# ------------------------------------------------------------------------ sampling
def philox_uniform(seed: int, counter: int) -> float:
    """Philox4x32-10, key = the 64-bit seed, counter = (counter, 0, 0, 0); first word -> [0, 1) with 24 bits."""
    mask = 0xFFFFFFFF
    c = [counter & mask, 0, 0, 0]
    k0, k1 = seed & mask, (seed >> 32) & mask
    for _ in range(10):
        p0 = 0xD2511F53 * c[0]
        p1 = 0xCD9E8D57 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & mask, p1 & mask, ((p0 >> 32) ^ c[3] ^ k1) & mask, p0 & mask]
        k0 = (k0 + 0x9E3779B9) & mask
        k1 = (k1 + 0xBB67AE85) & mask
    return float(c[0] >> 8) / 16777216.0


def penalised(logits: torch.Tensor, generated, penalty: float) -> torch.Tensor:
    """Divide positive and multiply negative logits of already generated tokens, once per distinct token
    (rapid_llm/engine/sampler.py:134-179)."""
    out = logits.clone().to(torch.float32)
    if penalty != 1.0:
        for token in set(int(t) for t in generated):
            out[token] = out[token] * penalty if out[token] < 0 else out[token] / penalty
    return out


def nucleus(weights: torch.Tensor, top_p: float) -> torch.Tensor:
    """Which tokens the nucleus keeps: those for which the mass ranked before them does not exceed
    ``top_p`` of the whole (rapid_llm/engine/sampler.py:223-244); ``weights`` need not be normalised."""
    keep = torch.ones_like(weights, dtype=torch.bool)
    if top_p < 1.0:
        total = float(weights.sum())
        order = torch.argsort(weights, descending=True, stable=True)
        sorted_w = weights[order]
        before = torch.cumsum(sorted_w.double(), 0) - sorted_w.double()     # mass ranked before each token
        # tokens of equal weight share the mass strictly above them: that of the first of their run
        _, run, counts = torch.unique_consecutive(sorted_w, return_inverse=True, return_counts=True)
        run_start = torch.cumsum(counts, 0) - counts
        strictly_above = before[run_start[run]]
        keep = torch.zeros_like(keep)
        keep[order[strictly_above <= top_p * total]] = True
    return keep


def sample_token(logits, temperature, top_p=1.0, penalty=1.0, generated=(), seed=0, counter=0) -> int:
    """Greedy = first index of the maximum (rapid_llm/engine/sampler.py:266-283).  Otherwise
    softmax(logits / T) (:669-672); keep tokens while the mass ranked before them is <= top_p (:223-244);
    draw by inverse CDF in index order over the kept mass with u = philox(seed, counter)."""
    values = penalised(torch.as_tensor(logits), generated, penalty)
    if temperature <= 0:
        return int(torch.argmax(values))
    scaled = values / temperature
    weights = torch.exp(scaled - scaled.max())
    keep = nucleus(weights, top_p)
    kept = torch.where(keep, weights, torch.zeros_like(weights))
    target = philox_uniform(seed, counter) * float(kept.sum())
    running = torch.cumsum(kept.double(), 0)
    picks = torch.nonzero((running > target) & keep)
    return int(picks[0]) if len(picks) else int(torch.argmax(values))


def greedy_generate(config, weights, prompt, steps: int, dtype=torch.float32) -> list[int]:
    tokens = list(prompt)
    for _ in range(steps):
        logits = forward_logits(config, weights, tokens, dtype)
        tokens.append(int(torch.argmax(logits[-1])))
    return tokens[len(prompt):]
