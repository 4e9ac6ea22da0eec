"""A mixer with per-request state of its own through the scheduler: slots handed on, requests evicted and recomputed.

The toy mixer keeps a running, decaying sum of its inputs per request in the state slot the cache manager gives it
(``StateNeed``); a second layer is the stock attention.  Twelve requests go through three slots and a pool of pages
that holds one of the longest and little more, in portions, beside decoded tokens: a slot's state must be zeroed when a request
takes it over, and a request that was evicted starts again from nothing.  Every request's greedy tokens are those of
a plain restatement that runs each sequence whole.
"""

from __future__ import annotations

import dataclasses

import pytest
import torch
from plain_qwen3 import apply_rope, causal_attention, load_model_dir, rms_norm, rope_angles, swiglu

pytestmark = pytest.mark.gpu

HIDDEN, VOCAB, EPS, THETA, POSITIONS, DECAY = 48, 131, 1e-5, 10000.0, 128, 0.75
HEADS, KV_HEADS, DIM, INTER = 3, 1, 16, 80


def register_parts():
    from rapid_llm_b200.parts import MIXERS, Mixer, StateNeed, TensorSpec

    if "running_sum" in MIXERS.kinds():
        return

    @MIXERS.register("running_sum")
    class RunningSum(Mixer):
        """s_t = decay * s_{t-1} + x_t per request; y_t = s_t @ W^T."""

        def __init__(self, *, hidden_size, decay, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.hidden, self.decay = hidden_size, decay
            self.weight = self.new_storage((hidden_size, hidden_size), "matrix")

        def state_need(self):
            return StateNeed((self.hidden,), torch.float32)

        def tensor_specs(self):
            return {"proj.weight": TensorSpec((self.hidden, self.hidden))}

        def load_tensor(self, name, tensor):
            assert name == "proj.weight"
            self.weight.copy_(tensor)

        def forward(self, x, batch, cache):
            out = torch.empty_like(x)
            for index in range(batch.num_entries):
                begin, end = int(batch.h_cu_seqlens[index]), int(batch.h_cu_seqlens[index + 1])
                state = cache.state[int(batch.h_entry_slot[index])]
                for row in range(begin, end):
                    state.mul_(self.decay).add_(x[row].float())
                    out[row] = (state @ self.weight.float().T).to(x.dtype)
            return out


@dataclasses.dataclass(frozen=True)
class RunningSumConfig:
    vocab_size: int = VOCAB
    hidden_size: int = HIDDEN
    architecture = "RunningSumForCausalLM"
    model_type = "running_sum_toy"

    @classmethod
    def from_dict(cls, raw, overrides=None):
        raw = dict(raw, **(overrides or {}))
        return cls(raw["vocab_size"], raw["hidden_size"])

    def to_dict(self):
        return {"architectures": [self.architecture], "model_type": self.model_type, **dataclasses.asdict(self)}

    def to_spec(self):
        from rapid_llm_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": EPS})
        summing = PartSpec("running_sum", {"hidden_size": self.hidden_size, "decay": DECAY})
        attention = PartSpec("gqa_attention", {
            "hidden_size": self.hidden_size, "num_heads": HEADS, "num_kv_heads": KV_HEADS, "head_dim": DIM, "qk_norm": True,
            "qk_norm_eps": EPS,
            "position": PartSpec("rope", {"head_dim": DIM, "rotary_dim": DIM, "theta": THETA, "max_positions": POSITIONS}),
        })
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": INTER})
        layers = tuple(LayerSpec("prenorm", mixer, ffn, norm, f"model.layers.{i}.") for i, mixer in enumerate((summing, attention)))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=self.hidden_size, max_positions=POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
            layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(2)), final_norm=norm,
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied": True}),
        )


def plain_logits(weights: dict, tokens: list[int]) -> torch.Tensor:
    count = len(tokens)
    h = weights["model.embed_tokens.weight"][tokens]
    # layer 0: the running sum
    prefix = "model.layers.0."
    x = rms_norm(h, weights[prefix + "input_layernorm.weight"], EPS)
    state, rows = torch.zeros(HIDDEN), []
    for row in range(count):
        state = state * DECAY + x[row]
        rows.append(state @ weights[prefix + "self_attn.proj.weight"].T)      # the arrangement names its mixer self_attn
    h = h + torch.stack(rows)
    h = h + swiglu(rms_norm(h, weights[prefix + "post_attention_layernorm.weight"], EPS), weights, prefix)
    # layer 1: attention
    prefix = "model.layers.1."
    cos, sin = rope_angles(torch.arange(count), DIM, THETA)
    x = rms_norm(h, weights[prefix + "input_layernorm.weight"], EPS)
    q = (x @ weights[prefix + "self_attn.q_proj.weight"].T).view(count, HEADS, DIM)
    k = (x @ weights[prefix + "self_attn.k_proj.weight"].T).view(count, KV_HEADS, DIM)
    v = (x @ weights[prefix + "self_attn.v_proj.weight"].T).view(count, KV_HEADS, DIM)
    q = apply_rope(rms_norm(q, weights[prefix + "self_attn.q_norm.weight"], EPS), cos, sin)
    k = apply_rope(rms_norm(k, weights[prefix + "self_attn.k_norm.weight"], EPS), cos, sin)
    h = h + causal_attention(q, k, v, DIM**-0.5).reshape(count, HEADS * DIM) @ weights[prefix + "self_attn.o_proj.weight"].T
    h = h + swiglu(rms_norm(h, weights[prefix + "post_attention_layernorm.weight"], EPS), weights, prefix)
    return rms_norm(h, weights["model.norm.weight"], EPS) @ weights["model.embed_tokens.weight"].T


def plain_greedy(weights: dict, prompt: list[int], count: int) -> list[int]:
    tokens, made = list(prompt), []
    for _ in range(count):
        made.append(int(plain_logits(weights, tokens)[-1].argmax()))
        tokens.append(made[-1])
    return made


def test_state_slots_survive_eviction_and_reuse(tmp_path):
    from rapid_llm_b200 import LLM, SamplingParams
    from rapid_llm_b200.config import register_architecture
    from rapid_llm_b200.weights import write_random_model

    register_parts()
    register_architecture(RunningSumConfig)
    folder = write_random_model(tmp_path / "model", RunningSumConfig(), seed=51, dtype=torch.float32)
    _, weights = load_model_dir(folder)
    generator = torch.Generator().manual_seed(53)
    lengths = torch.randint(3, 70, (12,), generator=generator).tolist()
    budgets = torch.randint(2, 14, (12,), generator=generator).tolist()
    prompts = [torch.randint(0, VOCAB, (n,), generator=generator).tolist() for n in lengths]
    page = 8
    llm = LLM(folder, dtype="float32", max_seq_len=POSITIONS, max_gpu_num_blocks=14, page_size=page,
              max_num_seqs=3, max_chunk_size=17, max_num_batched_tokens=40, use_cuda_graph=False)
    assert [need is not None for need in llm.runner.model.state_needs()] == [True, False]
    outputs = llm.generate(prompts, [SamplingParams.greedy(max_gen_len=n) for n in budgets])
    for prompt, budget, output in zip(prompts, budgets, outputs):
        assert output.token_ids == plain_greedy(weights, prompt, budget), (len(prompt), budget)
    llm.runner.cache.check()
    assert llm.runner.cache.num_free_slots == 3
    assert llm.scheduler.num_preemptions >= 1
