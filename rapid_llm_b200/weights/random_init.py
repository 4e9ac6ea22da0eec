"""Random-weights mode: write a model folder from a configuration and a seed.

The folder holds ``config.json`` and ``model.safetensors`` with the architecture's own
tensor names, so any other implementation can load the identical model.  Tensors are drawn
on the host from one ``torch.Generator`` seeded with ``seed``, in the fixed order of the
model's tensor list (embedding, each layer's tensors, final norm, head): matrices and
embeddings from N(0, ``std``), norm scales from 1 + N(0, ``norm_std``).  A tied head is not
written.  The reference has no such mode on its product path; its layer harness uses
``RANDOM_STD = 0.02`` (``rapid_llm/tools/harness/single_layer.py:33-37``).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Iterator

import torch

from ..models.causal_lm import CausalLM
from ..parts.base import TABLE, VECTOR, TensorSpec
from .safetensors_io import write_safetensors


def _draw(spec: TensorSpec, generator: torch.Generator, std: float, norm_std: float) -> torch.Tensor:
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=torch.float32)
    values = torch.empty(spec.shape, dtype=torch.float32).normal_(0.0, 1.0, generator=generator)
    if spec.init == "ones_normal":
        return 1.0 + norm_std * values
    if spec.init == "normal":
        return std * values
    raise ValueError(f"unknown init {spec.init!r}")


def random_tensors(
    config, seed: int, *, dtype: torch.dtype = torch.float32, std: float = 0.02, norm_std: float = 0.1
) -> Iterator[tuple[str, torch.Tensor]]:
    """``(name, tensor)`` in file order; matrices in ``dtype``, vectors in float32."""
    spec = config.to_spec()
    skeleton = CausalLM(spec, torch.float32, "meta")
    generator = torch.Generator(device="cpu").manual_seed(int(seed))
    for name, tensor_spec in skeleton.tensor_specs().items():
        if tensor_spec.optional:
            continue
        values = _draw(tensor_spec, generator, std, norm_std)
        if tensor_spec.kind == VECTOR:
            yield name, values
        elif tensor_spec.kind == TABLE:
            yield name, values.to(torch.int32)
        else:
            yield name, values.to(dtype)


def write_random_model(
    model_dir: str | Path,
    config,
    seed: int,
    *,
    dtype: torch.dtype = torch.float32,
    std: float = 0.02,
    norm_std: float = 0.1,
) -> Path:
    """Create ``model_dir`` with ``config.json`` and ``model.safetensors``."""
    out = Path(model_dir)
    out.mkdir(parents=True, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16"}[dtype]
    (out / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    tensors = dict(random_tensors(config, seed, dtype=dtype, std=std, norm_std=norm_std))
    write_safetensors(
        out / "model.safetensors", tensors,
        metadata={"format": "pt", "seed": str(seed), "std": str(std), "norm_std": str(norm_std)},
    )
    return out


def fill_random_on_device(model: CausalLM, seed: int, *, std: float = 0.02, norm_std: float = 0.0) -> None:
    """Fill a built model's storage in place from a device generator (for benchmarks).

    Same distributions as :func:`write_random_model`, but drawn on the GPU tensor by tensor,
    so a model of many gigabytes is ready in seconds.  The values differ from the host
    generator's; use the folder mode where another implementation must load the same model.
    """
    generator = torch.Generator(device=model.device).manual_seed(int(seed))
    loaded: set[str] = set()
    for name, spec in model.tensor_specs().items():
        if spec.optional:
            continue
        values = torch.empty(spec.shape, dtype=torch.float32, device=model.device)
        if spec.init == "zeros":
            values.zero_()
        else:
            values.normal_(0.0, 1.0, generator=generator)
            if spec.init == "ones_normal":
                values.mul_(norm_std).add_(1.0)
            else:
                values.mul_(std)
        model.load_tensor(name, values)
        loaded.add(name)
        del values
    model.finalize(loaded)
