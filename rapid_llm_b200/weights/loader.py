"""Loading a model folder's safetensors into a built model, by tensor name.

Every tensor the parts expect is looked up by its checkpoint name, checked against the
expected shape, and copied into the part's storage (matrix operands in the engine dtype,
scale vectors in float32, integer tables in int32).  Anything that does not fit is
collected and reported in ONE error that lists missing tensors, unexpected tensors and
wrong shapes.  The reference reports the same classes of fault
(``rapid_llm/models/weights.py:186-194,217-239``, ``rapid_llm/modules/linear.py:84-101``).
"""

from __future__ import annotations

from pathlib import Path

import torch

from .safetensors_io import SafetensorsFile, checkpoint_files

_FLOAT_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


class WeightLoadError(ValueError):
    """The folder's tensors do not match what the model expects."""

    def __init__(self, missing, unexpected, wrong_shape, other=()) -> None:
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.other = list(other)
        lines = ["model weights do not match the configuration:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}):")
            lines.extend(
                f"    {name}: file has {list(found)}, model expects {list(expected)}"
                for name, found, expected in self.wrong_shape
            )
        lines.extend(f"  {text}" for text in self.other)
        super().__init__("\n".join(lines))


def load_weights(model, model_dir: str | Path) -> dict[str, int]:
    """Fill ``model`` from ``model_dir``; returns counts for logging.

    Tensors of layers the configuration does not have (index beyond the layer count) are
    ignored, as the reference does (``rapid_llm/models/base.py:494-497``).
    """
    expected = model.tensor_specs()
    layer_prefixes = {layer.prefix.rsplit(".", 2)[0] + "." for layer in model.spec.layers}
    seen: set[str] = set()
    unexpected: list[str] = []
    wrong: list[tuple[str, tuple, tuple]] = []
    other: list[str] = []
    files = [SafetensorsFile(path) for path in checkpoint_files(model_dir)]
    try:
        for handle in files:
            for name in handle.keys():
                spec = expected.get(name)
                if spec is None:
                    if _is_surplus_layer(name, layer_prefixes, len(model.spec.layers)):
                        continue
                    unexpected.append(name)
                    continue
                if name in seen:
                    other.append(f"{name} appears in more than one file")
                    continue
                seen.add(name)
                found = handle.shape(name)
                if tuple(found) != tuple(spec.shape):
                    wrong.append((name, tuple(found), tuple(spec.shape)))
                    continue
                dtype = handle.dtype(name)
                if dtype not in _FLOAT_DTYPES and spec.kind != "table":
                    other.append(f"{name} is stored as {dtype}, expected a float type")
                    continue
        missing = [name for name, spec in expected.items() if name not in seen and not spec.optional]
        if missing or unexpected or wrong or other:
            raise WeightLoadError(missing, unexpected, wrong, other)
        for handle in files:
            for name in handle.keys():
                if name in expected:
                    model.load_tensor(name, handle.tensor(name))
        model.finalize(seen)
    finally:
        for handle in files:
            handle.close()
    return {"tensors": len(seen), "files": len(files)}


def _is_surplus_layer(name: str, layer_prefixes: set[str], num_layers: int) -> bool:
    for prefix in layer_prefixes:
        if name.startswith(prefix):
            index = name[len(prefix):].split(".", 1)[0]
            if index.isdigit() and int(index) >= num_layers:
                return True
    return False
