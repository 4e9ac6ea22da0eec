"""Reading and writing ``.safetensors`` files.

The format is an 8-byte little-endian header length, a JSON header mapping each
tensor name to ``{"dtype", "shape", "data_offsets"}``, and the raw tensor bytes.
Tensors are read one at a time from a memory map, so a folder far larger than
host memory's free part still loads.  The reference reads the same files through
the ``safetensors`` package, shard by shard in sorted order
(``rapid_llm/executor/weight_utils.py:28-47,100-133``).
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Iterator, Mapping

import torch

_DTYPE_NAMES = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES_OF_DTYPE = {dtype: name for name, dtype in _DTYPE_NAMES.items()}


class SafetensorsFile:
    """One memory-mapped file; ``tensor(name)`` returns a CPU tensor view."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        self._handle = open(self.path, "rb")
        head = self._handle.read(8)
        if len(head) != 8:
            raise ValueError(f"{self.path}: too short to be a safetensors file")
        (header_len,) = struct.unpack("<Q", head)
        size = self.path.stat().st_size
        if header_len <= 0 or 8 + header_len > size:
            raise ValueError(f"{self.path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(self._handle.read(header_len))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise ValueError(f"{self.path}: header is not valid JSON: {exc}") from exc
        self.metadata = header.pop("__metadata__", {})
        self.entries: dict[str, dict] = header
        self._base = 8 + header_len
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_READ)
        for name, entry in self.entries.items():
            begin, end = entry["data_offsets"]
            if entry["dtype"] not in _DTYPE_NAMES:
                raise ValueError(f"{self.path}: tensor {name!r} has unsupported dtype {entry['dtype']}")
            if begin > end or self._base + end > size:
                raise ValueError(f"{self.path}: tensor {name!r} lies outside the file (truncated?)")

    def keys(self) -> list[str]:
        return sorted(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPE_NAMES[self.entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        entry = self.entries[name]
        dtype = _DTYPE_NAMES[entry["dtype"]]
        shape = tuple(entry["shape"])
        begin, end = entry["data_offsets"]
        count = 1
        for extent in shape:
            count *= extent
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        expected = count * torch.empty((), dtype=dtype).element_size()
        if end - begin != expected:
            raise ValueError(
                f"{self.path}: tensor {name!r} holds {end - begin} bytes, "
                f"its shape {list(shape)} needs {expected}"
            )
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)  # read-only buffer
            flat = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._base + begin)
        return flat.view(shape)

    def close(self) -> None:
        try:
            self._map.close()
        except (BufferError, ValueError):
            pass  # tensors still view the map; the OS reclaims it with them
        self._handle.close()

    def __enter__(self) -> "SafetensorsFile":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def checkpoint_files(model_dir: str | Path) -> list[Path]:
    """All ``*.safetensors`` of a folder in name order; an error that names the folder if none."""
    files = sorted(Path(model_dir).glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no *.safetensors file in {Path(model_dir)}")
    return files


def iterate_tensors(model_dir: str | Path) -> Iterator[tuple[str, SafetensorsFile]]:
    """Yield ``(name, file)`` for every tensor of every shard, names sorted per shard."""
    for path in checkpoint_files(model_dir):
        handle = SafetensorsFile(path)
        for name in handle.keys():
            yield name, handle


def write_safetensors(
    path: str | Path, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None
) -> None:
    """Write tensors (any device) to one file, in the mapping's order."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    for name, tensor in tensors.items():
        if tensor.dtype not in _NAMES_OF_DTYPE:
            raise ValueError(f"tensor {name!r}: dtype {tensor.dtype} cannot be stored")
        nbytes = tensor.numel() * tensor.element_size()
        header[name] = {
            "dtype": _NAMES_OF_DTYPE[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + nbytes],
        }
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for tensor in tensors.values():
            data = tensor.detach().contiguous().cpu()
            if data.numel():
                handle.write(data.view(torch.uint8).numpy().tobytes() if data.dim() else
                             data.reshape(1).view(torch.uint8).numpy().tobytes())
