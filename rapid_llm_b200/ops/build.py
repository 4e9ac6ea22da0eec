"""Compiles the CUDA sources under ``csrc/`` for sm_100a and loads them with ``ctypes``.

The kernels are plain ``extern "C"`` entry points over raw device pointers, so a source
compiles in seconds without the PyTorch headers.  Sources are grouped into libraries that
are built on first use (``core`` has what every step needs, the others are the heavier
tensor-core families), keyed by a hash of their text and flags, into
``rapid_llm_b200/csrc/_build`` — or, when the package folder cannot be written, into
``$RAPID_LLM_B200_BUILD_DIR`` or a per-user folder under the system's temporary directory.
A line is printed to stderr for every file compiled, so a first call does not look hung.
There is no fallback: without ``nvcc`` or on a compile error, loading raises.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = [
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
]

# library name -> its sources (relative to csrc/); per-library flags in LIBRARY_FLAGS
LIBRARIES: dict[str, list[str]] = {
    "core": [
        "elementwise.cu",
        "rope_kv.cu",
        "attention_generic.cu",
        "gemm_f32.cu",
        "sampling.cu",
    ],
    "gemm": ["gemm_bf16.cu", "gemm_chain.cu", "gemm_bf16_pair.cu"],
}
LIBRARY_FLAGS: dict[str, list[str]] = {}

# head sizes whose attention library `build_all` compiles ahead of time unless told otherwise (the
# architecture's 128 and the common 64); any other multiple of 16 up to 256 is compiled when a model
# with that head size is first built
DEFAULT_HEAD_DIMS = (64, 128)


def attention_library(head_dim: int) -> str:
    """Name of the tensor-core attention library specialised for one head size."""
    head_dim = int(head_dim)
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise BuildError(f"the attention kernels take head sizes in steps of 16 up to 256, got {head_dim}")
    name = f"attention_d{head_dim}"
    if name not in LIBRARIES:
        LIBRARIES[name] = ["attention_mma.cu"]
        LIBRARY_FLAGS[name] = [f"-DRL_HEAD_DIM={head_dim}"]
    return name

_LOCK = threading.Lock()
_LOADED: dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    """The CUDA extension could not be built or loaded."""


def _say(message: str) -> None:
    print(f"[rapid_llm_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(Path(os.environ[var]) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        candidates.append(Path(found))
    candidates.append(Path("/usr/local/cuda/bin/nvcc"))
    for candidate in candidates:
        if candidate.is_file():
            return str(candidate)
    raise BuildError(
        "nvcc was not found (looked at $CUDA_HOME/bin, PATH and /usr/local/cuda/bin); "
        "the CUDA kernels cannot be built and there is no fallback path"
    )


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _digest(sources: list[Path], flags: list[str]) -> str:
    sha = hashlib.sha256()
    sha.update(" ".join(flags).encode())
    for path in _headers() + sources:
        sha.update(path.name.encode())
        sha.update(path.read_bytes())
    return sha.hexdigest()[:16]


def _writable_dir(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe_{os.getpid()}_{threading.get_ident()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    choices = []
    if os.environ.get("RAPID_LLM_B200_BUILD_DIR"):
        choices.append(Path(os.environ["RAPID_LLM_B200_BUILD_DIR"]))
    choices.append(CSRC / "_build")
    choices.append(Path(tempfile.gettempdir()) / f"rapid_llm_b200_build_{os.getuid()}")
    for choice in choices:
        if _writable_dir(choice):
            return choice
    raise BuildError(f"no writable build folder among {[str(c) for c in choices]}")


def _existing(name: str, digest: str) -> Path | None:
    """A library built earlier for exactly these sources, wherever it was written."""
    filename = f"librapid_llm_b200_{name}_{digest}.so"
    places = [CSRC / "_build"]
    if os.environ.get("RAPID_LLM_B200_BUILD_DIR"):
        places.insert(0, Path(os.environ["RAPID_LLM_B200_BUILD_DIR"]))
    places.append(Path(tempfile.gettempdir()) / f"rapid_llm_b200_build_{os.getuid()}")
    for place in places:
        if (place / filename).is_file():
            return place / filename
    return None


def _compile_one(nvcc: str, source: Path, obj: Path, flags: list[str]) -> None:
    started = time.time()
    _say(f"compiling {source.name} for sm_100a ...")
    cmd = [nvcc, *ARCH_FLAGS, *flags, "-I", str(CSRC), "-c", str(source), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {source.name}:\n{proc.stdout}\n{proc.stderr}")
    _say(f"compiled {source.name} in {time.time() - started:.1f}s")


def build_library(name: str, extra_flags: list[str] | None = None) -> Path:
    """Build (if needed) and return the path of one library."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library {name!r}; known: {sorted(LIBRARIES)}")
    sources = [CSRC / rel for rel in LIBRARIES[name]]
    missing = [str(p) for p in sources if not p.is_file()]
    if missing:
        raise BuildError(f"kernel sources missing: {missing}")
    flags = COMMON_FLAGS + LIBRARY_FLAGS.get(name, []) + list(extra_flags or [])
    digest = _digest(sources, flags)
    ready = _existing(name, digest)
    if ready is not None:
        return ready
    nvcc = find_nvcc()
    out_dir = build_dir()
    target = out_dir / f"librapid_llm_b200_{name}_{digest}.so"
    work = Path(tempfile.mkdtemp(prefix=f"{name}_", dir=out_dir))
    try:
        objects = [work / (src.stem + ".o") for src in sources]
        _say(f"building kernel library '{name}' ({len(sources)} files) into {out_dir}")
        with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
            futures = [
                pool.submit(_compile_one, nvcc, src, obj, flags)
                for src, obj in zip(sources, objects)
            ]
            for future in futures:
                future.result()
        staged = work / target.name
        link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(staged), *map(str, objects), "-lcudart"]
        proc = subprocess.run(link, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"linking {target.name} failed:\n{proc.stdout}\n{proc.stderr}")
        os.replace(staged, target)  # atomic: a concurrent builder sees all or nothing
        _say(f"built {target.name}")
        for older in out_dir.glob(f"librapid_llm_b200_{name}_*.so"):
            if older != target:         # of sources that no longer exist; a process that has it loaded keeps it
                older.unlink(missing_ok=True)
    finally:
        shutil.rmtree(work, ignore_errors=True)
    return target


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library, built first if this is the first use of these sources."""
    with _LOCK:
        if name not in _LOADED:
            path = build_library(name)
            try:
                _LOADED[name] = ctypes.CDLL(str(path))
            except OSError as exc:
                raise BuildError(f"cannot load {path}: {exc}") from exc
        return _LOADED[name]


def build_all(head_dims=None) -> list[Path]:
    """Compile every library, the attention library for each of ``head_dims`` (default
    :data:`DEFAULT_HEAD_DIMS`); several at a time."""
    for head_dim in (DEFAULT_HEAD_DIMS if head_dims is None else head_dims):
        attention_library(head_dim)
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        return list(pool.map(build_library, list(LIBRARIES)))
