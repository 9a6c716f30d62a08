"""Compiles the CUDA sources of this folder for sm_100a and loads them with ctypes.

Nothing is compiled at import.  The first call that needs a library compiles its
sources with nvcc (one object per file, in parallel), links them into one shared
object under `csrc/_build/` (or a per-user temporary folder when the package folder
is read-only) and prints a progress line every few seconds meanwhile.  The file name
carries a hash of the sources, the flags and the defines, so an edited kernel or a
different specialisation never loads a stale binary.  There is no fallback: without
nvcc or with a failing compile this raises.
"""

from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path
from typing import Dict, Iterable, Sequence, Tuple

CSRC = Path(__file__).resolve().parent

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]

# library name -> sources; a library may also be requested with -D defines (specialisations)
LIBRARIES: Dict[str, Sequence[str]] = {
    "core": ("elementwise.cu", "gemm_f32.cu", "attention_generic.cu", "sampling.cu"),
    # tensor-core attention, one build per head size: defines=("-DHEAD_DIM=128",)
    "attn_mma": ("attention_mma.cu",),
    # attention for prompt portions with scores and outputs in tensor memory (head size 64 or 128)
    "attn_tc": ("attention_tcgen05.cu",),
    # tcgen05 / TMA matrix product for steps of few tokens
    "gemm_decode": ("gemm_decode_tcgen05.cu",),
    # tcgen05 / TMA matrix product for steps of many tokens, with fused bias or SwiGLU
    "gemm_tiles": ("gemm_tiles_tcgen05.cu",),
    # mma.sync product without set-up for steps of few tokens against small matrices
    "gemm_skinny": ("gemm_skinny.cu",),
}
# specialisations compiled by build_all() beside the default form of every library
DEFAULT_SPECIALISATIONS = {"attn_mma": [("-DHEAD_DIM=128",)],
                           "attn_tc": [("-DHEAD_DIM=128",)]}

_loaded: Dict[Tuple[str, Tuple[str, ...]], ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise BuildError("nvcc was not found (set NVCC or put it on PATH); the engine has no "
                     "path without its CUDA kernels")


def _build_dir() -> Path:
    preferred = CSRC / "_build"
    try:
        preferred.mkdir(exist_ok=True)
        probe = preferred / f".write-test-{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return preferred
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"fsie-build-{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def _digest(sources: Iterable[Path], defines: Sequence[str]) -> str:
    h = hashlib.sha256()
    for header in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(header.name.encode())
        h.update(header.read_bytes())
    for source in sources:
        h.update(source.name.encode())
        h.update(source.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + list(defines)).encode())
    return h.hexdigest()[:16]


def _say(message: str) -> None:
    print(f"[fsie-build] {message}", file=sys.stderr, flush=True)


def _run_with_progress(commands, label: str) -> None:
    """Run the compile commands in parallel; print a line every few seconds until done."""
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    started = time.time()
    processes = [(cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                        text=True, env=env, cwd=str(CSRC)))
                 for cmd in commands]
    last = started
    while any(p.poll() is None for _, p in processes):
        time.sleep(0.2)
        if time.time() - last >= 5.0:
            running = sum(p.poll() is None for _, p in processes)
            _say(f"{label}: still compiling ({running} of {len(processes)} files, "
                 f"{time.time() - started:.0f} s)")
            last = time.time()
    for cmd, process in processes:
        output = process.stdout.read() if process.stdout else ""
        if process.returncode != 0:
            raise BuildError(f"nvcc failed ({process.returncode}): {' '.join(cmd)}\n{output}")


def library_path(name: str, defines: Sequence[str] = ()) -> Path:
    """Compile (if needed) and return the shared object of library `name`."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library '{name}' (known: {', '.join(LIBRARIES)})")
    sources = [CSRC / s for s in LIBRARIES[name]]
    defines = tuple(defines)
    tag = _digest(sources, defines)
    suffix = "".join("-" + d.replace("-D", "").replace("=", "") for d in defines)
    out_dir = _build_dir()
    target = out_dir / f"fsie_{name}{suffix}-{tag}.so"
    if target.exists():
        return target
    nvcc = _nvcc()
    lock_path = out_dir / f".{target.name}.lock"
    with open(lock_path, "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)
        try:
            if target.exists():
                return target
            label = f"{name}{suffix}"
            _say(f"compiling kernel library '{label}' for sm_100a ({len(sources)} files), "
                 f"first use only")
            started = time.time()
            work = Path(tempfile.mkdtemp(prefix="obj-", dir=str(out_dir)))
            try:
                objects = [work / (s.stem + ".o") for s in sources]
                commands = [[nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *defines, "-I", str(CSRC), "-c",
                             str(s), "-o", str(o)] for s, o in zip(sources, objects)]
                _run_with_progress(commands, label)
                partial = work / target.name
                _run_with_progress([[nvcc, "-shared", *ARCH_FLAGS, "-o", str(partial),
                                     *map(str, objects), "-lcudart"]], label + " (link)")
                os.replace(partial, target)
            finally:
                shutil.rmtree(work, ignore_errors=True)
            _say(f"built {target.name} in {time.time() - started:.0f} s")
        finally:
            fcntl.flock(lock_file, fcntl.LOCK_UN)
            try:
                lock_path.unlink()
            except OSError:
                pass
    return target


def load_library(name: str, defines: Sequence[str] = ()) -> ctypes.CDLL:
    key = (name, tuple(defines))
    with _lock:
        if key not in _loaded:
            _loaded[key] = ctypes.CDLL(str(library_path(name, defines)))
        return _loaded[key]


def build_all() -> None:
    """Compile every library in its default form (the build check of the package)."""
    for name in LIBRARIES:
        for defines in DEFAULT_SPECIALISATIONS.get(name, [()]):
            library_path(name, defines)
