#!/usr/bin/env python3
"""Builds the reference engine's CUDA path, unmodified, for the bench's reference arm.

    python baseline/build_reference.py [--reference /path/to/checkout]

The reference (BusyaPrime/from-scratch-inference-engine-) builds with CMake, which fetches
Eigen, nlohmann/json and GoogleTest from the network; none of that is reachable offline.  Its
GPU engine itself needs only nvcc and cuBLAS.  This script therefore

  1. copies the reference's `include/` and `src/` trees as they are into
     `baseline/_ref/reference/` (when a checkout is given or found; the copy is what travels
     to a GPU machine, where the checkout itself may not exist);
  2. compiles, with nvcc for sm_100a and against the toolkit's cuBLAS, the five files of
     `src/cuda/` and the CPU sources they link against (configuration, safetensors reader,
     sampler, the CPU model and cache they share types with), together with
     `baseline/ref_bench.cpp`, into `baseline/_ref/bin/ref_bench`.

Include path only: the `nlohmann/json.hpp` that ships inside the Python environment, and
the small stand-in for `<Eigen/Dense>` under tests/golden/eigen_standin (the CPU matrix
product of `src/model/nn.cpp` is the one expression that goes through it; the GPU path
never calls it).  No reference file is edited.  `baseline/_ref/` is not part of the
repository's history.
"""

from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
REF_COPY = HERE / "_ref" / "reference"
BINARY = HERE / "_ref" / "bin" / "ref_bench"
STAMP = HERE / "_ref" / "bin" / "ref_bench.sources"

CUDA_SOURCES = ["src/cuda/device.cu", "src/cuda/model.cu", "src/cuda/kv_cache.cu",
                "src/cuda/engine.cu", "src/cuda/block_manager.cu"]
CPU_SOURCES = ["src/model/model_config.cpp", "src/model/safetensors.cpp", "src/model/nn.cpp",
               "src/model/model.cpp", "src/kvcache/block_manager.cpp",
               "src/kvcache/paged_kv_cache.cpp", "src/sampler/sampler.cpp",
               "src/engine/engine.cpp", "src/quant/quant.cpp"]


def find_json_header() -> Path:
    for root in (Path(sysconfig.get_paths()["purelib"]), Path(sys.prefix)):
        for hit in root.rglob("nlohmann/json.hpp"):
            return hit.parent.parent
    raise SystemExit("build_reference: nlohmann/json.hpp not found in the Python environment")


def copy_reference(checkout: Path) -> None:
    for tree in ("include", "src", "benchmarks/harness"):
        target = REF_COPY / tree
        if target.exists():
            shutil.rmtree(target)
        shutil.copytree(checkout / tree, target)
    for name in ("LICENSE", "CMakeLists.txt", "README.md"):
        if (checkout / name).exists():
            shutil.copy2(checkout / name, REF_COPY / name)


def sources_digest(files) -> str:
    digest = hashlib.sha256()
    for path in files:
        digest.update(str(path.name).encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def build(checkout: Path | None = None, verbose: bool = True) -> Path:
    """Returns the path of the built binary (built only when sources changed)."""
    if checkout is None:
        # a checkout named `reference` beside this repository, or the one FSIE_REFERENCE names
        for candidate in (os.environ.get("FSIE_REFERENCE"), ROOT.parent / "reference"):
            if candidate and (Path(candidate) / "src/cuda/model.cu").exists():
                checkout = Path(candidate)
                break
    if checkout is not None and (checkout / "src/cuda/model.cu").exists():
        REF_COPY.mkdir(parents=True, exist_ok=True)
        copy_reference(checkout)
    if not (REF_COPY / "src/cuda/model.cu").exists():
        raise SystemExit("build_reference: no copy of the reference under baseline/_ref/reference "
                         "and no checkout given (--reference)")
    present = [s for s in CPU_SOURCES if (REF_COPY / s).exists()]
    files = [REF_COPY / s for s in CUDA_SOURCES + present] + [HERE / "ref_bench.cpp"]
    headers = sorted((REF_COPY / "include").rglob("*.hpp"))
    digest = sources_digest(files + headers)
    if BINARY.exists() and STAMP.exists() and STAMP.read_text().strip() == digest:
        return BINARY
    BINARY.parent.mkdir(parents=True, exist_ok=True)
    cmd = ["nvcc", "-std=c++20", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-DENGINE_WITH_CUDA=1",
           f"-I{REF_COPY / 'include'}", f"-I{ROOT / 'tests' / 'golden' / 'eigen_standin'}",
           f"-I{find_json_header()}", *map(str, files), "-lcublas", "-o", str(BINARY)]
    if verbose:
        print("build_reference:", " ".join(cmd), file=sys.stderr, flush=True)
    subprocess.run(cmd, check=True)
    STAMP.write_text(digest + "\n")
    return BINARY


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--reference", default=None, help="checkout of the reference project")
    args = parser.parse_args()
    print(build(Path(args.reference) if args.reference else None))


if __name__ == "__main__":
    main()
