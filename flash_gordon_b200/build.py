"""Builds the native library in-tree.

    python -m flash_gordon_b200.build            # library + CPU oracle
    python -m flash_gordon_b200.build --verbose  # also print ptxas resource usage

Output: flash_gordon_b200/lib/libfgsampler.so (CUDA kernels for sm_100a only,
C17 host layer, static cudart).  The CPU oracle under oracle/ is test
infrastructure and is built by its own Makefile; it is never linked into the
library.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB = LIB_DIR / "libfgsampler.so"
OBJ_DIR = PKG / "build"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CC = os.environ.get("CC", "gcc")

CUDA_SOURCES = ["fg_stream_kernels.cu", "fg_persistent_kernel.cu", "fg_nucleus_kernel.cu", "fg_ops_kernels.cu",
                "fg_runtime.cu", "fg_nccl.cu"]
HOST_SOURCES = ["fg_util.c", "fg_sampler_host.c", "fg_cuda_api.c", "fg_dist.c", "fg_output_wire.c",
                "fg_request.c", "fg_output_exec.c"]

# sm_100a only; -fmad=false so no fp32/fp64 multiply-add is contracted anywhere
# in the sampling arithmetic (parity with the reference's C code is bit for bit).
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-Xcompiler", "-fPIC", "-I", str(ROOT / "include"), "-I", str(CSRC / "cuda"),
]
CC_FLAGS = [
    "-O2", "-std=c17", "-D_GNU_SOURCE", "-fPIC", "-Wall", "-Wextra", "-ffp-contract=off",
    "-I", str(ROOT / "include"), "-I", str(CSRC / "host"),
]


def _newer(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return False
    stamp = target.stat().st_mtime
    return all(src.stat().st_mtime <= stamp for src in sources)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0 or verbose:
        sys.stderr.write(done.stdout + done.stderr)
    if done.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}")


def build_library(verbose: bool = False, force: bool = False) -> Path:
    headers = list((ROOT / "include").glob("*.h")) + list((CSRC / "cuda").glob("*.h")) + \
        list((CSRC / "cuda").glob("*.cuh")) + list((CSRC / "host").glob("*.h"))
    sources = [CSRC / "cuda" / s for s in CUDA_SOURCES] + [CSRC / "host" / s for s in HOST_SOURCES]
    if not force and LIB.exists() and os.environ.get("FG_USE_PREBUILT") == "1":
        return LIB  # the caller vouches for the library that is there
    if not force and _newer(LIB, sources + headers + [Path(__file__)]):
        return LIB
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    objects = []
    for name in CUDA_SOURCES:
        obj = OBJ_DIR / (name + ".o")
        extra = ["-Xptxas", "-v"] if verbose else []
        _run([NVCC, *NVCC_FLAGS, *extra, "-c", str(CSRC / "cuda" / name), "-o", str(obj)], verbose)
        objects.append(str(obj))
    for name in HOST_SOURCES:
        obj = OBJ_DIR / (name + ".o")
        _run([CC, *CC_FLAGS, "-c", str(CSRC / "host" / name), "-o", str(obj)], verbose)
        objects.append(str(obj))
    # linked beside the target and moved into place, so that nothing ever maps half a library
    fresh = LIB.with_suffix(".so.new")
    _run([NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
          "-Xlinker", "-Bsymbolic", "-o", str(fresh), *objects, "-lpthread", "-lm", "-ldl"], verbose)
    os.replace(fresh, LIB)
    return LIB


def reference_tree() -> Path | None:
    """Where the reference's source tree is mounted: the FG_REFERENCE_TREE variable, else a
    `reference` folder beside this repository.  None when there is none (the GPU box)."""
    named = os.environ.get("FG_REFERENCE_TREE")
    candidates = [Path(named)] if named else [ROOT.parent / "reference"]
    for tree in candidates:
        if (tree / "src" / "sampler.c").exists():
            return tree
    return None


def build_oracle(verbose: bool = False) -> None:
    """The checker: oracle/libfgoracle.so always; oracle/_ref/libfgref.so when the
    reference tree is mounted (elsewhere the prebuilt file is used as is)."""
    _run(["make", "-C", str(ROOT / "oracle"), "libfgoracle.so"], verbose)
    reference = reference_tree()
    if reference is not None:
        _run(["make", "-C", str(ROOT / "oracle"), "reference", f"REFERENCE={reference}"], verbose)
        if LIB.exists():  # the reference's own sampler test, unchanged, against the product library
            _run(["make", "-C", str(ROOT / "oracle"), "drop-in", f"REFERENCE={reference}"], verbose)


if __name__ == "__main__":
    chatty = "--verbose" in sys.argv
    print(build_library(verbose=chatty, force="--force" in sys.argv))
    build_oracle(verbose=chatty)
