"""Builds libsparsewave_b200.so in-tree with nvcc for sm_100a.

`python -m sparsewave_b200.build` compiles every translation unit under
`csrc/` to an object file and links them into
`sparsewave_b200/lib/libsparsewave_b200.so`.  Objects whose sources (and the
headers they include) are older than the object are not recompiled.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = PKG / "lib" / "obj"
LIB = LIBDIR / "libsparsewave_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; libsparsewave_b200.so cannot be built")
    return nvcc


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted((ROOT / "include").glob("*.h"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: Path, verbose: bool, extra: list[str]) -> Path:
    obj = OBJDIR / (src.stem + ".o")
    if _stale(obj, [src, Path(__file__)] + _headers()):
        cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-I", str(ROOT / "include"), "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return obj


def build(verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compiles and links the library; returns its path."""
    OBJDIR.mkdir(parents=True, exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    extra += os.environ.get("SWB_EXTRA_NVCC_FLAGS", "").split()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose, extra), srcs))
    if _stale(LIB, objs):
        # linked under another name and renamed: a reader never sees a half-written library
        fresh = LIB.with_suffix(".so.new")
        cmd = [_nvcc(), "-shared", "-o", str(fresh), *map(str, objs), "-lcudart", "-lcuda"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        os.replace(fresh, LIB)
    build_runner(verbose)
    build_loaders(verbose)
    return LIB


RUNNER_SRC = CSRC / "runner" / "swb_runner.cpp"
RUNNER = LIBDIR / "swb_runner"


def build_runner(verbose: bool = False) -> Path:
    """Native benchmark runner (C++ host program over the C ABI), linked against the library in-tree."""
    if _stale(RUNNER, [RUNNER_SRC, LIB] + _headers()):
        cmd = [_nvcc(), "-O2", "-std=c++17", "-x", "cu", "-gencode", "arch=compute_100a,code=sm_100a",
               str(RUNNER_SRC), "-o", str(RUNNER), "-L", str(LIBDIR), "-lsparsewave_b200",
               "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return RUNNER


LOADER_SRCS = sorted((CSRC / "loaders").glob("*.cpp"))
LOADERS = LIBDIR / "libsparsewave_benchmark_utils.so"


def build_loaders(verbose: bool = False) -> Path:
    """Host-only input loaders and Matrix Market converter (g++; no CUDA): the stand-in for the reference's
    libsparsewave_benchmark_utils.so.  No contraction of a*b+c, so that the expected outputs are the plain
    single-precision loop on every host."""
    LIBDIR.mkdir(parents=True, exist_ok=True)
    if _stale(LOADERS, LOADER_SRCS + [ROOT / "include" / "sparsewave_benchmark_utils.h", Path(__file__)]):
        cmd = [shutil.which("g++") or "g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
               "-ffp-contract=off", *map(str, LOADER_SRCS), "-o", str(LOADERS)]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return LOADERS


if __name__ == "__main__":
    if "--clean" in sys.argv and OBJDIR.exists():
        shutil.rmtree(OBJDIR)
    path = build(verbose=True, ptxas_info="--ptxas-info" in sys.argv)
    print(path)
