"""Builds the test oracle.

`python oracle/build.py` compiles oracle/swb_oracle.c (the CPU restatement) to
oracle/liboracle.so and, when the SparseWave reference tree is present,
compiles the reference's own benchmark/SparseBenchmarkUtils.cpp -- from where
it lies, unmodified, against the one-struct stand-in header in
oracle/ref_stub/ -- to oracle/_ref/libsparsewave_benchmark_utils.so.  Both are
checkers for tests and for the CPU-baseline legs of the benchmark; the product
library never loads them.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ORACLE_SRC = HERE / "swb_oracle.c"
ORACLE_LIB = HERE / "liboracle.so"
REF_DIR = HERE / "_ref"
REF_LIB = REF_DIR / "libsparsewave_benchmark_utils.so"
REF_FLAGS = ["-O2", "-ffp-contract=off", "-std=c++17", "-shared", "-fPIC"]


def reference_root() -> Path | None:
    """The SparseWave source tree: $SPARSEWAVE_REFERENCE, else a `reference` directory beside this
    repository; None when neither holds the helper's source (the reference build is then skipped)."""
    named = os.environ.get("SPARSEWAVE_REFERENCE")
    for root in ([Path(named)] if named else []) + [HERE.parent.parent / "reference"]:
        if (root / "benchmark" / "SparseBenchmarkUtils.cpp").exists():
            return root
    return None


def _stale(target: Path, deps: list[Path]) -> bool:
    return not target.exists() or any(d.stat().st_mtime > target.stat().st_mtime for d in deps)


def build_oracle(verbose: bool = False) -> Path:
    if _stale(ORACLE_LIB, [ORACLE_SRC, Path(__file__)]):
        cmd = ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-fvisibility=hidden",
               str(ORACLE_SRC), "-o", str(ORACLE_LIB), "-lm"]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
    return ORACLE_LIB


def build_reference(verbose: bool = False) -> Path | None:
    """Compiles the reference's CPU helper where it lies; None when the tree is absent."""
    root = reference_root()
    if root is None:
        return REF_LIB if REF_LIB.exists() else None
    src = root / "benchmark" / "SparseBenchmarkUtils.cpp"
    REF_DIR.mkdir(exist_ok=True)
    if _stale(REF_LIB, [src, HERE / "ref_stub" / "mlir" / "ExecutionEngine" / "CRunnerUtils.h"]):
        cmd = ["g++", *REF_FLAGS, "-I", str(HERE / "ref_stub"), str(src), "-o", str(REF_LIB)]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
    return REF_LIB


if __name__ == "__main__":
    print(build_oracle(verbose=True))
    print(build_reference(verbose=True))
