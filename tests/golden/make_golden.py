"""Writes tests/golden/reference_cpu.npz: outputs of the SparseWave reference's
own CPU loops (benchmark/SparseBenchmarkUtils.cpp, compiled unmodified by
oracle/build.py) on small seeded inputs.  Run where the reference tree is
present: `python tests/golden/make_golden.py`."""
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402
from sparsewave_b200 import formats  # noqa: E402
from tests.helpers import random_csr  # noqa: E402


def main():
    out = {}
    rows, cols = 257, 193
    rp, ci, v = random_csr(rows, cols, 7, seed=11)
    with tempfile.TemporaryDirectory() as d:
        path = Path(d) / "m.csr"
        formats.write_csr_binary(path, rows, cols, rp, ci, v)
        _, _, _, x, y = oracle.reference_csr_spmv(path, rows, cols, len(v))
        out.update(row_ptr=rp, col=ci, val=v, spmv_x=x, spmv_expected=y)
        for n in (1, 4, 7):
            _, _, _, B, C = oracle.reference_csr_spmm(path, rows, cols, len(v), n)
            out[f"spmm{n}_B"], out[f"spmm{n}_expected"] = B, C
        rng = np.random.default_rng(5)
        ri, cj = rng.integers(0, 37, 300), rng.integers(0, 29, 300)
        va = rng.integers(-4, 5, 300).astype(np.float32)
        m = formats.convert_to_bsr(37, 29, ri, cj, va, 4)
        bpath = Path(d) / "m.bsr"
        formats.write_bsr_binary(bpath, m)
        brp, bci, bv, B, C = oracle.reference_bsr_spmm(bpath, m["rows"], m["columns"], m["nnzb"], 4, 3)
        out.update(bsr_brp=brp, bsr_bci=bci, bsr_bv=bv, bsr_B=B, bsr_expected=C)
    np.savez_compressed(Path(__file__).resolve().parent / "reference_cpu.npz", **out)
    print("wrote reference_cpu.npz", {k: a.shape for k, a in out.items()})


if __name__ == "__main__":
    main()
