"""libsparsewave_benchmark_utils.so on the CPU: the four MLIR C-interface loaders against the reference's own
compiled helper (bit-exact, when it was built) and against the oracle; their fatal diagnostics; the Matrix
Market converter against the Python writers byte for byte."""
import ctypes as C
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import oracle
from sparsewave_b200 import build as swb_build, formats, loaders
from tests.helpers import random_csr

ROOT = Path(__file__).resolve().parents[1]
needs_reference = pytest.mark.skipif(not oracle.reference_available(), reason="reference helper not built")


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "sparsewave_benchmark_utils.h").read_text()
    declared = set(re.findall(r"SWBU_API\s+\w+\s+(\w+)\s*\(", header))
    assert declared == set(loaders.LOADER_SYMBOLS) | {"swbu_convert_matrix_market"}
    lib = C.CDLL(str(swb_build.build_loaders()))
    for name in declared:
        assert getattr(lib, name) is not None


def _csr_case(tmp_path, seed=3):
    rows, cols = 211, 157
    rp, ci, v = random_csr(rows, cols, 7, seed=seed, empty_fraction=0.2)
    path = tmp_path / "m.csr"
    formats.write_csr_binary(path, rows, cols, rp, ci, v)
    return path, rows, cols, rp, ci, v


def test_csr_spmv_loader(tmp_path):
    path, rows, cols, rp, ci, v = _csr_case(tmp_path)
    got = loaders.load_csr_spmv_inputs(path, rows, cols, len(v))
    assert np.array_equal(got[0], rp) and np.array_equal(got[1], ci) and np.array_equal(got[2], v)
    assert np.all(got[3] == 1.0)
    assert np.array_equal(got[4], oracle.csr_spmv(rp, ci, v, np.ones(cols, np.float32)))
    if oracle.reference_available():
        for a, b in zip(got, oracle.reference_csr_spmv(path, rows, cols, len(v))):
            assert np.array_equal(a, b)


def test_spmm_loader(tmp_path):
    path, rows, cols, rp, ci, v = _csr_case(tmp_path, seed=4)
    for n in (1, 4, 9):
        got = loaders.load_spmm_inputs(path, rows, cols, len(v), n)
        k, j = np.meshgrid(np.arange(cols), np.arange(n), indexing="ij")
        assert np.array_equal(got[3], (1.0 + ((k + j) % 7) * 0.125).astype(np.float32))
        assert np.array_equal(got[4], oracle.csr_spmm(rp, ci, v, got[3]))
        if oracle.reference_available():
            for a, b in zip(got, oracle.reference_csr_spmm(path, rows, cols, len(v), n)):
                assert np.array_equal(a, b)


def test_coo_spmv_loader(tmp_path):
    rng = np.random.default_rng(6)
    rows, cols, nnz = 50, 40, 400  # unsorted, with duplicate coordinates
    ri, ci = rng.integers(0, rows, nnz).astype(np.int32), rng.integers(0, cols, nnz).astype(np.int32)
    v = rng.uniform(-1, 1, nnz).astype(np.float32)
    path = tmp_path / "m.coo"
    formats.write_coo_binary(path, rows, cols, ri, ci, v)
    got = loaders.load_coo_spmv_inputs(path, rows, cols, nnz)
    assert np.array_equal(got[4], oracle.coo_spmv(rows, ri, ci, v, np.ones(cols, np.float32)))
    if oracle.reference_available():
        for a, b in zip(got, oracle.reference_coo_spmv(path, rows, cols, nnz)):
            assert np.array_equal(a, b)


def test_bsr_spmm_loader(tmp_path):
    rng = np.random.default_rng(7)
    rows, cols, nnz, bs, n = 45, 38, 300, 4, 5  # dimensions padded to 48 x 40
    ri, ci = rng.integers(0, rows, nnz), rng.integers(0, cols, nnz)
    v = rng.uniform(-1, 1, nnz).astype(np.float32)
    m = formats.convert_to_bsr(rows, cols, ri, ci, v, bs)
    path = tmp_path / "m.bsr"
    formats.write_bsr_binary(path, m)
    got = loaders.load_bsr_spmm_inputs(path, m["rows"], m["columns"], m["nnzb"], bs, n)
    assert np.array_equal(got[0], m["block_row_offsets"]) and np.array_equal(got[2], m["block_values"])
    want = np.zeros((m["rows"], n), np.float32)
    for r, k, val in zip(ri, ci, v):  # the original entries in file order, single precision
        want[r] += val * got[3][k]
    assert np.array_equal(got[4], want)
    # the padded blocks give the same product up to the order of the additions
    assert np.allclose(got[4], oracle.bsr_spmm_f32(got[0], got[1], got[2], got[3], bs), rtol=1e-5, atol=1e-5)
    if oracle.reference_available():
        for a, b in zip(got, oracle.reference_bsr_spmm(path, m["rows"], m["columns"], m["nnzb"], bs, n)):
            assert np.array_equal(a, b)


_CHILD = """
import sys, numpy as np
from sparsewave_b200 import loaders
kind, path, rows, cols, nnz = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5])
if kind == "unset":
    import os
    os.environ.pop("SPARSEWAVE_BENCHMARK_CSR", None)
    a = [np.empty(1, np.int32), np.empty(0, np.int32), np.empty(0, np.float32), np.empty(0, np.float32), np.empty(0, np.float32)]
    import ctypes as C
    d = [loaders.memref(x) for x in a]
    loaders.load()._mlir_ciface_loadCSRSpMVBenchmarkInputs(*[C.byref(m) for m in d])
else:
    loaders.load_csr_spmv_inputs(path, rows, cols, nnz)
"""


def _abort_message(*args):
    p = subprocess.run([sys.executable, "-c", _CHILD, *map(str, args)], capture_output=True, text=True, cwd=ROOT)
    assert p.returncode == -6, (p.returncode, p.stderr)  # SIGABRT, like the reference helper
    return p.stderr


def test_loader_failures_abort_with_the_reference_diagnostics(tmp_path):
    path, rows, cols, rp, ci, v = _csr_case(tmp_path)
    assert "SparseWave benchmark input error: SPARSEWAVE_BENCHMARK_CSR is not set" in _abort_message("unset", "-", 0, 0, 0)
    assert "could not open" in _abort_message("csr", tmp_path / "missing.csr", rows, cols, len(v))
    bad = tmp_path / "bad.csr"
    bad.write_bytes(b"SWCOO001" + path.read_bytes()[8:])
    assert "invalid CSR binary header" in _abort_message("csr", bad, rows, cols, len(v))
    cut = tmp_path / "cut.csr"
    cut.write_bytes(path.read_bytes()[:-10])
    assert "could not read values" in _abort_message("csr", cut, rows, cols, len(v))
    assert "row offsets memref has an unexpected layout" in _abort_message("csr", path, rows + 1, cols, len(v))
    assert "vector memref has an unexpected layout" in _abort_message("csr", path, rows, cols + 1, len(v))


MTX_GENERAL = """%%MatrixMarket matrix coordinate real general
% a comment

5 4 7
1 1 1.5
3 2 -2.25
3 2 0.75
5 4 1e-3
2 3 4
1 4 7.0
4 1 -1
"""
MTX_SYMMETRIC = """%%MatrixMarket matrix coordinate integer symmetric
4 4 4
1 1 2
3 1 5
4 2 -3
4 4 9
"""
MTX_PATTERN = "%%MatrixMarket matrix coordinate pattern general\n3 5 3\n1 5\n3 1\n2 2\n"


@pytest.mark.parametrize("text", [MTX_GENERAL, MTX_SYMMETRIC, MTX_PATTERN])
def test_matrix_market_conversion_matches_the_python_writers(tmp_path, text):
    mtx = tmp_path / "m.mtx"
    mtx.write_text(text)
    m = formats.read_matrix_market(mtx)
    rows, cols = m["rows"], m["columns"]
    ri, ci, v = m["row_indices"], m["column_indices"], m["values"]
    formats.write_coo_binary(tmp_path / "py.coo", rows, cols, ri, ci, v)
    rp, cc, vv = formats.coo_to_csr(rows, ri, ci, v)
    formats.write_csr_binary(tmp_path / "py.csr", rows, cols, rp, cc, vv)
    formats.write_bsr_binary(tmp_path / "py.bsr", formats.convert_to_bsr(rows, cols, ri, ci, m["values64"], 2))
    for fmt in ("coo", "csr", "bsr"):
        loaders.convert_matrix_market(mtx, fmt, tmp_path / f"cpp.{fmt}", block_size=2)
        assert (tmp_path / f"cpp.{fmt}").read_bytes() == (tmp_path / f"py.{fmt}").read_bytes(), fmt


def _matrix_market_golden():
    import json
    return json.loads((Path(__file__).parent / "golden" / "matrix_market_cases.json").read_text())


@pytest.mark.parametrize("name", sorted(_matrix_market_golden()["cases"]))
def test_matrix_market_conversion_matches_the_reference_converter(tmp_path, name):
    """tests/golden/matrix_market_cases.json holds what the SparseWave tree's own converter
    (benchmark/benchmark_utils.py) makes of each file: the bytes of the three binary formats - entries ordered by
    (row, column) whatever the file order, duplicates summed in that order - or its error text.  The C++
    converter and the Python reader reproduce both."""
    golden = _matrix_market_golden()
    case, bs = golden["cases"][name], golden["block_size"]
    mtx = tmp_path / "m.mtx"
    mtx.write_text(case["text"])
    if "error" in case:
        message = case["error"].replace("<path>", str(mtx))
        with pytest.raises(ValueError) as cpp:
            loaders.convert_matrix_market(mtx, "csr", tmp_path / "o.csr")
        assert str(cpp.value) == message
        with pytest.raises(ValueError) as py:
            formats.read_matrix_market(mtx)
        assert str(py.value) == message
        return
    for fmt in ("csr", "coo", "bsr"):
        loaders.convert_matrix_market(mtx, fmt, tmp_path / f"o.{fmt}", block_size=bs)
        assert (tmp_path / f"o.{fmt}").read_bytes().hex() == case[fmt], fmt
    m = formats.read_matrix_market(mtx)
    formats.write_coo_binary(tmp_path / "py.coo", m["rows"], m["columns"], m["row_indices"], m["column_indices"], m["values"])
    formats.write_bsr_binary(tmp_path / "py.bsr", formats.convert_to_bsr(m["rows"], m["columns"], m["row_indices"],
                                                                       m["column_indices"], m["values64"], bs))
    assert (tmp_path / "py.coo").read_bytes().hex() == case["coo"]
    assert (tmp_path / "py.bsr").read_bytes().hex() == case["bsr"]


def test_matrix_market_errors(tmp_path):
    mtx = tmp_path / "m.mtx"
    cases = {
        "%%MatrixMarket matrix coordinate real hermitian\n1 1 1\n1 1 1\n": "unsupported Matrix Market symmetry 'hermitian'",
        "%%MatrixMarket matrix coordinate real general\n2 2 2\n1 1 1.0\n": "header declares 2 entries, but the file contains 1",
        "hello\n": "expected a Matrix Market coordinate matrix",
    }
    for text, message in cases.items():
        mtx.write_text(text)
        with pytest.raises(ValueError, match=message):
            loaders.convert_matrix_market(mtx, "csr", tmp_path / "o.csr")
    mtx.write_text(MTX_GENERAL)
    with pytest.raises(ValueError, match="block size must be positive"):
        loaders.convert_matrix_market(mtx, "bsr", tmp_path / "o.bsr", block_size=0)
    with pytest.raises(ValueError, match="csr, coo or bsr"):
        loaders.convert_matrix_market(mtx, "ell", tmp_path / "o.ell")
    with pytest.raises(ValueError, match="could not open"):
        loaders.convert_matrix_market(tmp_path / "none.mtx", "csr", tmp_path / "o.csr")
