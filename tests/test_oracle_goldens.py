"""The oracle against every runtime golden vector the reference's tests hold
for the SpMV / SpMM / BSR-SpMM path, against the reference's own CPU loops
(compiled from benchmark/SparseBenchmarkUtils.cpp when available) and against
committed outputs of those loops (tests/golden/)."""
from pathlib import Path

import numpy as np
import pytest

import oracle
from sparsewave_b200 import formats
from tests.helpers import (BSR_GOLDEN, COO_GOLDEN, SPMM_GOLDEN, SPMM_GOLDEN_TORCH, SPMV_GOLDEN, SPMV_GOLDEN_4X4, random_csr)

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("g", [SPMV_GOLDEN, SPMV_GOLDEN_4X4])
def test_spmv_golden(g):
    y = oracle.csr_spmv(g["row_ptr"], g["col"], g["val"], g["x"])
    assert y.tolist() == g["y"]
    for kw in (dict(chunk=1), dict(chunk=4), dict(chunk=4, segmented=True)):
        assert oracle.spmv_thread_position(g["row_ptr"], g["col"], g["val"], g["x"], **kw).tolist() == g["y"]
    for batch in (1, 2):
        assert oracle.spmv_wave_position(g["row_ptr"], g["col"], g["val"], g["x"], block=128,
                                         batch=batch).tolist() == g["y"]


@pytest.mark.parametrize("g", [SPMM_GOLDEN, SPMM_GOLDEN_TORCH])
def test_spmm_golden(g):
    B = np.array(g["B"], np.float32)
    assert oracle.csr_spmm(g["row_ptr"], g["col"], g["val"], B).tolist() == g["C"]
    assert oracle.spmm_thread_position(g["row_ptr"], g["col"], g["val"], B, chunk=4).tolist() == g["C"]


def test_coo_golden():
    g = COO_GOLDEN
    assert oracle.coo_spmv(g["rows"], g["row"], g["col"], g["val"], g["x"]).tolist() == g["y"]


def test_bsr_golden():
    g = BSR_GOLDEN
    B = np.array(g["B"], np.float32)
    assert oracle.bsr_spmm_f32(g["brp"], g["bci"], g["bv"], B, g["bs"]).tolist() == g["C"]


def test_bsr_bf16_matches_f32_on_exact_inputs():
    import torch
    g = BSR_GOLDEN
    bv = torch.tensor(g["bv"], dtype=torch.bfloat16).view(torch.uint16).numpy()
    B = torch.tensor(g["B"], dtype=torch.bfloat16).view(torch.uint16).numpy()
    bits, f32 = oracle.bsr_spmm_bf16(g["brp"], g["bci"], bv, B, g["bs"])
    assert f32.tolist() == g["C"]
    back = torch.from_numpy(bits.copy()).view(torch.bfloat16).float().numpy()
    assert back.tolist() == [[17, 170], [45, 450], [7, 70], [16, 160]]


def test_index_known_answers():
    # test/Dialect/SparseWave/position-space-lowering.mlir:200-222, 226-243, 245-260, 343-356
    assert oracle.partition(10, 17, 1, 3) == (13, 15)
    assert oracle.chunk_bounds(5, 15, 2, 4) == (13, 15)
    b, e = oracle.chunk_bounds(0, 10, 3, 4)
    assert b == e
    assert oracle.partition(0, 3, 4, 5) == (3, 3)


def test_row_search_skips_empty_rows():
    rp = [0, 2, 2, 3, 5, 6]
    assert [oracle.row_at_position(rp, p) for p in range(6)] == [0, 0, 2, 3, 3, 4]
    rp = [0, 0, 0, 1, 1, 4, 4]
    assert [oracle.row_at_position(rp, p) for p in range(4)] == [2, 4, 4, 4]


def test_parallel_loops_equal_serial():
    rp, ci, v = random_csr(3000, 500, 9, seed=3)
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, 500).astype(np.float32)
    B = rng.uniform(-1, 1, (500, 5)).astype(np.float32)
    assert np.array_equal(oracle.csr_spmv(rp, ci, v, x), oracle.csr_spmv(rp, ci, v, x, parallel=True))
    assert np.array_equal(oracle.csr_spmm(rp, ci, v, B), oracle.csr_spmm(rp, ci, v, B, parallel=True))


def _ref_inputs():
    rp, ci, v = random_csr(257, 193, 7, seed=11)
    return 257, 193, rp, ci, v


@pytest.mark.skipif(not oracle.reference_available(), reason="reference CPU helper not built")
def test_against_reference_cpu_loops(tmp_path):
    rows, cols, rp, ci, v = _ref_inputs()
    path = tmp_path / "m.csr"
    formats.write_csr_binary(path, rows, cols, rp, ci, v)
    r_rp, r_ci, r_v, x, expected = oracle.reference_csr_spmv(path, rows, cols, len(v))
    assert np.array_equal(r_rp, rp) and np.array_equal(r_ci, ci) and np.array_equal(r_v, v)
    assert np.array_equal(x, np.ones(cols, np.float32))
    assert np.array_equal(oracle.csr_spmv(rp, ci, v, x), expected)
    for n in (1, 4, 7):
        _, _, _, B, expected = oracle.reference_csr_spmm(path, rows, cols, len(v), n)
        assert np.array_equal(oracle.csr_spmm(rp, ci, v, B), expected)


@pytest.mark.skipif(not oracle.reference_available(), reason="reference CPU helper not built")
def test_bsr_against_reference_cpu_loops(tmp_path):
    # Integer-valued entries keep every partial sum exact, so the reference's
    # COO-ordered accumulation and the block-ordered one agree bit for bit.
    rng = np.random.default_rng(5)
    rows, cols, nnz = 37, 29, 300
    ri, cj = rng.integers(0, rows, nnz), rng.integers(0, cols, nnz)
    va = rng.integers(-4, 5, nnz).astype(np.float32)
    for bs in (2, 4, 8):
        m = formats.convert_to_bsr(rows, cols, ri, cj, va, bs)
        path = tmp_path / f"m{bs}.bsr"
        formats.write_bsr_binary(path, m)
        brp, bci, bv, B, expected = oracle.reference_bsr_spmm(path, m["rows"], m["columns"], m["nnzb"], bs, 3)
        assert np.array_equal(brp, m["block_row_offsets"]) and np.array_equal(bci, m["block_column_indices"])
        assert np.array_equal(oracle.bsr_spmm_f32(brp, bci, bv, B, bs), expected)


def test_against_committed_reference_outputs():
    """tests/golden/reference_cpu.npz holds outputs of the reference's own CPU
    loops (made by tests/golden/make_golden.py where the reference was built)."""
    z = np.load(GOLDEN / "reference_cpu.npz")
    rp, ci, v = z["row_ptr"], z["col"], z["val"]
    assert np.array_equal(oracle.csr_spmv(rp, ci, v, z["spmv_x"]), z["spmv_expected"])
    for n in (1, 4, 7):
        assert np.array_equal(oracle.csr_spmm(rp, ci, v, z[f"spmm{n}_B"]), z[f"spmm{n}_expected"])
    assert np.array_equal(oracle.bsr_spmm_f32(z["bsr_brp"], z["bsr_bci"], z["bsr_bv"], z["bsr_B"], 4),
                          z["bsr_expected"])


def test_mismatch_counters():
    e = np.array([0.0, 1.0, 100.0, -3.0], np.float32)
    a = e + np.array([5e-5, 2e-4, 5e-3, 0], np.float32)
    assert oracle.count_mismatches_reference(a, e) == 1
    assert oracle.count_mismatches_bound(a, e, np.array([10.0, 10.0, 1000.0, 1.0]), rel=1e-5) == 1


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_against_scipy_in_float64(seed):
    """An independent restatement: scipy.sparse in float64 on random ragged matrices.  The f32 loops of the
    oracle (sequential, schedules of the position mappings, BSR) must lie within 1e-5 * sum|a b| of it."""
    sp = pytest.importorskip("scipy.sparse")
    rp, ci, v = random_csr(300, 257, 12, seed=seed, empty_fraction=0.2)
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1, 1, 257).astype(np.float32)
    B = rng.uniform(-1, 1, (257, 9)).astype(np.float32)
    A = sp.csr_matrix((v.astype(np.float64), ci, rp), shape=(300, 257))
    absA = sp.csr_matrix((np.abs(v).astype(np.float64), ci, rp), shape=(300, 257))
    want_y, bound_y = A @ x.astype(np.float64), absA @ np.abs(x).astype(np.float64)
    for got in (oracle.csr_spmv(rp, ci, v, x), oracle.spmv_thread_position(rp, ci, v, x, chunk=8, segmented=True),
                oracle.spmv_wave_position(rp, ci, v, x, block=64, batch=2)):
        assert np.all(np.abs(got - want_y) <= 1e-5 * bound_y + 1e-30)
    assert np.allclose(oracle.csr_abs_bound(rp, ci, v, x), bound_y, rtol=1e-5, atol=1e-30)
    want_C, bound_C = A @ B.astype(np.float64), absA @ np.abs(B).astype(np.float64)
    for got in (oracle.csr_spmm(rp, ci, v, B), oracle.spmm_thread_position(rp, ci, v, B, chunk=4)):
        assert np.all(np.abs(got - want_C) <= 1e-5 * bound_C + 1e-30)
    # BSR: 7 x 6 grid of 4 x 4 blocks, one block row empty
    present = rng.random((7, 6)) < 0.4
    present[3] = False
    brp = np.zeros(8, np.int32)
    brp[1:] = np.cumsum(present.sum(1))
    bci = np.concatenate([np.nonzero(r)[0] for r in present]).astype(np.int32)
    bv = rng.uniform(-1, 1, (len(bci), 4, 4)).astype(np.float32)
    Bb = rng.uniform(-1, 1, (24, 5)).astype(np.float32)
    M = sp.bsr_matrix((bv.astype(np.float64), bci, brp), shape=(28, 24))
    absM = sp.bsr_matrix((np.abs(bv).astype(np.float64), bci, brp), shape=(28, 24))
    got = oracle.bsr_spmm_f32(brp, bci, bv.reshape(-1), Bb, 4)
    assert np.all(np.abs(got - M @ Bb.astype(np.float64)) <= 1e-5 * (absM @ np.abs(Bb).astype(np.float64)) + 1e-30)
