"""Benchmark file formats and synthetic workloads (no GPU)."""
import struct

import numpy as np
import pytest
import torch

from sparsewave_b200 import formats, workloads as W


def test_csr_binary_header_and_round_trip(tmp_path):
    # test/Benchmark/spmv_benchmark_test.py:166-181
    p = tmp_path / "m.mtx"
    p.write_text("%%MatrixMarket matrix coordinate real general\n2 3 2\n1 2 2\n2 3 3\n")
    m = formats.read_matrix_market(p)
    rp, ci, v = formats.coo_to_csr(m["rows"], m["row_indices"], m["column_indices"], m["values"])
    out = tmp_path / "m.csr"
    formats.write_csr_binary(out, m["rows"], m["columns"], rp, ci, v)
    raw = out.read_bytes()
    assert raw[:8] == b"SWCSR001" and struct.unpack("<QQQ", raw[8:32]) == (2, 3, 2)
    rows, cols, rp2, ci2, v2 = formats.read_csr_binary(out)
    assert (rows, cols) == (2, 3) and rp2.tolist() == [0, 1, 2] and ci2.tolist() == [1, 2] and v2.tolist() == [2, 3]


def test_coo_binary_preserves_duplicates(tmp_path):
    # test/Benchmark/spmv_benchmark_test.py:183-201
    p = tmp_path / "d.mtx"
    p.write_text("%%MatrixMarket matrix coordinate real general\n2 3 3\n1 2 2\n1 2 3\n2 3 4\n")
    m = formats.read_matrix_market(p)
    out = tmp_path / "m.coo"
    formats.write_coo_binary(out, m["rows"], m["columns"], m["row_indices"], m["column_indices"], m["values"])
    raw = out.read_bytes()
    assert raw[:8] == b"SWCOO001" and struct.unpack("<QQQ", raw[8:32]) == (2, 3, 3)
    assert struct.unpack("<3i", raw[32:44]) == (0, 0, 1) and struct.unpack("<3i", raw[44:56]) == (1, 1, 2)


def test_bsr_conversion_known_answers(tmp_path):
    # test/Benchmark/spmm_benchmark_test.py:67-96 (2 x 3 matrix with entries (0,0)=1 (0,2)=2 (1,1)=3)
    bsr = formats.convert_to_bsr(2, 3, [0, 0, 1], [0, 2, 1], [1.0, 2.0, 3.0], 2)
    assert (bsr["rows"], bsr["columns"], bsr["nnzb"]) == (2, 4, 2)
    assert bsr["block_row_offsets"].tolist() == [0, 2] and bsr["block_column_indices"].tolist() == [0, 1]
    assert bsr["block_values"].tolist() == [1, 0, 0, 3, 2, 0, 0, 0]
    assert bsr["block_density"] == 1.0 and bsr["internal_zero_fraction"] == 0.625
    assert bsr["storage_overhead"] == 8.0 / 3.0
    dup = formats.convert_to_bsr(2, 3, [0, 0, 0, 1], [0, 0, 2, 1], [1.0, 4.0, 2.0, 3.0], 2)
    assert dup["block_values"][0] == 5.0 and dup["storage_overhead"] == 8.0 / 3.0
    out = tmp_path / "m.bsr"
    formats.write_bsr_binary(out, bsr)
    assert out.read_bytes()[:8] == b"SWBSR001"
    back = formats.read_bsr_binary(out)
    assert back["block_values"].tolist() == bsr["block_values"].tolist() and back["nnz"] == 3


def test_reference_synthetic_shapes():
    # test/Benchmark/spmv_benchmark_test.py:279-304
    for dist in ("uniform", "alternating", "skewed"):
        m = W.reference_synthetic(16, 64, 8, dist)
        assert m.nnz == 128
    m = W.reference_synthetic(8, 16, 4, "skewed")
    assert m.row_ptr.tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 32]
    assert m.values.tolist() == [1.0] * 32 and m.col_idx.tolist() == [p % 16 for p in range(32)]


def test_algorithmic_bytes():
    assert W.spmv_bytes(4096, 4096, 65536) == 573444
    assert W.spmm_bytes(65536, 65536, 2097152, 4) == 19136516
    assert W.spmm_bytes(2097152, 2097152, 134217728, 64) == 2155872260


def _check_sorted_distinct(a):
    rp, ci, _ = a.numpy()
    for r in range(a.rows):
        row = ci[rp[r]:rp[r + 1]]
        assert np.all(np.diff(row) > 0) and (len(row) == 0 or (row[0] >= 0 and row[-1] < a.cols))


def test_config_generators_small():
    a, x = W.config_c1(rows=256)
    assert a.nnz == 256 * 16 and x.shape == (256,) and float(x.abs().max()) <= 1.0
    _check_sorted_distinct(a)
    a2, _ = W.config_c1(rows=256)
    assert torch.equal(a.col_idx, a2.col_idx) and torch.equal(a.values, a2.values)  # seeded
    a, x = W.config_c3(rows=2000, max_len=500)
    lens = np.diff(a.row_ptr.numpy())
    assert lens.min() >= 1 and lens.max() <= 500 and (lens == 1).mean() > 0.4
    _check_sorted_distinct(a)
    a, B = W.config_c4(rows=3000, n_rhs=8)
    rp, ci, _ = a.numpy()
    c = ci.reshape(-1, 64)
    assert np.all(np.diff(rp) == 64) and np.all((np.abs(c - np.arange(3000)[:, None]) <= 1024).sum(1) >= 32)
    _check_sorted_distinct(a)
    a, B = W.config_c5(block_grid=32, n_rhs=16)
    assert a.block_values.dtype == torch.bfloat16 and B.dtype == torch.bfloat16
    assert a.block_values.numel() == a.nnzb * 256 and 20 < a.nnzb < 90
    brp = a.block_row_ptr.numpy()
    for r in range(32):
        assert np.all(np.diff(a.block_col_idx.numpy()[brp[r]:brp[r + 1]]) > 0)


def test_zipf_mean_matches_distribution():
    lens = W.zipf_lengths(200000, 1.8, 1, 65536, seed=3).numpy()
    k = np.arange(1, 65537, dtype=np.float64)
    w = k ** -1.8
    assert abs((lens == 1).mean() - w[0] / w.sum()) < 0.01
