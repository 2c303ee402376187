"""Host side of the C ABI, no GPU needed: the library loads and exports every
declared symbol, option parsing / validation reproduce the reference's
diagnostics, index helpers match the oracle and the reference's folded
answers, launch geometry follows the reference's grid arithmetic."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import oracle
import sparsewave_b200 as swb
from sparsewave_b200 import _lib, api

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "sparsewave_b200.h").read_text()
    declared = set(re.findall(r"SWB_API\s+[\w\s\*]+?\b(\w+)\s*\(", header))
    assert len(declared) >= 25
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert b"sm_100a" in lib.swb_version()


def test_defaults_follow_the_reference():
    o = swb.make_options()
    assert (o.mapping, o.block_size, o.wave_size, o.position_block_size, o.position_chunk_size) == (0, 256, 32, 256, 1)
    assert (o.spmm_mapping, o.spmm_block_size, o.spmm_tile_size, o.position_reduction) == (0, 256, 4, 0)


def test_parse_both_spellings():
    o = swb.make_options("spmv-mapping=wave-per-position spmv-block-size=128 wavefront-size=32")
    assert (o.mapping, o.block_size) == (2, 128)
    o = swb.make_options("mapping=block-per-row block-size=64, spmm-mapping=wave-per-row-tile spmm-tile-size=8")
    assert (o.mapping, o.block_size, o.spmm_mapping, o.spmm_tile_size) == (4, 64, 1, 8)
    o = swb.make_options("mapping=thread thread-chunk-size=4 thread-reduction=segmented")
    assert (o.mapping, o.position_chunk_size, o.position_reduction) == (1, 4, 1)
    o = swb.make_options("sddmm-block-size=64 elementwise-block-size=32")  # foreign keys are accepted
    assert o.block_size == 256


# (option text, expected diagnostic) -- test/Dialect/SparseWave/invalid-lowering-options.mlir:92-116
INVALID = [
    ("mapping=unknown", "unsupported SpMV mapping strategy 'unknown'; expected 'thread-per-row', 'wave-per-row', or 'block-per-row'"),
    ("block-size=0", "SpMV block size must be between 1 and 1024, but got 0"),
    ("block-size=1025", "SpMV block size must be between 1 and 1024, but got 1025"),
    ("mapping=wave-per-row wave-size=64", "wave-per-row currently requires Wave32, but got wave size 64"),
    ("mapping=wave-per-row block-size=48", "wave-per-row requires the SpMV block size to be a multiple of 32, but got 48"),
    ("mapping=block", "unsupported position mapping 'block'; expected 'thread' or 'wave'"),
    ("mapping=thread block-size=0", "position block size must be between 1 and 1024, but got 0"),
    ("mapping=wave wave-size=64", "wave position mapping currently requires Wave32, but got 64"),
    ("mapping=wave block-size=48", "wave position mapping requires the block size to be a multiple of 32, but got 48"),
    ("mapping=thread thread-chunk-size=0", "thread position chunk size must be positive, but got 0"),
    ("mapping=wave thread-chunk-size=2", "thread position chunk size applies only to thread mapping"),
    ("thread-reduction=tree", "unsupported thread position reduction 'tree'; expected 'atomic' or 'segmented'"),
    ("mapping=wave thread-reduction=segmented", "thread position reduction applies only to thread mapping"),
    ("mapping=block-per-row wave-size=64", "block-per-row currently requires Wave32, but got wave size 64"),
    ("mapping=block-per-row block-size=48", "block-per-row requires the SpMV block size to be a multiple of 32, but got 48"),
    ("spmm-mapping=unknown", "unsupported SpMM mapping strategy 'unknown'; expected 'thread-per-output' or 'wave-per-row-tile'"),
    ("spmm-block-size=0", "SpMM block size must be between 1 and 1024, but got 0"),
    ("spmm-block-size=1025", "SpMM block size must be between 1 and 1024, but got 1025"),
    ("spmm-tile-size=0", "SpMM tile size must be between 1 and 32, but got 0"),
    ("spmm-tile-size=33", "SpMM tile size must be between 1 and 32, but got 33"),
    ("spmm-mapping=wave-per-row-tile wave-size=64", "wave-per-row-tile currently requires Wave32, but got wave size 64"),
    ("spmm-mapping=wave-per-row-tile spmm-block-size=48", "wave-per-row-tile requires the SpMM block size to be a multiple of 32, but got 48"),
    ("sddmm-block-size=0", "SDDMM block size must be between 1 and 1024, but got 0"),
    ("row-reduction-block-size=1025", "CSR row-reduction block size must be between 1 and 1024, but got 1025"),
    ("rowwise-map-block-size=0", "CSR row-wise map block size must be between 1 and 1024, but got 0"),
    ("elementwise-block-size=1025", "elementwise block size must be between 1 and 1024, but got 1025"),
    # test/Dialect/SparseWave/position-parallel-invalid-lowering-options.mlir:14
    ("position-block-size=0", "position-parallel block size must be between 1 and 1024, but got 0"),
    ("position-block-size=1025", "position-parallel block size must be between 1 and 1024, but got 1025"),
]


@pytest.mark.parametrize("text,message", INVALID)
def test_invalid_options(text, message):
    with pytest.raises(swb.SparseWaveError) as e:
        swb.validate_options(swb.make_options(text))
    assert message in str(e.value)
    assert e.value.status == _lib.SWB_ERR_INVALID_OPTION


def test_unknown_key_and_bad_value():
    with pytest.raises(swb.SparseWaveError, match="unknown option 'frobnicate'"):
        swb.make_options("frobnicate=1")
    with pytest.raises(swb.SparseWaveError, match="expects an integer"):
        swb.make_options("block-size=abc")


def test_index_helpers_match_oracle_and_folded_answers():
    assert swb.partition(10, 17, 1, 3) == (13, 15)
    assert swb.chunk_bounds(5, 15, 2, 4) == (13, 15)
    assert swb.chunk_bounds(0, 10, 3, 4)[0] == swb.chunk_bounds(0, 10, 3, 4)[1]
    assert swb.partition(0, 3, 4, 5) == (3, 3)
    rng = np.random.default_rng(0)
    for _ in range(300):
        lo = int(rng.integers(0, 50)); hi = lo + int(rng.integers(0, 5000))
        count = int(rng.integers(1, 200)); w = int(rng.integers(0, count))
        assert swb.partition(lo, hi, w, count) == oracle.partition(lo, hi, w, count)
        f = int(rng.integers(1, 64)); w2 = int(rng.integers(0, 300))
        b, e = swb.chunk_bounds(lo, hi, w2, f)
        ob, oe = oracle.chunk_bounds(lo, hi, w2, f)
        assert (e - b, b if e > b else 0) == (oe - ob, ob if oe > ob else 0)
    # partitions tile the range in order
    edges = [swb.partition(3, 1003, w, 37) for w in range(37)]
    assert edges[0][0] == 3 and edges[-1][1] == 1003
    assert all(edges[i][1] == edges[i + 1][0] for i in range(36))


def test_row_search_matches_oracle_with_empty_rows():
    rng = np.random.default_rng(1)
    lens = rng.integers(0, 4, 500) * (rng.random(500) < 0.6)
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    for p in range(int(rp[-1])):
        r = swb.row_at_position(rp, p)
        assert r == oracle.row_at_position(rp, p)
        assert rp[r] <= p < rp[r + 1]


def test_launch_shapes_follow_reference_grid_arithmetic():
    # SparseGPUUtils.cpp:11-59, SparseWaveToGPU.cpp:380, SparsePositionScheduling.cpp:340-350
    s = swb.launch_shape("mapping=thread-per-row block-size=128", rows=4096, nnz=65536)
    assert (s.logical_grid, s.logical_block, s.kernels) == (32, 128, 1)
    s = swb.launch_shape("mapping=wave-per-row block-size=128", rows=4096, nnz=65536)
    assert (s.logical_grid, s.work_units) == (1024, 4096)
    s = swb.launch_shape("mapping=block-per-row block-size=64", rows=4096, nnz=65536)
    assert s.logical_grid == 4096
    s = swb.launch_shape("mapping=thread-per-position block-size=256 thread-chunk-size=8", rows=10, nnz=65537)
    assert (s.work_units, s.logical_grid, s.kernels) == (8193, 33, 2)
    s = swb.launch_shape("mapping=wave-per-position block-size=128", rows=5, nnz=6)
    assert (s.logical_grid, s.work_units, s.kernels) == (1, 4, 2)
    s = swb.launch_shape("mapping=wave-per-row", rows=0, nnz=0)
    assert s.logical_grid == 1  # the grid clamps to one inactive block
    # C2: 65536 rows, N = 4, tile 4, block 64 -> 65536 units, 32768 blocks
    s = swb.launch_shape("spmm-mapping=wave-per-row-tile spmm-tile-size=4 spmm-block-size=64", 65536, 2097152, 4)
    assert (s.work_units, s.logical_grid) == (65536, 32768)
    assert s.physical_grid == 8192  # 32 nnz per row: 8 lanes per row, 4 rows per warp, 2 warps per block
    s = swb.launch_shape("spmm-mapping=wave-per-row-tile spmm-tile-size=16 spmm-block-size=256", 2097152, 134217728, 64)
    assert (s.work_units, s.logical_grid, s.physical_grid) == (4 * 2097152, 1048576, 262144)  # tiles of a row fused
    s = swb.launch_shape("spmm-mapping=thread-per-output spmm-block-size=64", 65536, 2097152, 4)
    assert s.logical_grid == 4096
    s = swb.launch_shape("spmm-mapping=wave-per-row-tile spmm-tile-size=16 spmm-block-size=64", 100, 1000, 70)
    assert s.work_units == 500 and s.physical_grid == s.logical_grid == 250  # ceil(70 / 16) = 5 tiles per row
    # lanes per matrix row follow the mean row length: N = 64 with 5 per row takes half a warp per row (two rows
    # per warp, 8 warps per block), with 13 per row the whole warp; N = 16 with 24 per row takes 8 lanes
    s = swb.launch_shape("spmm-mapping=wave-per-row-tile spmm-tile-size=16 spmm-block-size=256", 1 << 20, 5 << 20, 64)
    assert s.physical_grid == (1 << 20) // 2 // 8
    s = swb.launch_shape("spmm-mapping=wave-per-row-tile spmm-tile-size=16 spmm-block-size=256", 1 << 20, 13 << 20, 64)
    assert s.physical_grid == (1 << 20) // 8
    s = swb.launch_shape("spmm-mapping=wave-per-row-tile spmm-tile-size=16 spmm-block-size=256", 1 << 20, 24 << 20, 16)
    assert s.physical_grid == (1 << 20) // 4 // 8
    # rows of B of 256, 384 and 512 floats: one warp per matrix row whatever the tile size says
    s = swb.launch_shape("spmm-mapping=wave-per-row-tile spmm-tile-size=32 spmm-block-size=128", 1000, 64000, 512)
    assert (s.work_units, s.physical_grid) == (16000, 250)


def test_shard_rows_by_nnz():
    rp = np.array([0, 10, 10, 30, 31, 100, 100, 120], np.int32)
    b = swb.shard_rows_by_nnz(rp, 4)
    assert b[0] == 0 and b[-1] == 7 and np.all(np.diff(b) >= 0)
    # boundary k is the first row whose offset reaches k * nnz / shards
    for k in range(1, 4):
        t = k * 120 // 4
        assert rp[b[k]] >= t and (b[k] == 0 or rp[b[k] - 1] < t)
    assert swb.shard_rows_by_nnz(rp, 1).tolist() == [0, 7]
    empty = swb.shard_rows_by_nnz(np.zeros(5, np.int32), 3)
    assert empty[0] == 0 and empty[-1] == 4


def test_host_content_check_needs_no_gpu():
    lib = _lib.load()
    rp = np.array([0, 2, 1], np.int32); ci = np.array([0, 1], np.int32)
    st = lib.swb_check_csr_host(None, 2, 4, 2, rp.ctypes.data, ci.ctypes.data)
    assert st == _lib.SWB_ERR_INVALID_DATA and b"non-decreasing" in lib.swb_last_error(None)
    rp = np.array([0, 1, 2], np.int32); ci = np.array([0, 9], np.int32)
    st = lib.swb_check_csr_host(None, 2, 4, 2, rp.ctypes.data, ci.ctypes.data)
    assert st == _lib.SWB_ERR_INVALID_DATA and b"out of bounds" in lib.swb_last_error(None)
    ci = np.array([0, 3], np.int32)
    assert lib.swb_check_csr_host(None, 2, 4, 2, rp.ctypes.data, ci.ctypes.data) == 0


def test_compute_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(swb.SparseWaveError) as e:
        swb.Context(0)
    assert e.value.status == _lib.SWB_ERR_CUDA


def test_plan_row_panels():
    """Row panels of a resident matrix: contiguous, strictly increasing, aligned first positions, about
    equal nnz; no cut where no row starts at an aligned position or the matrix is small."""
    from sparsewave_b200.api import plan_row_panels
    rng = np.random.default_rng(5)
    lens = rng.integers(0, 40, 20000)
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    nnz = int(rp[-1])
    cuts = plan_row_panels(rp, nnz // 8)
    assert cuts[0] == 0 and cuts[-1] == 20000 and len(cuts) == 9
    assert np.all(np.diff(cuts) > 0)
    assert all(rp[c] % 4 == 0 for c in cuts[1:-1])
    per_panel = np.diff(rp[cuts])
    assert per_panel.max() < 1.2 * nnz / 8 and per_panel.min() > 0.8 * nnz / 8
    assert len(plan_row_panels(rp, nnz // 3)) == 4               # nnz / panel_nnz panels
    assert list(plan_row_panels(rp, nnz)) == [0, 20000]           # too small to cut
    assert list(plan_row_panels(rp, 10 * nnz)) == [0, 20000]
    # every interior row starts at position 1 mod 4: nothing to cut at
    odd = np.concatenate([[0, 1], 1 + 4 * np.arange(1, 5000)]).astype(np.int32)
    assert list(plan_row_panels(odd, 100)) == [0, 5000]
    # one giant row holds most positions: the cuts that fall inside it collapse
    giant = np.concatenate([[0], np.cumsum([8] * 10 + [100000] + [8] * 10)]).astype(np.int32)
    cuts = plan_row_panels(giant, 1000)
    assert cuts[0] == 0 and cuts[-1] == 21 and np.all(np.diff(cuts) > 0)
    assert list(plan_row_panels(np.zeros(1, np.int32), 4)) == [0, 0]  # no rows


def test_headers_are_plain_c(tmp_path):
    """Both public headers compile as C99 (the boundary is a C ABI: no C++ or torch types in it) and as C++."""
    import shutil
    import subprocess
    src = tmp_path / "include_check.c"
    src.write_text('#include "sparsewave_b200.h"\n#include "sparsewave_benchmark_utils.h"\n'
                   "int main(void) { swb_options o; swb_options_default(&o); return 0; }\n")
    gcc, gxx = shutil.which("gcc"), shutil.which("g++")
    if not gcc or not gxx:
        pytest.skip("no host compiler")
    inc = str(ROOT / "include")
    subprocess.run([gcc, "-std=c99", "-pedantic", "-Werror", "-Wall", "-I", inc, "-fsyntax-only", str(src)], check=True)
    subprocess.run([gxx, "-std=c++17", "-Werror", "-Wall", "-I", inc, "-fsyntax-only", "-x", "c++", str(src)], check=True)


def test_launches_beyond_the_cuda_grid_limit_are_refused():
    """A grid holds 2^31 - 1 blocks in x: legal options on a matrix that still fits the i32 CSR type can ask for
    more (4 M rows x 2048 right-hand sides, one column per warp), and such a launch is refused, not truncated."""
    opts = "spmm-mapping=wave-per-row-tile spmm-tile-size=1 spmm-block-size=32"
    with pytest.raises(swb.SparseWaveError) as err:
        swb.launch_shape(opts, rows=4 << 20, nnz=64 << 20, n_rhs=2048)
    assert err.value.status == _lib.SWB_ERR_UNSUPPORTED and "2147483647" in str(err.value)
    ok = swb.launch_shape(opts, rows=1 << 20, nnz=16 << 20, n_rhs=2047)
    assert ok.physical_grid == (1 << 20) * 2047
    with pytest.raises(swb.SparseWaveError):
        swb.launch_shape("spmm-mapping=thread-per-output spmm-block-size=32", rows=1 << 30, nnz=1 << 30, n_rhs=128)
    with pytest.raises(swb.SparseWaveError):
        swb.launch_shape("spmm-mapping=thread-per-position spmm-block-size=1", rows=8, nnz=1 << 30, n_rhs=4)


def test_host_calls_refuse_accumulate_before_anything_else():
    """accumulate=1 on a host-buffer entry point is refused up front (their result buffer is never read), with or
    without a context or a device."""
    lib = _lib.load()
    o = swb.make_options("spmv-mapping=wave-per-position spmm-mapping=wave-per-row-tile accumulate=1")
    calls = [lambda: lib.swb_spmv_host(None, C.byref(o), 1, 1, 0, None, None, None, None, None),
             lambda: lib.swb_spmm_host(None, C.byref(o), 1, 1, 0, 1, None, None, None, None, None),
             lambda: lib.swb_spmv_resident_host(None, C.byref(o), None, None, None),
             lambda: lib.swb_spmm_resident_host(None, C.byref(o), None, 1, None, None),
             lambda: lib.swb_spmv_sharded_host(None, C.byref(o), None, None, None),
             lambda: lib.swb_spmm_sharded_host(None, C.byref(o), None, 1, None, None)]
    for call in calls:
        assert call() == _lib.SWB_ERR_UNSUPPORTED
        assert b"write-only" in lib.swb_last_error(None)


def test_static_status_needs_an_output_pointer():
    lib = _lib.load()
    assert lib.swb_bsr16_static_status(None, None) == _lib.SWB_ERR_INVALID_ARGUMENT
