"""CSR SpMV parity on the GPU, through the C ABI, against the oracle."""
import numpy as np
import pytest
import torch

import oracle
from sparsewave_b200 import workloads as W
from tests.helpers import (COO_GOLDEN, SPMV_GOLDEN, SPMV_GOLDEN_4X4, SPMV_MAPPING_OPTIONS, assert_within_bound, dev, random_csr)

pytestmark = pytest.mark.gpu

BLOCKS = [32, 64, 128, 256, 1024]


def run(ctx, opts, rp, ci, v, x):
    y = ctx.spmv(opts, dev(rp, torch.int32), dev(ci, torch.int32), dev(v, torch.float32), dev(x, torch.float32))
    torch.cuda.synchronize()
    return y.cpu().numpy()


@pytest.mark.parametrize("opts", SPMV_MAPPING_OPTIONS)
@pytest.mark.parametrize("g", [SPMV_GOLDEN, SPMV_GOLDEN_4X4])
def test_runtime_goldens_every_mapping(ctx, opts, g):
    # spmv-runtime.mlir runs all mappings with spmv-block-size=128
    y = run(ctx, opts + " spmv-block-size=128", g["row_ptr"], g["col"], g["val"], g["x"])
    assert y.tolist() == g["y"]


@pytest.mark.parametrize("opts", SPMV_MAPPING_OPTIONS)
@pytest.mark.parametrize("block", BLOCKS)
def test_ragged_with_empty_rows(ctx, opts, block):
    rp, ci, v = random_csr(1531, 997, 9, seed=block)
    x = np.random.default_rng(1).uniform(-1, 1, 997).astype(np.float32)
    expected = oracle.csr_spmv(rp, ci, v, x)
    bound = oracle.csr_abs_bound(rp, ci, v, x)
    y = run(ctx, f"{opts} spmv-block-size={block}", rp, ci, v, x)
    assert_within_bound(y, expected, bound)
    assert oracle.count_mismatches_reference(y, expected) == 0


def test_thread_per_row_is_bit_exact(ctx):
    rp, ci, v = random_csr(5000, 3000, 40, seed=2, empty_fraction=0.1)
    x = np.random.default_rng(2).uniform(-1, 1, 3000).astype(np.float32)
    y = run(ctx, "mapping=thread-per-row block-size=64", rp, ci, v, x)
    assert np.array_equal(y, oracle.csr_spmv(rp, ci, v, x))


@pytest.mark.parametrize("opts", SPMV_MAPPING_OPTIONS)
def test_long_rows_take_the_vector_path(ctx, opts):
    # rows longer than 128 positions use 128-bit loads with unaligned heads and tails
    rng = np.random.default_rng(7)
    lens = np.array([0, 1, 129, 3, 700, 131, 0, 4097, 2, 513, 128, 127], dtype=np.int64)
    cols = 6000
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ci = np.concatenate([np.sort(rng.choice(cols, n, replace=False)) for n in lens]).astype(np.int32)
    v = rng.uniform(-1, 1, rp[-1]).astype(np.float32)
    x = rng.uniform(-1, 1, cols).astype(np.float32)
    y = run(ctx, opts + " spmv-block-size=128", rp, ci, v, x)
    assert_within_bound(y, oracle.csr_spmv(rp, ci, v, x), oracle.csr_abs_bound(rp, ci, v, x))


@pytest.mark.parametrize("opts", SPMV_MAPPING_OPTIONS)
def test_degenerate_shapes(ctx, opts):
    # rows == 0 and nnz == 0 are legal: the grid clamps to one inactive block
    z = np.zeros(1, np.int32)
    e32, ef = np.zeros(0, np.int32), np.zeros(0, np.float32)
    assert run(ctx, opts, z, e32, ef, np.ones(3, np.float32)).shape == (0,)
    rp = np.zeros(6, np.int32)
    assert run(ctx, opts, rp, e32, ef, np.ones(3, np.float32)).tolist() == [0] * 5
    # one nonzero in the last row after many empty rows
    rp = np.array([0] * 40 + [1], np.int32)
    y = run(ctx, opts, rp, np.array([2], np.int32), np.array([3.0], np.float32), np.array([1, 2, 5], np.float32))
    assert y.tolist() == [0] * 39 + [15]


def test_output_is_overwritten_not_accumulated(ctx):
    g = SPMV_GOLDEN
    for opts in SPMV_MAPPING_OPTIONS:
        y = torch.full((5,), 1e6, dtype=torch.float32, device="cuda")
        ctx.spmv(opts, dev(g["row_ptr"], torch.int32), dev(g["col"], torch.int32), dev(g["val"], torch.float32),
                 dev(g["x"], torch.float32), y)
        assert y.cpu().tolist() == g["y"]


@pytest.mark.parametrize("opts,kind", [
    ("mapping=thread-per-position", ("thread", 1, False)),
    ("mapping=thread-per-position thread-chunk-size=4", ("thread", 4, False)),
    ("mapping=thread-per-position thread-chunk-size=5 thread-reduction=segmented", ("thread", 5, True)),
    ("mapping=wave-per-position wave-position-batch=1", ("wave", 1, None)),
    ("mapping=wave-per-position wave-position-batch=5", ("wave", 5, None)),
    ("mapping=wave-per-position wave-position-batch=16", ("wave", 16, None)),
])
@pytest.mark.parametrize("block", [64, 256])
def test_position_indexing_is_bit_exact(ctx, opts, kind, block):
    """Row recovered for every position, owning worker and segment ends equal the reference schedule's."""
    rp, ci, v = random_csr(3001, 800, 6, seed=17, empty_fraction=0.35)
    x = np.random.default_rng(3).uniform(-1, 1, 800).astype(np.float32)
    y, row, worker, seg = ctx.spmv_position_trace(f"{opts} block-size={block}", dev(rp, torch.int32),
                                                  dev(ci, torch.int32), dev(v), dev(x))
    torch.cuda.synchronize()
    if kind[0] == "thread":
        oy, orow, oworker, oseg = oracle.spmv_thread_position(rp, ci, v, x, chunk=kind[1], segmented=kind[2], trace=True)
    else:
        oy, orow, oworker, oseg = oracle.spmv_wave_position(rp, ci, v, x, block=block, batch=kind[1], trace=True)
    assert np.array_equal(row.cpu().numpy(), orow)
    assert np.array_equal(worker.cpu().numpy(), oworker)
    assert np.array_equal(seg.cpu().numpy(), oseg)
    assert_within_bound(y.cpu().numpy(), oy, oracle.csr_abs_bound(rp, ci, v, x))


def test_config_c1_wave_per_row_block_128(ctx):
    a, x = W.config_c1()
    rp, ci, v = a.numpy()
    expected = oracle.csr_spmv(rp, ci, v, x.numpy())
    y = ctx.spmv("spmv-mapping=wave-per-row spmv-block-size=128", a.row_ptr.cuda(), a.col_idx.cuda(),
                 a.values.cuda(), x.cuda())
    assert_within_bound(y.cpu().numpy(), expected, oracle.csr_abs_bound(rp, ci, v, x.numpy()))


@pytest.mark.parametrize("opts", [
    "mapping=thread-per-row", "mapping=wave-per-row block-size=128", "mapping=block-per-row block-size=64",
    "mapping=thread-per-position", "mapping=thread-per-position thread-chunk-size=8 thread-reduction=segmented",
    "mapping=thread-per-position thread-chunk-size=16 thread-reduction=segmented",
    "mapping=wave-per-position", "mapping=wave-per-position block-size=512"])
def test_power_law_rows(ctx, opts):
    """Config-3 shape at a size the oracle finishes in seconds: Zipf(1.8) row lengths up to 65536."""
    a, x = W.config_c3(device="cuda", rows=1 << 18)
    y = ctx.spmv(opts, a.row_ptr, a.col_idx, a.values, x)
    rp, ci, v = a.numpy()
    xh = x.cpu().numpy()
    expected = oracle.csr_spmv(rp, ci, v, xh, parallel=True)
    assert_within_bound(y.cpu().numpy(), expected, oracle.csr_abs_bound(rp, ci, v, xh))


def test_full_size_power_law_properties(ctx):
    """Config 3 at full size: linearity in x and agreement between mappings (size-independent properties)."""
    a, x = W.config_c3(device="cuda")
    assert a.rows == 4194304 and a.nnz > 60_000_000
    opts = "mapping=wave-per-position"
    y1 = ctx.spmv(opts, a.row_ptr, a.col_idx, a.values, x)
    x2 = W.dense_uniform((a.cols,), seed=33, device="cuda")
    y2 = ctx.spmv(opts, a.row_ptr, a.col_idx, a.values, x2)
    y12 = ctx.spmv(opts, a.row_ptr, a.col_idx, a.values, x + x2)
    ones = torch.ones_like(x)
    babs = ctx.spmv("mapping=thread-per-row", a.row_ptr, a.col_idx, a.values.abs(), ones)  # sum |a| >= sum |a x|
    tol = 4e-5 * babs + 1e-6
    assert bool(((y1 + y2 - y12).abs() <= tol).all())
    yr = ctx.spmv("mapping=thread-per-row", a.row_ptr, a.col_idx, a.values, x)
    assert bool(((y1 - yr).abs() <= tol).all())
    # checksum against the host: sum_r y[r] == sum_p val[p] * x[col[p]] in f64
    total = (a.values.double() * x[a.col_idx.long()].double()).sum()
    assert abs(float(y1.double().sum() - total)) <= 1e-6 * float(babs.double().sum())


@pytest.mark.parametrize("block", [32, 128, 1024])
def test_coo_spmv(ctx, block):
    g = COO_GOLDEN
    y = ctx.coo_spmv(f"block-size={block}", g["rows"], dev(g["row"], torch.int32), dev(g["col"], torch.int32),
                     dev(g["val"], torch.float32), dev(g["x"], torch.float32))
    assert y.cpu().tolist() == g["y"]
    # unordered entries with duplicates against the oracle's sequential accumulation
    rng = np.random.default_rng(block)
    rows, cols, nnz = 700, 500, 20000
    ri, ci = rng.integers(0, rows, nnz).astype(np.int32), rng.integers(0, cols, nnz).astype(np.int32)
    v, x = rng.uniform(-1, 1, nnz).astype(np.float32), rng.uniform(-1, 1, cols).astype(np.float32)
    y = ctx.coo_spmv(f"block-size={block}", rows, dev(ri), dev(ci), dev(v), dev(x)).cpu().numpy()
    bound = np.zeros(rows)
    np.add.at(bound, ri, np.abs(v.astype(np.float64) * x[ci]))
    assert_within_bound(y, oracle.coo_spmv(rows, ri, ci, v, x), bound)
    assert ctx.coo_spmv("", 3, dev(np.zeros(0, np.int32)), dev(np.zeros(0, np.int32)), dev(np.zeros(0, np.float32)),
                        dev(x)).cpu().tolist() == [0, 0, 0]


def _offset_view(a, k, dtype):
    """A CUDA copy of `a` that starts k elements past a 16-byte boundary."""
    t = torch.empty(len(a) + 4, dtype=dtype, device="cuda")
    assert t.data_ptr() % 16 == 0
    t[k:k + len(a)].copy_(torch.as_tensor(np.ascontiguousarray(a)).to(dtype))
    return t[k:k + len(a)]


@pytest.mark.parametrize("k", [1, 2, 3])
@pytest.mark.parametrize("batch", [3, 16])
def test_wave_per_position_on_views_off_a_16_byte_boundary(ctx, k, batch):
    """col and val views that start the same number of elements past a 16-byte boundary (slices of larger
    arrays, as a row shard cut without a copy is) keep the vectorised span kernel: rows, owning waves and
    segment ends stay bit-exact, and so does a view whose two arrays are offset differently (scalar kernel)."""
    rp, ci, v = random_csr(3001, 800, 6, seed=23 + k, empty_fraction=0.35)
    x = np.random.default_rng(5).uniform(-1, 1, 800).astype(np.float32)
    opts = f"mapping=wave-per-position wave-position-batch={batch} block-size=128"
    oy, orow, oworker, oseg = oracle.spmv_wave_position(rp, ci, v, x, block=128, batch=batch, trace=True)
    bound = oracle.csr_abs_bound(rp, ci, v, x)
    for kc, kv in ((k, k), (k, (k + 1) % 4)):
        cv, vv = _offset_view(ci, kc, torch.int32), _offset_view(v, kv, torch.float32)
        assert cv.data_ptr() % 16 == 4 * kc
        y, row, worker, seg = ctx.spmv_position_trace(opts, dev(rp, torch.int32), cv, vv, dev(x))
        assert np.array_equal(row.cpu().numpy(), orow) and np.array_equal(worker.cpu().numpy(), oworker)
        assert np.array_equal(seg.cpu().numpy(), oseg)
        assert_within_bound(y.cpu().numpy(), oy, bound)
        assert_within_bound(ctx.spmv(opts, dev(rp, torch.int32), cv, vv, dev(x)).cpu().numpy(), oy, bound)


def test_long_rows_through_shared_memory_bands(ctx, monkeypatch):
    """The opt-in long-row path of wave-per-position (SWB_BAND_MIN_NNZ): rows of at least 32 positions per
    band of 32768 columns go through shared-memory bands of x, the span kernel leaves them out.  Power-law
    rows, a wide matrix with few very long rows and a column count that is no multiple of 4, every row long,
    and no long row at all."""
    monkeypatch.setenv("SWB_BAND_MIN_NNZ", "1")
    cases = [W.zipf_csr(50000, 50000, 1.5, 1, 20000, seed=7, device="cuda"),
             W.zipf_csr(1200, 1000003, 1.01, 1, 60000, seed=9, device="cuda"),
             W.uniform_csr(2000, 200000, 3000, seed=11, device="cuda"),
             W.uniform_csr(400000, 70001, 12, seed=12, device="cuda")]  # each large enough for spans of >= 2 partitions
    for a in cases:
        x = W.dense_uniform((a.cols,), seed=8, device="cuda")
        launches = ctx.kernel_launches
        y = ctx.spmv("spmv-mapping=wave-per-position spmv-block-size=256", a.row_ptr, a.col_idx, a.values, x)
        assert ctx.kernel_launches - launches == 4  # long-row list, band boundaries, span kernel, band kernel
        rp, ci, v = a.numpy()
        xh = x.cpu().numpy()
        assert_within_bound(y.cpu().numpy(), oracle.csr_spmv(rp, ci, v, xh, parallel=True),
                            oracle.csr_abs_bound(rp, ci, v, xh))
    # accumulate adds to y instead of overwriting it
    a = cases[0]
    x = W.dense_uniform((a.cols,), seed=8, device="cuda")
    y = torch.ones(a.rows, device="cuda")
    ctx.spmv("spmv-mapping=wave-per-position accumulate=1", a.row_ptr, a.col_idx, a.values, x, y)
    rp, ci, v = a.numpy()
    xh = x.cpu().numpy()
    assert_within_bound(y.cpu().numpy() - 1.0, oracle.csr_spmv(rp, ci, v, xh, parallel=True),
                        oracle.csr_abs_bound(rp, ci, v, xh) + 1.0)
    monkeypatch.delenv("SWB_BAND_MIN_NNZ")
    launches = ctx.kernel_launches
    ctx.spmv("spmv-mapping=wave-per-position", a.row_ptr, a.col_idx, a.values, x)
    assert ctx.kernel_launches - launches == 2  # zero fill and span kernel: the path is opt-in


def test_gather_probe_adds_every_product(ctx):
    """swb_probe_stream_gather: the sinks add up to sum val[p] * x[col[p]] over the positions it covers."""
    a, x = W.config_c3(device="cuda", rows=1 << 16, max_len=2048)
    sink = ctx.probe_stream_gather(a.col_idx, a.values, x)
    n = a.nnz - a.nnz % 4
    want = float((a.values[:n].double() * x[a.col_idx[:n].long()].double()).sum())
    scale = float((a.values[:n].double() * x[a.col_idx[:n].long()].double()).abs().sum())
    assert abs(float(sink.double().sum()) - want) <= 1e-5 * scale
