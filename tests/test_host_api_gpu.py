"""Host-buffer entry points, memref-descriptor entry points and argument errors on the GPU."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from sparsewave_b200 import SparseWaveError, _lib, make_options
from tests.helpers import BSR_GOLDEN, SPMM_GOLDEN, SPMV_GOLDEN, assert_within_bound, dev, random_csr

pytestmark = pytest.mark.gpu


def test_spmv_host_buffers(ctx):
    rp, ci, v = random_csr(2000, 1500, 11, seed=9)
    x = np.random.default_rng(9).uniform(-1, 1, 1500).astype(np.float32)
    for opts in ("mapping=wave-per-row block-size=128", "mapping=wave-per-position", "mapping=thread-per-row"):
        y = np.full(2000, np.nan, np.float32)
        ctx.spmv_host(opts, rp, ci, v, x, y)
        assert_within_bound(y, oracle.csr_spmv(rp, ci, v, x), oracle.csr_abs_bound(rp, ci, v, x))
    # pinned torch tensors work the same way; a second, larger call regrows the workspace
    rp2, ci2, v2 = random_csr(9000, 1500, 14, seed=10)
    t = [torch.from_numpy(a).pin_memory() for a in (rp2, ci2, v2, x)]
    y = torch.empty(9000, dtype=torch.float32).pin_memory()
    ctx.spmv_host("mapping=wave-per-row", *t, y)
    assert_within_bound(y.numpy(), oracle.csr_spmv(rp2, ci2, v2, x), oracle.csr_abs_bound(rp2, ci2, v2, x))


def test_spmm_and_bsr_host_buffers(ctx):
    rp, ci, v = random_csr(1200, 800, 10, seed=12)
    B = np.random.default_rng(12).uniform(-1, 1, (800, 8)).astype(np.float32)
    Cout = np.empty((1200, 8), np.float32)
    ctx.spmm_host("spmm-mapping=wave-per-row-tile spmm-tile-size=8 spmm-block-size=64", rp, ci, v, B, Cout)
    assert_within_bound(Cout, oracle.csr_spmm(rp, ci, v, B), oracle.csr_abs_bound(rp, ci, v, B))
    g = BSR_GOLDEN
    bv = torch.tensor(g["bv"], dtype=torch.bfloat16)
    Bb = torch.tensor(g["B"], dtype=torch.bfloat16)
    out = torch.empty((4, 2), dtype=torch.bfloat16)
    ctx.bsr_spmm_bf16_host("", torch.tensor(g["brp"], dtype=torch.int32), torch.tensor(g["bci"], dtype=torch.int32),
                           bv, Bb, g["bs"], out)
    assert out.float().tolist() == [[17, 170], [45, 450], [7, 70], [16, 160]]


def _m1(t):
    return _lib.Memref1D(t.data_ptr(), t.data_ptr(), 0, (C.c_int64 * 1)(t.numel()), (C.c_int64 * 1)(1))


def _m2(t):
    return _lib.Memref2D(t.data_ptr(), t.data_ptr(), 0, (C.c_int64 * 2)(*t.shape), (C.c_int64 * 2)(t.shape[1], 1))


def test_memref_entry_points(ctx):
    lib = _lib.load()
    g = SPMV_GOLDEN
    t = [dev(g["row_ptr"], torch.int32), dev(g["col"], torch.int32), dev(g["val"], torch.float32),
         dev(g["x"], torch.float32), torch.zeros(5, device="cuda")]
    d = [_m1(a) for a in t]
    o = make_options("mapping=wave-per-row block-size=128")
    st = lib.swb_spmv_memref(ctx._ctx, C.byref(o), *[C.byref(m) for m in d], None)
    torch.cuda.synchronize()
    assert st == 0 and t[4].cpu().tolist() == g["y"]
    # the emit_c_interface symbol itself (process-wide context, options from the environment)
    t[4].zero_()
    lib._mlir_ciface_sparsewave_spmv(*[C.byref(m) for m in d])
    assert t[4].cpu().tolist() == g["y"]
    # verifier diagnostics (SparseWaveOps.cpp:83-108)
    bad = _m1(torch.zeros(4, device="cuda"))
    st = lib.swb_spmv_memref(ctx._ctx, C.byref(o), C.byref(d[0]), C.byref(d[1]), C.byref(d[2]), C.byref(d[3]),
                             C.byref(bad), None)
    assert st == _lib.SWB_ERR_INVALID_SHAPE
    assert b"row offsets size must equal output size plus one, but got 6 and 4" in lib.swb_last_error(ctx._ctx)
    short = _m1(torch.zeros(5, device="cuda"))
    st = lib.swb_spmv_memref(ctx._ctx, C.byref(o), C.byref(d[0]), C.byref(d[1]), C.byref(short), C.byref(d[3]),
                             C.byref(d[4]), None)
    assert b"column indices and values must have the same size, but got 6 and 5" in lib.swb_last_error(ctx._ctx)

    g = SPMM_GOLDEN
    t = [dev(g["row_ptr"], torch.int32), dev(g["col"], torch.int32), dev(g["val"], torch.float32),
         dev(g["B"], torch.float32), torch.zeros((2, 2), device="cuda")]
    st = lib.swb_spmm_memref(ctx._ctx, C.byref(make_options("spmm-mapping=wave-per-row-tile spmm-block-size=64")),
                             C.byref(_m1(t[0])), C.byref(_m1(t[1])), C.byref(_m1(t[2])), C.byref(_m2(t[3])),
                             C.byref(_m2(t[4])), None)
    torch.cuda.synchronize()
    assert st == 0 and t[4].cpu().tolist() == g["C"]

    g = BSR_GOLDEN
    t = [dev(g["brp"], torch.int32), dev(g["bci"], torch.int32), dev(g["bv"], torch.float32),
         dev(g["B"], torch.float32), torch.zeros((4, 2), device="cuda")]
    args = [C.byref(_m1(t[0])), C.byref(_m1(t[1])), C.byref(_m1(t[2])), C.byref(_m2(t[3])), C.byref(_m2(t[4]))]
    st = lib.swb_bsr_spmm_memref(ctx._ctx, C.byref(make_options("spmm-block-size=64")), *args, 2, None)
    torch.cuda.synchronize()
    assert st == 0 and t[4].cpu().tolist() == g["C"]
    st = lib.swb_bsr_spmm_memref(ctx._ctx, C.byref(make_options("")), *args, 3, None)
    assert st == _lib.SWB_ERR_INVALID_SHAPE
    assert b"output rows must be divisible by block size, but got 4 and 3" in lib.swb_last_error(ctx._ctx)


def test_argument_errors(ctx):
    g = SPMV_GOLDEN
    t = [dev(g["row_ptr"], torch.int32), dev(g["col"], torch.int32), dev(g["val"], torch.float32),
         dev(g["x"], torch.float32)]
    with pytest.raises(SparseWaveError, match="wave-per-row requires the SpMV block size to be a multiple of 32"):
        ctx.spmv("mapping=wave-per-row block-size=48", *t)
    with pytest.raises(SparseWaveError, match="block size must be positive"):
        ctx.bsr_spmm("", t[0], t[1], torch.zeros(0, device="cuda"), torch.zeros((4, 2), device="cuda"), 0)
    with pytest.raises(SparseWaveError, match="bundle supports spmm"):
        ctx.bundle_launch("spmv", 5, t + [t[3]])
    with pytest.raises(TypeError):
        ctx.spmv("", t[0].cpu(), t[1], t[2], t[3])
    before = ctx.kernel_launches
    ctx.spmv("mapping=wave-per-position", *t)
    assert ctx.kernel_launches == before + 2  # zero fill + compute
    # declared sizes at the edge of the i32 range are refused before anything is launched: the wave kernels
    # step through positions in 32-bit strides past a row's end
    B = torch.zeros((4, 4), device="cuda")
    out = torch.zeros((5, 4), device="cuda")
    o = make_options("spmm-mapping=wave-per-row-tile")
    before = ctx.kernel_launches
    st = ctx._lib.swb_spmm(ctx._ctx, C.byref(o), 5, 4, 2 ** 31 - 100, 4, t[0].data_ptr(), t[1].data_ptr(),
                           t[2].data_ptr(), B.data_ptr(), out.data_ptr(), None)
    assert st == _lib.SWB_ERR_UNSUPPORTED and b"at most 2147483391 nonzeros are supported" in ctx._lib.swb_last_error(ctx._ctx)
    assert ctx.kernel_launches == before


def test_accumulate_option(ctx):
    """accumulate=1 adds to the existing output (no zero fill / add on store); other mappings refuse it."""
    rp, ci, v = random_csr(900, 400, 10, seed=5)
    rng = np.random.default_rng(5)
    x = rng.uniform(-1, 1, 400).astype(np.float32)
    B = rng.uniform(-1, 1, (400, 8)).astype(np.float32)
    t = [dev(rp, torch.int32), dev(ci, torch.int32), dev(v), dev(x)]
    bound = oracle.csr_abs_bound(rp, ci, v, x)
    for opts in ("mapping=wave-per-position", "mapping=wave-per-position wave-position-batch=1",
                 "mapping=thread-per-position thread-chunk-size=4 thread-reduction=segmented"):
        y = ctx.spmv(opts, *t)
        ctx.spmv(opts + " accumulate=1", *t, y)
        assert_within_bound(y.cpu().numpy() / 2, oracle.csr_spmv(rp, ci, v, x), bound, rel=2e-5)
    with pytest.raises(SparseWaveError, match="accumulate is available for the position mappings"):
        ctx.spmv("mapping=wave-per-row accumulate=1", *t)
    Bd = dev(B)
    boundB = oracle.csr_abs_bound(rp, ci, v, B)
    for opts in ("spmm-mapping=wave-per-row-tile spmm-tile-size=8 spmm-block-size=64",
                 "spmm-mapping=wave-per-row-tile spmm-tile-size=3 spmm-block-size=64",
                 "spmm-mapping=thread-per-position spmm-position-chunk-size=4"):
        Cm = ctx.spmm(opts, t[0], t[1], t[2], Bd)
        ctx.spmm(opts + " accumulate=1", t[0], t[1], t[2], Bd, Cm)
        assert_within_bound(Cm.cpu().numpy() / 2, oracle.csr_spmm(rp, ci, v, B), boundB, rel=2e-5)
    with pytest.raises(SparseWaveError, match="accumulate is not available"):
        ctx.spmm("spmm-mapping=thread-per-output accumulate=1", t[0], t[1], t[2], Bd)


def test_resident_matrix_host_calls(ctx):
    """Matrix uploaded once (content-checked), dense operand in and result out per call."""
    rp, ci, v = random_csr(3000, 2000, 9, seed=14)
    rng = np.random.default_rng(14)
    m = ctx.csr_upload(3000, 2000, rp, ci, v)
    for seed in (1, 2):  # two different x through the same resident matrix
        x = np.random.default_rng(seed).uniform(-1, 1, 2000).astype(np.float32)
        y = np.empty(3000, np.float32)
        m.spmv_host("mapping=wave-per-position", x, y)
        assert_within_bound(y, oracle.csr_spmv(rp, ci, v, x), oracle.csr_abs_bound(rp, ci, v, x))
    B = rng.uniform(-1, 1, (2000, 4)).astype(np.float32)
    Cm = np.empty((3000, 4), np.float32)
    m.spmm_host("spmm-mapping=wave-per-row-tile spmm-block-size=64", B, Cm)
    assert_within_bound(Cm, oracle.csr_spmm(rp, ci, v, B), oracle.csr_abs_bound(rp, ci, v, B))
    m.release()
    bad = ci.copy()
    bad[5] = 2000  # column out of range: rejected on the host before anything is copied
    with pytest.raises(SparseWaveError, match="out of bounds for 2000 columns"):
        ctx.csr_upload(3000, 2000, rp, bad, v)
    badrp = rp.copy()
    badrp[10] = badrp[11] + 1
    with pytest.raises(SparseWaveError, match="non-decreasing"):
        ctx.csr_upload(3000, 2000, badrp, ci, v)


ALL_SPMV = ["mapping=thread-per-row", "mapping=wave-per-row block-size=128", "mapping=block-per-row block-size=64",
            "mapping=thread-per-position spmv-position-chunk-size=4",
            "mapping=thread-per-position spmv-position-reduction=segmented spmv-position-chunk-size=8",
            "mapping=wave-per-position", "mapping=wave-per-position wave-position-batch=1"]


@pytest.mark.parametrize("halves", [False, True])
def test_resident_matrix_row_panels(ctx, monkeypatch, halves):
    """A resident matrix cut into row panels (result rows copied out while later panels run) and, with
    `halves`, also stored as two column halves (first half of the dense operand used while the second is
    still being copied in) gives the result of the plain call: every SpMV mapping, SpMM with aligned and
    ragged widths, rows of very different lengths and empty rows around the cuts."""
    from sparsewave_b200.api import plan_row_panels
    monkeypatch.setenv("SWB_RESIDENT_PANEL_NNZ", "2000")
    monkeypatch.setenv("SWB_RESIDENT_PANEL_BYTES", "1")
    monkeypatch.setenv("SWB_RESIDENT_SPLIT_NNZ", "1000" if halves else "1000000000")
    rng = np.random.default_rng(21)
    rows, cols = 4000, 3000
    lens = rng.integers(0, 12, rows)
    lens[rng.integers(0, rows, 40)] = 0
    lens[[7, 1500, 3999]] = [900, 2500, 333]
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ci = np.concatenate([np.sort(rng.choice(cols, n, replace=False)) for n in lens]).astype(np.int32)
    v = rng.uniform(-1, 1, rp[-1]).astype(np.float32)
    cuts = plan_row_panels(rp, 2000)
    assert len(cuts) - 1 == 8 and all(rp[c] % 4 == 0 for c in cuts[1:-1])
    m = ctx.csr_upload(rows, cols, rp, ci, v)
    x = rng.uniform(-1, 1, cols).astype(np.float32)
    want, bound = oracle.csr_spmv(rp, ci, v, x), oracle.csr_abs_bound(rp, ci, v, x)
    for opt in ALL_SPMV:
        y = np.full(rows, np.nan, np.float32)
        m.spmv_host(opt, x, y)
        assert_within_bound(y, want, bound)
        if "thread-per-row" in opt:
            assert np.array_equal(y, want)  # the sequential mapping is bit-exact, cut or not
    for n in (1, 4, 5, 64):
        B = rng.uniform(-1, 1, (cols, n)).astype(np.float32)
        for opt in ("spmm-mapping=thread-per-output", "spmm-mapping=wave-per-row-tile spmm-tile-size=4",
                    "spmm-mapping=thread-per-position spmm-position-chunk-size=3"):
            Cm = np.full((rows, n), np.nan, np.float32)
            m.spmm_host(opt, B, Cm)
            assert_within_bound(Cm, oracle.csr_spmm(rp, ci, v, B), oracle.csr_abs_bound(rp, ci, v, B))
    m.release()


def test_unaligned_operands_take_the_scalar_kernels(ctx):
    """Operands that are not 16-byte aligned (views at an odd offset) must not reach the 128-bit paths."""
    rng = np.random.default_rng(8)
    lens = np.array([300, 0, 5, 700, 129, 1, 64, 4097], np.int64)
    cols = 5000
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ci = np.concatenate([np.sort(rng.choice(cols, n, replace=False)) for n in lens]).astype(np.int32)
    v = rng.uniform(-1, 1, rp[-1]).astype(np.float32)
    x = rng.uniform(-1, 1, cols).astype(np.float32)

    def odd(a):  # same values at a 4-byte offset from a 16-byte aligned allocation
        t = torch.empty(len(a) + 1, dtype=torch.from_numpy(a).dtype, device="cuda")
        t[1:] = torch.from_numpy(a).cuda()
        return t[1:]

    expected, bound = oracle.csr_spmv(rp, ci, v, x), oracle.csr_abs_bound(rp, ci, v, x)
    for opts in ("mapping=wave-per-row block-size=128", "mapping=block-per-row block-size=64",
                 "mapping=wave-per-position wave-position-batch=8", "mapping=wave-per-position"):
        y = ctx.spmv(opts, dev(rp), odd(ci), odd(v), odd(x))
        assert odd(ci).data_ptr() % 16 != 0
        assert_within_bound(y.cpu().numpy(), expected, bound)
    B = rng.uniform(-1, 1, (cols, 8)).astype(np.float32)
    Bo = odd(B.reshape(-1)).view(cols, 8)
    Cm = ctx.spmm("spmm-mapping=wave-per-row-tile spmm-tile-size=8 spmm-block-size=64", dev(rp), dev(ci), dev(v), Bo)
    assert_within_bound(Cm.cpu().numpy(), oracle.csr_spmm(rp, ci, v, B), oracle.csr_abs_bound(rp, ci, v, B))
    # BSR 16 x 16 with a misaligned B falls back to the CUDA-core kernel and still matches
    from sparsewave_b200 import workloads as W
    a = W.random_bsr(6, 5, 16, 0.5, seed=3, device="cuda")
    Bb = W.dense_normal((80, 16), seed=3, device="cuda")
    Bbo = torch.empty(80 * 16 + 1, dtype=torch.bfloat16, device="cuda")[1:]
    Bbo.copy_(Bb.reshape(-1))
    C1 = ctx.bsr_spmm("", a.block_row_ptr, a.block_col_idx, a.block_values, Bb, 16)
    C2 = ctx.bsr_spmm("", a.block_row_ptr, a.block_col_idx, a.block_values, Bbo.view(80, 16), 16)
    # tensor-core and CUDA-core kernels add the same exact products in f32 in different orders: the rounded
    # outputs differ by at most one bf16 ulp (two where both sit one ulp either side of the oracle's)
    b1, b2 = C1.view(torch.int16).int(), C2.view(torch.int16).int()
    o1, o2 = torch.where(b1 < 0, -(b1 & 0x7FFF), b1), torch.where(b2 < 0, -(b2 & 0x7FFF), b2)
    big = C1.float().abs() >= 2.0 ** -4 * C1.float().abs().max()
    assert int(((o1 - o2).abs() > 2)[big].sum()) == 0
    assert float((C1.float() - C2.float()).abs().max()) <= 2.0 ** -7 * float(C1.float().abs().max())


def test_host_calls_refuse_accumulate_and_sharded_host_without_a_communicator(ctx):
    """The host-buffer calls never read the caller's result buffer, so accumulate=1 is refused by all of
    them; the sharded host calls on a context without a communicator are the plain resident operators."""
    from sparsewave_b200 import SparseWaveError, _lib
    rp, ci, v = random_csr(900, 700, 8, seed=31)
    rng = np.random.default_rng(31)
    x = rng.uniform(-1, 1, 700).astype(np.float32)
    B = rng.uniform(-1, 1, (700, 8)).astype(np.float32)
    y, C = np.empty(900, np.float32), np.empty((900, 8), np.float32)
    acc = "spmv-mapping=wave-per-position spmm-mapping=wave-per-row-tile accumulate=1"
    resident = ctx.csr_upload(900, 700, rp, ci, v)
    for call in (lambda: ctx.spmv_host(acc, rp, ci, v, x, y), lambda: ctx.spmm_host(acc, rp, ci, v, B, C),
                 lambda: resident.spmv_host(acc, x, y), lambda: resident.spmm_host(acc, B, C),
                 lambda: resident.spmv_sharded_host(acc, x, y), lambda: resident.spmm_sharded_host(acc, B, C)):
        with pytest.raises(SparseWaveError) as err:
            call()
        assert err.value.status == _lib.SWB_ERR_UNSUPPORTED and "write-only" in str(err.value)
    resident.release()
    # rows [200, 650) of the matrix, cut and rebased by the library
    part = ctx.csr_upload_rows(700, rp, ci, v, 200, 650)
    rows = slice(200, 650)
    yp, Cp = np.empty(450, np.float32), np.empty((450, 8), np.float32)
    part.spmv_sharded_host("spmv-mapping=wave-per-position", x, yp)
    assert_within_bound(yp, oracle.csr_spmv(rp, ci, v, x)[rows], oracle.csr_abs_bound(rp, ci, v, x)[rows])
    part.spmm_sharded_host("spmm-mapping=wave-per-row-tile spmm-tile-size=8", B, Cp)
    assert_within_bound(Cp, oracle.csr_spmm(rp, ci, v, B)[rows], oracle.csr_abs_bound(rp, ci, v, B)[rows])
    part.release()
    with pytest.raises(SparseWaveError):
        ctx.csr_upload_rows(700, rp, ci, v, 650, 200)
    # device operands: without a communicator the sharded operators are the plain ones
    t = [dev(rp, torch.int32), dev(ci, torch.int32), dev(v), dev(x)]
    ys = ctx.spmv_sharded("spmv-mapping=wave-per-position", t[0], t[1], t[2], t[3], 700)
    assert_within_bound(ys.cpu().numpy(), oracle.csr_spmv(rp, ci, v, x), oracle.csr_abs_bound(rp, ci, v, x))


def test_resident_bsr_with_host_operands(ctx):
    """swb_bsr_upload + swb_bsr_spmm_bf16_resident_host: the block structure is checked and copied once, a call
    sends B and returns C; the result equals the device-operand call's bit for bit, and a malformed structure
    is refused at upload."""
    from sparsewave_b200 import workloads as W
    a = W.random_bsr(40, 30, 16, 0.2, seed=21)
    B = W.dense_normal((30 * 16, 64), seed=21)
    resident = ctx.bsr_upload(a.cols, a.block_row_ptr, a.block_col_idx, a.block_values, 16)
    C_host = torch.empty((a.rows, 64), dtype=torch.bfloat16)
    for _ in range(2):
        resident.spmm_host("", B, C_host)
        C_dev = ctx.bsr_spmm("", a.block_row_ptr.cuda(), a.block_col_idx.cuda(), a.block_values.cuda(), B.cuda(), 16)
        assert torch.equal(C_host.view(torch.uint16), C_dev.cpu().view(torch.uint16))
    assert ctx.device_status() == 0
    resident.release()
    bad = a.block_col_idx.clone()
    bad[3] = 30  # one block column past the end
    with pytest.raises(SparseWaveError) as err:
        ctx.bsr_upload(a.cols, a.block_row_ptr, bad, a.block_values, 16)
    assert err.value.status == _lib.SWB_ERR_INVALID_DATA and "out of bounds" in str(err.value)
    short = a.block_row_ptr.clone()
    short[-1] -= 1
    with pytest.raises(SparseWaveError, match="last block-row offset"):
        ctx.bsr_upload(a.cols, short, a.block_col_idx, a.block_values, 16)
