"""CSR SpMM and BSR SpMM parity on the GPU, through the C ABI, against the oracle."""
import numpy as np
import pytest
import torch

import oracle
from sparsewave_b200 import workloads as W
from tests.helpers import (BSR_GOLDEN, SPMM_GOLDEN, SPMM_GOLDEN_TORCH, assert_bf16_close, assert_within_bound, dev,
                           random_csr)

pytestmark = pytest.mark.gpu

# spmm-sparse-tensor-runtime.mlir:2-29 runs these four pipelines (tile 4 > N = 2 exercises the tail path)
SPMM_GOLDEN_OPTIONS = [
    "spmm-mapping=thread-per-output spmm-block-size=64",
    "spmm-mapping=wave-per-row-tile spmm-block-size=64 spmm-tile-size=2",
    "spmm-mapping=wave-per-row-tile spmm-block-size=64 spmm-tile-size=4",
    "spmm-mapping=thread-per-position spmm-block-size=64 spmm-position-chunk-size=4",
]


def run(ctx, opts, rp, ci, v, B):
    C = ctx.spmm(opts, dev(rp, torch.int32), dev(ci, torch.int32), dev(v, torch.float32), dev(B, torch.float32))
    torch.cuda.synchronize()
    return C.cpu().numpy()


@pytest.mark.parametrize("opts", SPMM_GOLDEN_OPTIONS)
@pytest.mark.parametrize("g", [SPMM_GOLDEN, SPMM_GOLDEN_TORCH])
def test_runtime_goldens(ctx, opts, g):
    C = run(ctx, opts, g["row_ptr"], g["col"], g["val"], np.array(g["B"], np.float32))
    assert C.tolist() == g["C"]


@pytest.mark.parametrize("tile", [1, 2, 3, 4, 5, 8, 12, 16, 31, 32])
@pytest.mark.parametrize("n", [1, 4, 7, 24, 32, 48, 64, 70, 96, 128, 256, 384, 512])
def test_wave_per_row_tile_all_tiles(ctx, tile, n):
    rp, ci, v = random_csr(701, 433, 20, seed=tile * 100 + n, empty_fraction=0.15)
    B = np.random.default_rng(4).uniform(-1, 1, (433, n)).astype(np.float32)
    opts = f"spmm-mapping=wave-per-row-tile spmm-tile-size={tile} spmm-block-size=64"
    want, bound = oracle.csr_spmm(rp, ci, v, B), oracle.csr_abs_bound(rp, ci, v, B)
    C = run(ctx, opts, rp, ci, v, B)
    assert_within_bound(C, want, bound)
    if tile == 32 and n >= 96:  # the kernels for wide rows of B also add to an existing C
        Cd = torch.full((701, n), 2.0, dtype=torch.float32, device="cuda")
        ctx.spmm(opts + " accumulate=1", dev(rp, torch.int32), dev(ci, torch.int32), dev(v, torch.float32),
                 dev(B, torch.float32), Cd)
        assert_within_bound(Cd.cpu().numpy(), want + 2.0, bound + 2.0)


@pytest.mark.parametrize("mean_len", [2, 9, 14, 30, 90])
@pytest.mark.parametrize("n", [4, 8, 16, 32, 64])
def test_wave_per_row_tile_short_rows(ctx, mean_len, n):
    """Rows of B of up to 64 floats: the lanes that serve one matrix row (4, 8, 16 or the whole warp) follow
    the mean row length; row counts that do not fill the last warp, one row, and accumulation."""
    for rows in (701, 1):
        rp, ci, v = random_csr(rows, 433, mean_len, seed=mean_len * 10 + n, empty_fraction=0.1)
        B = np.random.default_rng(5).uniform(-1, 1, (433, n)).astype(np.float32)
        want, bound = oracle.csr_spmm(rp, ci, v, B), oracle.csr_abs_bound(rp, ci, v, B)
        opts = "spmm-mapping=wave-per-row-tile spmm-tile-size=4 spmm-block-size=128"
        assert_within_bound(run(ctx, opts, rp, ci, v, B), want, bound)
        t = [dev(rp, torch.int32), dev(ci, torch.int32), dev(v, torch.float32), dev(B, torch.float32)]
        C = torch.ones((rows, n), dtype=torch.float32, device="cuda")
        ctx.spmm(opts + " accumulate=1", t[0], t[1], t[2], t[3], C)
        assert_within_bound(C.cpu().numpy(), want + 1.0, bound + 1.0)


@pytest.mark.parametrize("block", [32, 64, 256, 1024])
def test_thread_per_output_is_bit_exact(ctx, block):
    rp, ci, v = random_csr(997, 600, 12, seed=block)
    B = np.random.default_rng(5).uniform(-1, 1, (600, 5)).astype(np.float32)
    C = run(ctx, f"spmm-mapping=thread-per-output spmm-block-size={block}", rp, ci, v, B)
    assert np.array_equal(C, oracle.csr_spmm(rp, ci, v, B))


@pytest.mark.parametrize("chunk", [1, 3, 4, 64])
def test_thread_per_position(ctx, chunk):
    rp, ci, v = random_csr(400, 300, 8, seed=chunk, empty_fraction=0.3)
    B = np.random.default_rng(6).uniform(-1, 1, (300, 6)).astype(np.float32)
    C = run(ctx, f"spmm-mapping=thread-per-position spmm-position-chunk-size={chunk} spmm-block-size=128", rp, ci, v, B)
    assert_within_bound(C, oracle.csr_spmm(rp, ci, v, B), oracle.csr_abs_bound(rp, ci, v, B))


def test_degenerate_shapes(ctx):
    for opts in SPMM_GOLDEN_OPTIONS:
        C = run(ctx, opts, np.zeros(5, np.int32), np.zeros(0, np.int32), np.zeros(0, np.float32),
                np.ones((3, 2), np.float32))
        assert C.tolist() == [[0, 0]] * 4
        C = run(ctx, opts, np.zeros(1, np.int32), np.zeros(0, np.int32), np.zeros(0, np.float32),
                np.ones((3, 2), np.float32))
        assert C.shape == (0, 2)


def test_config_c2_bundle_shape(ctx):
    """65536 x 65536, 32 nnz per row, N = 4, wave-per-row-tile tile 4 block 64."""
    a, B = W.config_c2(device="cuda")
    C = ctx.spmm("spmm-mapping=wave-per-row-tile spmm-tile-size=4 spmm-block-size=64", a.row_ptr, a.col_idx,
                 a.values, B)
    rp, ci, v = a.numpy()
    Bh = B.cpu().numpy()
    want, bound = oracle.csr_spmm(rp, ci, v, Bh, parallel=True), oracle.csr_abs_bound(rp, ci, v, Bh)
    assert_within_bound(C.cpu().numpy(), want, bound)
    # the lrrt-style launch (five bare pointers, n = output rows; NNZ is not part of that contract, so it
    # runs the warp-per-row schedule whatever the row lengths) meets the same bound
    C2 = torch.empty_like(C)
    ctx.bundle_launch("spmm", a.rows, [a.row_ptr, a.col_idx, a.values, B, C2])
    assert_within_bound(C2.cpu().numpy(), want, bound)


@pytest.mark.parametrize("tile", [4, 8, 16])
def test_config_c4_shape_reduced(ctx, tile):
    """Banded-plus-random structure, N = 64, at 1/64 of the full row count."""
    a, B = W.config_c4(device="cuda", rows=32768)
    C = ctx.spmm(f"spmm-mapping=wave-per-row-tile spmm-tile-size={tile} spmm-block-size=256", a.row_ptr, a.col_idx,
                 a.values, B)
    rp, ci, v = a.numpy()
    Bh = B.cpu().numpy()
    assert_within_bound(C.cpu().numpy(), oracle.csr_spmm(rp, ci, v, Bh, parallel=True),
                        oracle.csr_abs_bound(rp, ci, v, Bh))


def test_bsr_runtime_golden(ctx):
    g = BSR_GOLDEN
    C = ctx.bsr_spmm("spmm-block-size=64", dev(g["brp"], torch.int32), dev(g["bci"], torch.int32),
                     dev(g["bv"], torch.float32), dev(g["B"], torch.float32), g["bs"])
    assert C.cpu().tolist() == g["C"]
    Cb = ctx.bsr_spmm("spmm-block-size=64", dev(g["brp"], torch.int32), dev(g["bci"], torch.int32),
                      dev(g["bv"], torch.float32).bfloat16(), dev(g["B"], torch.float32).bfloat16(), g["bs"])
    assert Cb.float().cpu().tolist() == [[17, 170], [45, 450], [7, 70], [16, 160]]


@pytest.mark.parametrize("bs", [2, 4, 8])
def test_bsr_f32_is_bit_exact(ctx, bs):
    a = W.random_bsr(40, 30, bs, 0.2, seed=bs, dtype=torch.float32)
    B = W.dense_uniform((30 * bs, 9), seed=bs)
    C = ctx.bsr_spmm("", a.block_row_ptr.cuda(), a.block_col_idx.cuda(), a.block_values.cuda(), B.cuda(), bs)
    expected = oracle.bsr_spmm_f32(a.block_row_ptr.numpy(), a.block_col_idx.numpy(), a.block_values.numpy(),
                                   B.numpy(), bs)
    assert np.array_equal(C.cpu().numpy(), expected)


@pytest.mark.parametrize("bs,n", [(4, 32), (16, 64), (32, 96), (48, 32), (33, 64)])
def test_bsr_f32_rows_shared_by_a_warp_are_bit_exact(ctx, bs, n):
    """N a multiple of 32: a warp's outputs share the block row's values (one load, passed on by shuffles);
    block sizes below, at and above the warp width, and one that is no power of two."""
    a = W.random_bsr(20, 17, bs, 0.3, seed=bs + n, dtype=torch.float32)
    B = W.dense_uniform((17 * bs, n), seed=bs)
    C = ctx.bsr_spmm("spmm-block-size=128", a.block_row_ptr.cuda(), a.block_col_idx.cuda(), a.block_values.cuda(),
                     B.cuda(), bs)
    expected = oracle.bsr_spmm_f32(a.block_row_ptr.numpy(), a.block_col_idx.numpy(), a.block_values.numpy(),
                                   B.numpy(), bs)
    assert np.array_equal(C.cpu().numpy(), expected)


def _bsr_bf16_case(ctx, grid_rows, grid_cols, bs, n, density, seed):
    a = W.random_bsr(grid_rows, grid_cols, bs, density, seed=seed)
    B = W.dense_normal((grid_cols * bs, n), seed=seed)
    C = ctx.bsr_spmm("", a.block_row_ptr.cuda(), a.block_col_idx.cuda(), a.block_values.cuda(), B.cuda(), bs)
    assert ctx.device_status() == 0  # no bounded wait of the tensor-core kernel gave up
    bits = assert_bf16_close(C, a.block_row_ptr.numpy(), a.block_col_idx.numpy(),
                             a.block_values.view(torch.uint16).numpy(), B.view(torch.uint16).numpy(), bs)
    return C.float().cpu().numpy(), bits


@pytest.mark.parametrize("bs", [4, 8, 16, 32])
def test_bsr_bf16(ctx, bs):
    _bsr_bf16_case(ctx, 24, 20, bs, 24, 0.25, seed=bs)
    if bs != 16:  # (16 is the tensor-core kernel) rows shared by a warp
        _bsr_bf16_case(ctx, 24, 20, bs, 64, 0.25, seed=bs + 1)


@pytest.mark.parametrize("n", [8, 64, 128, 200, 512])
def test_bsr16_bf16_shapes(ctx, n):
    """16 x 16 blocks (the tensor-core path), with empty block rows and ragged N."""
    _bsr_bf16_case(ctx, 48, 40, 16, n, 0.08, seed=n)


def test_config_c5_reduced(ctx):
    a, B = W.config_c5(device="cuda", block_grid=256, n_rhs=512)
    C = ctx.bsr_spmm("", a.block_row_ptr, a.block_col_idx, a.block_values, B, 16)
    assert ctx.device_status() == 0
    assert_bf16_close(C, a.block_row_ptr.cpu().numpy(), a.block_col_idx.cpu().numpy(),
                      a.block_values.view(torch.uint16).cpu().numpy(), B.view(torch.uint16).cpu().numpy(), 16)


def test_full_size_c4_properties(ctx):
    """Config 4 at full size (2,097,152 rows, N = 64): tile sizes agree with each other and with the bit-exact
    thread-per-output mapping on sampled rows, and C is linear in B."""
    a, B = W.config_c4(device="cuda")
    assert a.nnz == 134217728
    C16 = ctx.spmm("spmm-mapping=wave-per-row-tile spmm-tile-size=16 spmm-block-size=256", a.row_ptr, a.col_idx,
                   a.values, B)
    C32 = ctx.spmm("spmm-mapping=wave-per-row-tile spmm-tile-size=32 spmm-block-size=256", a.row_ptr, a.col_idx,
                   a.values, B)
    C5 = ctx.spmm("spmm-mapping=wave-per-row-tile spmm-tile-size=5 spmm-block-size=64", a.row_ptr, a.col_idx,
                  a.values, B)  # scalar-load kernel with a tail tile (64 = 12 * 5 + 4)
    # |a| <= 1 and |b| <= 1, 64 terms per output: the bound sum|a b| is at most 64
    tol = 1e-5 * 64
    assert float((C16 - C32).abs().max()) <= tol and float((C16 - C5).abs().max()) <= tol
    # oracle on a sample of rows (row slices keep global column numbering)
    rp, ci, v = a.row_ptr.cpu().numpy(), a.col_idx.cpu().numpy(), a.values.cpu().numpy()
    Bh = B.cpu().numpy()
    for r0 in (0, 1000000, 2097152 - 512):
        sl = slice(rp[r0], rp[r0 + 512])
        sub = (rp[r0:r0 + 513] - rp[r0]).astype(np.int32)
        expected = oracle.csr_spmm(sub, ci[sl], v[sl], Bh)
        bound = oracle.csr_abs_bound(sub, ci[sl], v[sl], Bh)
        assert_within_bound(C16[r0:r0 + 512].cpu().numpy(), expected, bound)
    B2 = W.dense_uniform(tuple(B.shape), seed=44, device="cuda")
    lhs = ctx.spmm("spmm-mapping=wave-per-row-tile spmm-tile-size=16 spmm-block-size=256", a.row_ptr, a.col_idx,
                   a.values, B + B2)
    C2 = ctx.spmm("spmm-mapping=wave-per-row-tile spmm-tile-size=16 spmm-block-size=256", a.row_ptr, a.col_idx,
                  a.values, B2)
    assert float((lhs - C16 - C2).abs().max()) <= 4 * tol


def test_full_size_c5_properties(ctx):
    """Config 5 at full size: the tensor-core kernel against the oracle on sampled block rows, and
    against the CUDA-core thread-per-output kernel run on the same operands as 8 x 8 blocks."""
    a, B = W.config_c5(device="cuda")
    C = ctx.bsr_spmm("", a.block_row_ptr, a.block_col_idx, a.block_values, B, 16)
    assert ctx.device_status() == 0
    brp = a.block_row_ptr.cpu().numpy()
    bci = a.block_col_idx.cpu().numpy()
    bv = a.block_values.view(torch.uint16).cpu().numpy()
    Bh = B.view(torch.uint16).cpu().numpy()
    for b0 in (0, 500, 1024 - 8):
        sub = (brp[b0:b0 + 9] - brp[b0]).astype(np.int32)
        sl = slice(brp[b0], brp[b0 + 8])
        assert_bf16_close(C[b0 * 16:(b0 + 8) * 16], sub, bci[sl], bv[sl.start * 256:sl.stop * 256], Bh, 16)
    # every output was written (no NaN from uninitialised memory) and the checksum matches the f64 total
    assert bool(torch.isfinite(C.float()).all())


@pytest.mark.parametrize("rows,band,half,rnd,n", [(5000, 8, 100, 8, 16), (70001, 32, 1024, 32, 64), (3000, 4, 2000, 0, 32),
                                                  (1025, 0, 1, 6, 48)])
def test_wave_per_row_tile_with_a_staged_window_of_b(ctx, monkeypatch, rows, band, half, rnd, n):
    """The opt-in TMA-staged variant of wave-per-row-tile (SWB_SPMM_STAGED=1): 1024 matrix rows x 16 columns per
    CTA, the rows of B around the diagonal read from shared memory and the others from global memory.  Banded,
    banded plus random, a band wider than the window, no band at all; row counts that leave a partial last block;
    the result equals the oracle's whatever falls into the window, and accumulate adds to C."""
    a = W.banded_random_csr(rows, rows, band, half, rnd, seed=rows, device="cuda")
    B = W.dense_uniform((rows, n), seed=3, device="cuda")
    opts = "spmm-mapping=wave-per-row-tile spmm-tile-size=16 spmm-block-size=256"
    monkeypatch.setenv("SWB_SPMM_STAGED", "1")
    C = ctx.spmm(opts, a.row_ptr, a.col_idx, a.values, B)
    C2 = torch.ones((rows, n), device="cuda")
    ctx.spmm(opts + " accumulate=1", a.row_ptr, a.col_idx, a.values, B, C2)
    monkeypatch.delenv("SWB_SPMM_STAGED")
    assert ctx.device_status() == 0
    rp, ci, v = a.numpy()
    Bh = B.cpu().numpy()
    want, bound = oracle.csr_spmm(rp, ci, v, Bh, parallel=True), oracle.csr_abs_bound(rp, ci, v, Bh)
    assert_within_bound(C.cpu().numpy(), want, bound)
    assert_within_bound(C2.cpu().numpy(), want + 1.0, bound + 1.0)
