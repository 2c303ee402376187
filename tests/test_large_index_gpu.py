"""Element offsets past 2^31: outputs of more than 2^31 elements and column indices up to the int32 maximum.
The operands are far too large for the CPU oracle, so the expected values come from the structure of the
matrices: one nonzero per row makes every output a single rounded product (bit-exact by construction), and
the SpMV case is summed in float64 on the device and held to the same bound as everywhere else."""
import pytest
import torch

from sparsewave_b200 import workloads as W

pytestmark = pytest.mark.gpu

CHUNK = 1 << 22


def _one_per_row(rows, cols, seed, empty_every):
    g = torch.Generator(device="cuda").manual_seed(seed)
    keep = torch.ones(rows, dtype=torch.bool, device="cuda")
    keep[::empty_every] = False  # empty rows in between
    row_ptr = torch.zeros(rows + 1, dtype=torch.int32, device="cuda")
    row_ptr[1:] = torch.cumsum(keep.to(torch.int32), 0, dtype=torch.int32)
    nnz = int(row_ptr[-1])
    col = torch.randint(0, cols, (nnz,), generator=g, device="cuda", dtype=torch.int32)
    val = torch.rand(nnz, generator=g, device="cuda") * 2 - 1
    return keep, row_ptr, col, val


@pytest.mark.parametrize("opts", [
    "spmm-mapping=wave-per-row-tile spmm-tile-size=16 spmm-block-size=256",
    "spmm-mapping=wave-per-row-tile spmm-tile-size=5 spmm-block-size=64",
    "spmm-mapping=thread-per-output spmm-block-size=256",
    "spmm-mapping=thread-per-position spmm-position-chunk-size=4",
])
def test_spmm_outputs_past_2_pow_31_elements(ctx, opts):
    rows, cols, n = (1 << 25) + 77, 5000, 64  # rows * n = 2^31 + 4928 output elements (8.6 GB)
    keep, row_ptr, col, val = _one_per_row(rows, cols, 61, 1000)
    B = W.dense_uniform((cols, n), seed=62, device="cuda")
    C = ctx.spmm(opts, row_ptr, col, val, B)
    assert ctx.device_status() == 0 and C.shape == (rows, n)
    pos = row_ptr[:-1].long()
    for r0 in range(0, rows, CHUNK):
        r1 = min(rows, r0 + CHUNK)
        k = keep[r0:r1]
        p = pos[r0:r1].clamp(max=col.numel() - 1)
        expected = (val[p][:, None] * B[col[p].long()]) * k[:, None]
        assert torch.equal(C[r0:r1], expected), f"rows {r0}..{r1}"
    del C
    torch.cuda.empty_cache()


def test_spmv_column_indices_up_to_the_int32_maximum(ctx):
    from tests.helpers import SPMV_MAPPING_OPTIONS
    cols = (1 << 31) - 1  # x holds 2^31 - 1 floats (8.6 GB); the last column index is the int32 maximum - 1
    g = torch.Generator(device="cuda").manual_seed(63)
    lens = torch.randint(0, 200, (4096,), generator=g, device="cuda")
    lens[7], lens[8], lens[4095] = 70000, 0, 1025  # one long row, an empty one behind it, a ragged last row
    rows, nnz = lens.numel(), int(lens.sum())
    row_ptr = torch.zeros(rows + 1, dtype=torch.int32, device="cuda")
    row_ptr[1:] = torch.cumsum(lens, 0).to(torch.int32)
    row_of = torch.repeat_interleave(torch.arange(rows, device="cuda"), lens)
    # distinct sorted columns within a row: a random start plus a strictly increasing walk over the whole range
    step = torch.randint(1, cols // 70001, (nnz,), generator=g, device="cuda")
    walk = torch.cumsum(step, 0)
    first = torch.repeat_interleave(walk[row_ptr[:-1].long().clamp(max=nnz - 1)] - step[row_ptr[:-1].long().clamp(max=nnz - 1)], lens)
    col64 = walk - first - 1
    col64[int(row_ptr[8]) - 1] = cols - 1  # the long row ends on the last column
    assert int(col64.max()) == cols - 1 and int(col64.min()) >= 0
    col = col64.to(torch.int32)
    val = torch.rand(nnz, generator=g, device="cuda") * 2 - 1
    x = torch.empty(cols, device="cuda").uniform_(-1, 1, generator=g)
    prod = val.double() * x[col64].double()
    expected = torch.zeros(rows, dtype=torch.float64, device="cuda").index_add_(0, row_of, prod)
    bound = torch.zeros(rows, dtype=torch.float64, device="cuda").index_add_(0, row_of, prod.abs())
    for opts in SPMV_MAPPING_OPTIONS:
        y = ctx.spmv(opts, row_ptr, col, val, x)
        assert ctx.device_status() == 0
        excess = (y.double() - expected).abs() - 1e-5 * bound
        assert float(excess.max()) <= 0, opts


def test_bsr16_bf16_outputs_past_2_pow_31_elements(ctx):
    grid_rows, grid_cols, n = (1 << 17) + 3, 300, 1024  # 16 * grid_rows * n = 2^31 + 49152 outputs (4.3 GB of bf16)
    keep, brp, bci, _ = _one_per_row(grid_rows, grid_cols, 64, 777)
    nb = bci.numel()
    g = torch.Generator(device="cuda").manual_seed(65)
    blocks = (torch.rand((nb, 16, 16), generator=g, device="cuda") * 2 - 1).to(torch.bfloat16)
    B = W.dense_normal((grid_cols * 16, n), seed=66, device="cuda")
    assert B.dtype == torch.bfloat16
    C = ctx.bsr_spmm("", brp, bci, blocks.reshape(-1), B, 16)
    assert ctx.device_status() == 0 and C.shape == (grid_rows * 16, n)
    Bt = B.float().view(grid_cols, 16, n)
    pos = brp[:-1].long().clamp(max=nb - 1)
    step = 4096
    for b0 in range(0, grid_rows, step):
        b1 = min(grid_rows, b0 + step)
        k = keep[b0:b1][:, None, None]
        a = blocks[pos[b0:b1]].float()
        b = Bt[bci[pos[b0:b1]].long()]
        expected = torch.bmm(a, b) * k                 # products of bf16 values are exact in fp32
        bound = torch.bmm(a.abs(), b.abs()) * k
        got = C[b0 * 16:b1 * 16].float().view(b1 - b0, 16, n)
        # one bf16 ulp around the fp32 sum, plus the slack of the accumulation order where terms cancel
        excess = (got - expected).abs() - (2.0 ** -7) * expected.abs() - 1e-2 * (2.0 ** -6) * bound
        assert float(excess.max()) <= 0, f"block rows {b0}..{b1}"
