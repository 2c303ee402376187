"""The BSR entry point for callers that cannot allocate device memory
(swb_bsr16_spmm_bf16_static: no context, status words in a fixed array inside
the library).  It must give the same bits as the regular context-based entry
point, on two calls in a row that share the fixed array, and it must refuse
what does not fit.  Collected last on purpose: a failure here stops nothing
else."""
import pytest
import torch

from sparsewave_b200 import SparseWaveError, _lib, api, workloads as W

pytestmark = pytest.mark.gpu


def _case(grid_rows, grid_cols, n, density, seed):
    a = W.random_bsr(grid_rows, grid_cols, 16, density, seed=seed, device="cuda")
    B = W.dense_normal((grid_cols * 16, n), seed=seed, device="cuda")
    return a, B


def test_matches_the_context_entry_point_twice_in_a_row(ctx):
    # two different shapes back to back: the second call reuses (and must first clear) the status words
    for grid_rows, grid_cols, n, density, seed in [(96, 80, 256, 0.1, 41), (40, 64, 200, 0.2, 42)]:
        a, B = _case(grid_rows, grid_cols, n, density, seed)
        expected = ctx.bsr_spmm("", a.block_row_ptr, a.block_col_idx, a.block_values, B, 16)
        assert ctx.device_status() == 0
        got = api.bsr16_spmm_bf16_static(a.block_row_ptr, a.block_col_idx, a.block_values, B)
        # same kernel, same arithmetic: bit-identical bf16 outputs
        assert torch.equal(got.view(torch.uint16), expected.view(torch.uint16))
    # asynchronous form (no status read-back in the call): the outcome is asked for afterwards, through the
    # same fixed array and again without any allocation
    out = torch.empty_like(expected)
    api.bsr16_spmm_bf16_static(a.block_row_ptr, a.block_col_idx, a.block_values, B, out, wait=False)
    assert api.bsr16_static_status() == 0  # waits for the stream; no CTA of that call gave up
    assert torch.equal(out.view(torch.uint16), expected.view(torch.uint16))


def test_rejects_what_exceeds_the_fixed_array():
    # 4097 block rows x 8 tiles of 256 columns = 32776 CTAs > 32768 status words
    brp = torch.zeros(4097 + 1, dtype=torch.int32, device="cuda")
    brp[1:] = 1
    bci = torch.zeros(1, dtype=torch.int32, device="cuda")
    bv = torch.zeros(256, dtype=torch.bfloat16, device="cuda")
    B = torch.zeros((16, 2048), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(SparseWaveError) as e:
        api.bsr16_spmm_bf16_static(brp, bci, bv, B)
    assert e.value.status == _lib.SWB_ERR_CAPACITY and "at most 32768" in str(e.value)
    with pytest.raises(SparseWaveError) as e:  # 12 columns: rows of B are not 16-byte multiples
        api.bsr16_spmm_bf16_static(brp[:3].contiguous(), bci, bv, torch.zeros((16, 12), dtype=torch.bfloat16, device="cuda"))
    assert e.value.status == _lib.SWB_ERR_UNSUPPORTED
