"""Randomised shapes, block sizes and options through the C ABI against the oracle (hypothesis)."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings, strategies as st

import oracle
from tests.helpers import assert_bf16_close, assert_within_bound, dev

pytestmark = pytest.mark.gpu

SETTINGS = dict(max_examples=40, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.function_scoped_fixture])


@st.composite
def csr_case(draw):
    rows = draw(st.integers(0, 400))
    cols = draw(st.integers(1, 300))
    seed = draw(st.integers(0, 2 ** 31 - 1))
    kind = draw(st.sampled_from(["short", "mixed", "long", "sparse"]))
    rng = np.random.default_rng(seed)
    if kind == "short":
        lens = rng.integers(0, 4, rows)
    elif kind == "long":
        lens = rng.integers(100, 300, rows)
    elif kind == "sparse":
        lens = (rng.random(rows) < 0.1) * rng.integers(1, 40, rows)
    else:
        lens = rng.geometric(0.05, rows) * (rng.random(rows) < 0.8)
    lens = np.minimum(lens, cols).astype(np.int64)
    rp = np.zeros(rows + 1, np.int64)
    rp[1:] = np.cumsum(lens)
    ci = np.concatenate([np.sort(rng.choice(cols, n, replace=False)) for n in lens] + [np.zeros(0, np.int64)])
    v = rng.uniform(-1, 1, rp[-1]).astype(np.float32)
    return rp.astype(np.int32), ci.astype(np.int32), v, cols, rng


SPMV_OPTIONS = st.one_of(
    st.builds(lambda b: f"mapping=thread-per-row block-size={b}", st.sampled_from([1, 7, 32, 100, 256, 1024])),
    st.builds(lambda m, b: f"mapping={m} block-size={b}", st.sampled_from(["wave-per-row", "block-per-row"]),
              st.sampled_from([32, 64, 128, 512, 1024])),
    st.builds(lambda b, c, r: f"mapping=thread-per-position block-size={b} thread-chunk-size={c} thread-reduction={r}",
              st.sampled_from([1, 33, 64, 256, 1024]), st.integers(1, 40), st.sampled_from(["atomic", "segmented"])),
    st.builds(lambda b, k: f"mapping=wave-per-position block-size={b} wave-position-batch={k}",
              st.sampled_from([32, 96, 256, 1024]), st.integers(0, 70)),
)


@settings(**SETTINGS)
@given(case=csr_case(), opts=SPMV_OPTIONS)
def test_spmv_any_shape_any_option(ctx, case, opts):
    rp, ci, v, cols, rng = case
    x = rng.uniform(-1, 1, cols).astype(np.float32)
    y = ctx.spmv(opts, dev(rp), dev(ci), dev(v), dev(x))
    torch.cuda.synchronize()
    assert_within_bound(y.cpu().numpy(), oracle.csr_spmv(rp, ci, v, x), oracle.csr_abs_bound(rp, ci, v, x))


SPMM_OPTIONS = st.one_of(
    st.builds(lambda b: f"spmm-mapping=thread-per-output spmm-block-size={b}", st.sampled_from([1, 48, 256, 1024])),
    st.builds(lambda b, t: f"spmm-mapping=wave-per-row-tile spmm-block-size={b} spmm-tile-size={t}",
              st.sampled_from([32, 64, 256, 1024]), st.integers(1, 32)),
    st.builds(lambda b, c: f"spmm-mapping=thread-per-position spmm-block-size={b} spmm-position-chunk-size={c}",
              st.sampled_from([32, 100, 256]), st.integers(1, 50)),
)


@settings(**SETTINGS)
@given(case=csr_case(), n=st.integers(1, 70), opts=SPMM_OPTIONS)
def test_spmm_any_shape_any_option(ctx, case, n, opts):
    rp, ci, v, cols, rng = case
    B = rng.uniform(-1, 1, (cols, n)).astype(np.float32)
    C = ctx.spmm(opts, dev(rp), dev(ci), dev(v), dev(B))
    torch.cuda.synchronize()
    assert_within_bound(C.cpu().numpy(), oracle.csr_spmm(rp, ci, v, B), oracle.csr_abs_bound(rp, ci, v, B))


@settings(max_examples=25, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.function_scoped_fixture])
@given(brows=st.integers(1, 40), bcols=st.integers(1, 40), n8=st.integers(1, 40), density=st.floats(0.0, 0.6),
       seed=st.integers(0, 10 ** 6))
def test_bsr16_tensor_core_any_shape(ctx, brows, bcols, n8, density, seed):
    from sparsewave_b200 import workloads as W
    a = W.random_bsr(brows, bcols, 16, density, seed=seed)
    B = W.dense_normal((bcols * 16, n8 * 8), seed=seed)
    C = ctx.bsr_spmm("", a.block_row_ptr.cuda(), a.block_col_idx.cuda(), a.block_values.cuda(), B.cuda(), 16)
    assert ctx.device_status() == 0
    assert_bf16_close(C, a.block_row_ptr.numpy(), a.block_col_idx.numpy(), a.block_values.view(torch.uint16).numpy(),
                      B.view(torch.uint16).numpy(), 16)
