"""Shared test helpers: golden cases of the reference's runtime tests, random
CSR builders with empty and ragged rows, and the tolerance check."""
import numpy as np
import torch

import oracle

# test/Dialect/SparseWave/spmv-runtime.mlir:64-126 (5 x 4, one empty row)
SPMV_GOLDEN = dict(row_ptr=[0, 2, 2, 3, 5, 6], col=[0, 2, 1, 0, 3, 2], val=[1, 2, 3, 4, 5, 6],
                   x=[10, 20, 30, 40], y=[70, 0, 60, 240, 180])
# test/Dialect/SparseWave/sparse-tensor-runtime.mlir:29-44
SPMV_GOLDEN_4X4 = dict(row_ptr=[0, 2, 3, 5, 6], col=[0, 2, 1, 0, 3, 2], val=[1, 2, 3, 4, 5, 6],
                       x=[10, 20, 30, 40], y=[70, 60, 240, 180])
# test/Dialect/SparseWave/spmm-sparse-tensor-runtime.mlir:50-67
SPMM_GOLDEN = dict(row_ptr=[0, 2, 4], col=[0, 2, 1, 2], val=[1, 2, 3, 4],
                   B=[[1, 10], [2, 20], [3, 30]], C=[[7, 70], [18, 180]])
# examples/pytorch/csr_spmm.py:35-49 with test/TorchExport/csr_spmm_hip_runtime.mlir:12
SPMM_GOLDEN_TORCH = dict(row_ptr=[0, 2, 3], col=[0, 2, 1], val=[1, 2, 3],
                         B=[[0, 1], [2, 3], [4, 5]], C=[[8, 11], [6, 9]])
# test/Dialect/SparseWave/bsr-spmm-runtime.mlir:24-42
BSR_GOLDEN = dict(brp=[0, 2, 3], bci=[0, 1, 0], bv=[1, 2, 0, 3, 4, 0, 5, 6, 7, 0, 0, 8], bs=2,
                  B=[[1, 10], [2, 20], [3, 30], [4, 40]], C=[[17, 170], [45, 450], [7, 70], [16, 160]])

# test/Dialect/SparseWave/coo-spmv-runtime.mlir:22-40 (duplicate coordinate (0, 0))
COO_GOLDEN = dict(rows=4, row=[0, 0, 0, 1, 2, 2, 3], col=[0, 0, 2, 1, 0, 3, 2], val=[0.25, 0.75, 2, 3, 4, 5, 6],
                  x=[10, 20, 30, 40], y=[70, 60, 240, 180])

SPMV_MAPPING_OPTIONS = [
    "spmv-mapping=thread-per-row",
    "spmv-mapping=wave-per-row",
    "spmv-mapping=block-per-row",
    "spmv-mapping=thread-per-position",
    "spmv-mapping=thread-per-position spmv-position-chunk-size=4",
    "spmv-mapping=thread-per-position spmv-position-chunk-size=4 spmv-position-reduction=segmented",
    "spmv-mapping=thread-per-position spmv-position-chunk-size=16 spmv-position-reduction=segmented",
    "spmv-mapping=wave-per-position",
    "spmv-mapping=wave-per-position wave-position-batch=1",
    "spmv-mapping=wave-per-position wave-position-batch=3",
    "spmv-mapping=wave-per-position wave-position-batch=16",
]


def random_csr(rows, cols, mean_len, seed, empty_fraction=0.2, max_len=None):
    """Ragged CSR with empty rows, sorted distinct columns, values in [-1, 1]."""
    rng = np.random.default_rng(seed)
    lens = rng.geometric(1.0 / max(mean_len, 1), size=rows)
    if max_len is not None:
        lens = np.minimum(lens, max_len)
    lens = np.minimum(lens, cols)
    lens[rng.random(rows) < empty_fraction] = 0
    row_ptr = np.zeros(rows + 1, dtype=np.int64)
    row_ptr[1:] = np.cumsum(lens)
    col = np.empty(row_ptr[-1], dtype=np.int32)
    for r in range(rows):
        if lens[r]:
            col[row_ptr[r]:row_ptr[r + 1]] = np.sort(rng.choice(cols, size=lens[r], replace=False))
    val = rng.uniform(-1, 1, size=row_ptr[-1]).astype(np.float32)
    return row_ptr.astype(np.int32), col, val


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def assert_within_bound(actual, expected, bound, rel=1e-5):
    """|actual - expected| <= rel * sum|a*x| per output element."""
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    err = np.abs(actual - expected)
    bad = err > rel * np.asarray(bound) + 1e-30
    assert not bad.any(), (f"{int(bad.sum())} of {bad.size} outputs out of tolerance; worst "
                           f"err/bound = {np.max(err / (np.asarray(bound) + 1e-30)):.3e}")


def assert_bf16_close(C, brp, bci, bv_bits, B_bits, bs):
    """BF16 bar of the BSR path (1e-2 relative, read strictly): against the oracle's own rounded bits the output
    may differ by one bf16 ulp (0.4 % to 0.8 %) wherever the exact sum is at least 2**-6 of the size of its terms;
    outputs of cancelling sums are held to 1e-2 * 2**-6 of that size instead.  `C` is a bf16 CUDA or CPU tensor."""
    import torch
    import oracle
    brp, bci = np.asarray(brp, np.int32), np.asarray(bci, np.int32)
    bits, f32 = oracle.bsr_spmm_bf16(brp, bci, bv_bits, B_bits, bs)
    bound = oracle.bsr_abs_bound_bf16(brp, bci, bv_bits, B_bits, bs)
    got = C.detach().contiguous().view(torch.uint16).cpu().numpy()
    off_by_more_than_an_ulp, cancelling_bad = oracle.bf16_mismatches(got, bits, f32, bound)
    assert (off_by_more_than_an_ulp, cancelling_bad) == (0, 0)
    return bits
