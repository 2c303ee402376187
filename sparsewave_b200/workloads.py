"""Seeded synthetic workloads.

Random numbers come from a counter-based generator (the SplitMix64 finaliser of
``seed``, ``stream`` and the element index) written with integer tensor ops, so
the same seed gives the same matrix on the CPU and on a GPU and every element
can be generated independently of the others.

``reference_synthetic`` reproduces the reference runner's own controlled
workloads (benchmark/run_spmv_benchmark.py:225-263 in the SparseWave tree).
The ``config_*`` functions build the five benchmark configurations: fixed-
degree uniform CSR, Zipf row lengths, banded-plus-random CSR and block-sparse
BSR, with uniform-random distinct columns sorted within each row.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

_M1 = -7046029254386353131   # 0x9E3779B97F4A7C15 as int64
_M2 = -4658895280553007687   # 0xBF58476D1CE4E5B9
_M3 = -7723592293110705685   # 0x94D049BB133111EB


def _wrap64(v: int) -> int:
    """Python int reduced to the signed 64-bit value with the same low bits."""
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def _lsr(x: torch.Tensor, k: int) -> torch.Tensor:
    """Logical right shift of int64."""
    return (x >> k) & ((1 << (64 - k)) - 1)


def hash64(seed: int, stream: int, idx: torch.Tensor) -> torch.Tensor:
    """SplitMix64 finaliser of (seed, stream, idx); int64 bit patterns."""
    z = idx.to(torch.int64) * _M1 + _wrap64((seed * 1000003 + stream) * _M2 + _M3)
    z = (z ^ _lsr(z, 30)) * _M2
    z = (z ^ _lsr(z, 27)) * _M3
    return z ^ _lsr(z, 31)


def uniform01(seed: int, stream: int, idx: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """Uniform in [0, 1): 24 random bits for f32, 53 for f64."""
    h = hash64(seed, stream, idx)
    if dtype == torch.float64:
        return _lsr(h, 11).to(torch.float64) * (1.0 / (1 << 53))
    return _lsr(h, 40).to(torch.float32) * (1.0 / (1 << 24))


def uniform_pm1(seed: int, stream: int, idx: torch.Tensor) -> torch.Tensor:
    """Uniform in [-1, 1), f32."""
    return uniform01(seed, stream, idx) * 2.0 - 1.0


def randint(seed: int, stream: int, idx: torch.Tensor, span) -> torch.Tensor:
    """Integer in [0, span) (span: int or int64 tensor)."""
    return _lsr(hash64(seed, stream, idx), 1) % span


def normal(seed: int, stream: int, idx: torch.Tensor) -> torch.Tensor:
    """Standard normal by Box-Muller, f32."""
    u1 = 1.0 - uniform01(seed, stream, idx)           # (0, 1]
    u2 = uniform01(seed, stream + 7919, idx)
    return torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(6.283185307179586 * u2)


@dataclass
class CsrMatrix:
    rows: int
    cols: int
    row_ptr: torch.Tensor   # int32 [rows + 1]
    col_idx: torch.Tensor   # int32 [nnz]
    values: torch.Tensor    # float32 [nnz]

    @property
    def nnz(self) -> int:
        return int(self.values.numel())

    def to(self, device) -> "CsrMatrix":
        return CsrMatrix(self.rows, self.cols, self.row_ptr.to(device), self.col_idx.to(device),
                         self.values.to(device))

    def numpy(self):
        return (self.row_ptr.cpu().numpy(), self.col_idx.cpu().numpy(), self.values.cpu().numpy())


@dataclass
class BsrMatrix:
    rows: int
    cols: int
    block_size: int
    block_row_ptr: torch.Tensor   # int32 [rows/bs + 1]
    block_col_idx: torch.Tensor   # int32 [nnzb]
    block_values: torch.Tensor    # [nnzb * bs * bs], f32 or bf16

    @property
    def nnzb(self) -> int:
        return int(self.block_col_idx.numel())


# ---------------------------------------------------------------------------
# bytes and flops of one operator call (i32 = f32 = 4 bytes, bf16 = 2)
# ---------------------------------------------------------------------------

def spmv_bytes(rows: int, cols: int, nnz: int) -> int:
    return 8 * nnz + 4 * (rows + 1) + 4 * cols + 4 * rows


def spmm_bytes(rows: int, cols: int, nnz: int, n: int) -> int:
    return 8 * nnz + 4 * (rows + 1) + 4 * cols * n + 4 * rows * n


def bsr_bytes(rows: int, cols: int, nnzb: int, bs: int, n: int, elem: int = 2) -> int:
    return elem * nnzb * bs * bs + 4 * nnzb + 4 * (rows // bs + 1) + elem * cols * n + elem * rows * n


# ---------------------------------------------------------------------------
# the reference runner's own synthetic matrices
# ---------------------------------------------------------------------------

def reference_row_length(nnz_per_row: int, distribution: str, row: int) -> int:
    if distribution == "uniform":
        return nnz_per_row
    if distribution == "alternating":
        return 1 if row % 2 == 0 else 2 * nnz_per_row - 1
    if distribution == "skewed":
        return 8 * nnz_per_row - 7 if row % 8 == 7 else 1
    raise ValueError(f"unknown distribution: {distribution}")


def reference_synthetic(rows: int, cols: int, nnz_per_row: int, distribution: str) -> CsrMatrix:
    """Row lengths by `distribution`, column = position mod cols, value 1."""
    lengths = np.array([reference_row_length(nnz_per_row, distribution, r) for r in range(rows)], dtype=np.int64)
    row_ptr = np.concatenate([[0], np.cumsum(lengths)])
    nnz = int(row_ptr[-1])
    return CsrMatrix(rows, cols, torch.from_numpy(row_ptr.astype(np.int32)),
                     torch.from_numpy((np.arange(nnz) % cols).astype(np.int32)),
                     torch.ones(nnz, dtype=torch.float32))


# ---------------------------------------------------------------------------
# random CSR structure
# ---------------------------------------------------------------------------

def _finish_csr(rows: int, cols: int, lengths: torch.Tensor, draw, seed: int, device) -> CsrMatrix:
    """`draw(slot, row, attempt)` proposes a column for each slot; duplicates
    within a row are redrawn until every row has distinct columns, then slots
    are ordered by (row, column)."""
    lengths = lengths.to(torch.int64)
    row_ptr = torch.zeros(rows + 1, dtype=torch.int64, device=device)
    row_ptr[1:] = torch.cumsum(lengths, 0)
    nnz = int(row_ptr[-1])
    if nnz > (1 << 31) - 1:
        raise ValueError("matrix rows and NNZ must fit in the i32 CSR type")
    slot = torch.arange(nnz, dtype=torch.int64, device=device)
    row = torch.repeat_interleave(torch.arange(rows, dtype=torch.int64, device=device), lengths)
    col = draw(slot, row, 0)
    order = None
    for attempt in range(1, 64):
        key = row * cols + col
        skey, order = torch.sort(key)
        dup = skey[1:] == skey[:-1]
        if not bool(dup.any()):
            break
        redo = order[1:][dup]
        col[redo] = draw(redo, row[redo], attempt)
    else:
        raise RuntimeError("could not make the columns of every row distinct")
    col_sorted = col[order]
    values = uniform_pm1(seed, 101, slot)
    return CsrMatrix(rows, cols, row_ptr.to(torch.int32), col_sorted.to(torch.int32), values)


def uniform_csr(rows: int, cols: int, nnz_per_row: int, seed: int, device="cpu") -> CsrMatrix:
    """Exactly `nnz_per_row` distinct uniform-random columns per row, sorted."""
    if nnz_per_row > cols:
        raise ValueError("nnz_per_row exceeds the number of columns")
    lengths = torch.full((rows,), nnz_per_row, dtype=torch.int64, device=device)

    def draw(slot, row, attempt):
        return randint(seed, 11 + attempt, slot, cols)

    return _finish_csr(rows, cols, lengths, draw, seed, device)


def zipf_lengths(rows: int, exponent: float, min_len: int, max_len: int, seed: int, device="cpu") -> torch.Tensor:
    """Row lengths with P(len = k) proportional to k**-exponent on [min_len, max_len]
    (inverse CDF of the truncated Zipf distribution)."""
    k = torch.arange(min_len, max_len + 1, dtype=torch.float64, device=device)
    cdf = torch.cumsum(k.pow(-exponent), 0)
    cdf = cdf / cdf[-1]
    u = uniform01(seed, 3, torch.arange(rows, dtype=torch.int64, device=device), torch.float64)
    idx = torch.searchsorted(cdf, u, right=True).clamp_(max=max_len - min_len)
    return idx + min_len


def zipf_csr(rows: int, cols: int, exponent: float, min_len: int, max_len: int, seed: int,
             device="cpu") -> CsrMatrix:
    lengths = zipf_lengths(rows, exponent, min_len, min(max_len, cols), seed, device)

    def draw(slot, row, attempt):
        return randint(seed, 11 + attempt, slot, cols)

    return _finish_csr(rows, cols, lengths, draw, seed, device)


def banded_random_csr(rows: int, cols: int, band_nnz: int, half_band: int, random_nnz: int, seed: int,
                      device="cpu") -> CsrMatrix:
    """Per row: `band_nnz` distinct columns within +-half_band of the diagonal and
    `random_nnz` distinct uniform-random columns not already chosen, merged and sorted."""
    per_row = band_nnz + random_nnz
    if band_nnz > min(cols, half_band + 1) or per_row > cols:
        raise ValueError("row degree exceeds the available columns")
    lengths = torch.full((rows,), per_row, dtype=torch.int64, device=device)

    def draw(slot, row, attempt):
        in_band = (slot % per_row) < band_nnz
        lo = torch.clamp(row - half_band, min=0)
        hi = torch.clamp(row + half_band, max=cols - 1)
        lo = torch.where(in_band, lo, torch.zeros_like(lo))
        span = torch.where(in_band, hi - lo + 1, torch.full_like(lo, cols))
        return lo + randint(seed, 11 + attempt, slot, span)

    return _finish_csr(rows, cols, lengths, draw, seed, device)


def random_bsr(block_rows: int, block_cols: int, block_size: int, density: float, seed: int,
               dtype=torch.bfloat16, device="cpu") -> BsrMatrix:
    """Each block of the block grid present independently with probability
    `density`; block values standard normal, rounded to `dtype`."""
    grid = torch.arange(block_rows * block_cols, dtype=torch.int64, device=device)
    present = uniform01(seed, 5, grid, torch.float64) < density
    where = grid[present]
    brow = where // block_cols
    counts = torch.bincount(brow, minlength=block_rows)
    brp = torch.zeros(block_rows + 1, dtype=torch.int64, device=device)
    brp[1:] = torch.cumsum(counts, 0)
    nnzb = int(where.numel())
    vals = normal(seed, 6, torch.arange(nnzb * block_size * block_size, dtype=torch.int64, device=device))
    return BsrMatrix(block_rows * block_size, block_cols * block_size, block_size, brp.to(torch.int32),
                     (where % block_cols).to(torch.int32), vals.to(dtype))


def dense_uniform(shape, seed: int, stream: int = 201, device="cpu") -> torch.Tensor:
    n = int(np.prod(shape))
    return uniform_pm1(seed, stream, torch.arange(n, dtype=torch.int64, device=device)).reshape(shape)


def dense_normal(shape, seed: int, stream: int = 202, dtype=torch.bfloat16, device="cpu") -> torch.Tensor:
    n = int(np.prod(shape))
    return normal(seed, stream, torch.arange(n, dtype=torch.int64, device=device)).to(dtype).reshape(shape)


# ---------------------------------------------------------------------------
# the five benchmark configurations (scale < 1 shrinks them for tests)
# ---------------------------------------------------------------------------

def config_c1(device="cpu", rows: int = 4096):
    """CSR SpMV 4096 x 4096, 16 nnz per row; mapping wave-per-row, block 128."""
    a = uniform_csr(rows, rows, 16, seed=1, device=device)
    return a, dense_uniform((rows,), seed=1, device=device)


def config_c2(device="cpu", rows: int = 65536):
    """CSR SpMM 65536 x 65536, 32 nnz per row, B 65536 x 4; wave-per-row-tile, tile 4, block 64."""
    a = uniform_csr(rows, rows, 32, seed=2, device=device)
    return a, dense_uniform((rows, 4), seed=2, device=device)


def config_c3(device="cpu", rows: int = 4194304, max_len: int = 65536):
    """Power-law CSR SpMV: row lengths Zipf(1.8) on [1, 65536]."""
    a = zipf_csr(rows, rows, 1.8, 1, max_len, seed=3, device=device)
    return a, dense_uniform((rows,), seed=3, device=device)


def config_c4(device="cpu", rows: int = 2097152, n_rhs: int = 64):
    """CSR SpMM: 32 nnz within +-1024 of the diagonal plus 32 uniform-random nnz per row; B rows x 64."""
    a = banded_random_csr(rows, rows, 32, 1024, 32, seed=4, device=device)
    return a, dense_uniform((rows, n_rhs), seed=4, device=device)


def config_c5(device="cpu", block_grid: int = 1024, n_rhs: int = 512):
    """BSR SpMM: 16 x 16 bf16 blocks at 5% block density, B bf16 N(0,1)."""
    a = random_bsr(block_grid, block_grid, 16, 0.05, seed=5, device=device)
    return a, dense_normal((block_grid * 16, n_rhs), seed=5, device=device)
