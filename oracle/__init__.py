"""Python face of the test oracle (oracle/swb_oracle.c) and of the reference's
own CPU helper when it was compiled (oracle/_ref).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke test and by the
CPU-baseline legs of bench.py.  The product package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import tempfile
from pathlib import Path

import numpy as np

from . import build as _build

_HERE = Path(__file__).resolve().parent
_lib = None
_ref = None

_I64 = C.c_int64
_P = C.c_void_p


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = _build.ORACLE_LIB
        if not path.exists() or _build._stale(path, [_build.ORACLE_SRC]):
            _build.build_oracle()
        _lib = C.CDLL(str(path))
        _lib.oracle_row_at_position.restype = _I64
        _lib.oracle_count_mismatches_reference.restype = _I64
        _lib.oracle_count_mismatches_bound.restype = _I64
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u16(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint16
    return a


def _ptr(a):
    return C.c_void_p(a.ctypes.data) if a is not None else None


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> int:
    """Sets the thread count of the parallel loops (`parallel=True`); returns the count now in effect."""
    lib().oracle_set_num_threads(C.c_int(int(n)))
    return num_threads()


def use_all_cores() -> int:
    """One thread per core this process may run on, whatever OMP_NUM_THREADS says (multi-process
    launchers export OMP_NUM_THREADS=1 to every rank)."""
    return set_num_threads(len(os.sched_getaffinity(0)))


def csr_spmv(row_ptr, col, val, x, parallel: bool = False) -> np.ndarray:
    row_ptr, col, val, x = _i32(row_ptr), _i32(col), _f32(val), _f32(x)
    rows = len(row_ptr) - 1
    y = np.empty(rows, dtype=np.float32)
    fn = lib().oracle_csr_spmv_omp if parallel else lib().oracle_csr_spmv
    fn(_I64(rows), _ptr(row_ptr), _ptr(col), _ptr(val), _ptr(x), _ptr(y))
    return y


def coo_spmv(rows, row, col, val, x) -> np.ndarray:
    row, col, val, x = _i32(row), _i32(col), _f32(val), _f32(x)
    y = np.empty(rows, dtype=np.float32)
    lib().oracle_coo_spmv(_I64(rows), _I64(len(val)), _ptr(row), _ptr(col), _ptr(val), _ptr(x), _ptr(y))
    return y


def csr_spmm(row_ptr, col, val, B, parallel: bool = False) -> np.ndarray:
    row_ptr, col, val, B = _i32(row_ptr), _i32(col), _f32(val), _f32(B)
    rows, n = len(row_ptr) - 1, B.shape[1]
    out = np.empty((rows, n), dtype=np.float32)
    fn = lib().oracle_csr_spmm_omp if parallel else lib().oracle_csr_spmm
    fn(_I64(rows), _I64(n), _ptr(row_ptr), _ptr(col), _ptr(val), _ptr(B), _ptr(out))
    return out


def csr_abs_bound(row_ptr, col, val, B) -> np.ndarray:
    """sum_p |val[p] * B[col[p], j]| per output element, f64 (B may be a vector)."""
    row_ptr, col, val, B = _i32(row_ptr), _i32(col), _f32(val), _f32(B)
    vec = B.ndim == 1
    B2 = B.reshape(-1, 1) if vec else B
    rows, n = len(row_ptr) - 1, B2.shape[1]
    out = np.empty((rows, n), dtype=np.float64)
    lib().oracle_csr_abs_bound(_I64(rows), _I64(n), _ptr(row_ptr), _ptr(col), _ptr(val), _ptr(B2), _ptr(out))
    return out[:, 0] if vec else out


def bsr_spmm_f32(brp, bci, bv, B, bs: int) -> np.ndarray:
    brp, bci, bv, B = _i32(brp), _i32(bci), _f32(bv), _f32(B)
    rows, n = (len(brp) - 1) * bs, B.shape[1]
    out = np.empty((rows, n), dtype=np.float32)
    lib().oracle_bsr_spmm_f32(_I64(rows), _I64(bs), _I64(n), _ptr(brp), _ptr(bci), _ptr(bv), _ptr(B), _ptr(out))
    return out


def bsr_spmm_bf16(brp, bci, bv_bits, B_bits, bs: int):
    """bf16 bit patterns in (uint16); returns (C bits uint16, C before rounding f32)."""
    brp, bci, bv_bits, B_bits = _i32(brp), _i32(bci), _u16(bv_bits), _u16(B_bits)
    rows, n = (len(brp) - 1) * bs, B_bits.shape[1]
    out = np.empty((rows, n), dtype=np.uint16)
    out32 = np.empty((rows, n), dtype=np.float32)
    lib().oracle_bsr_spmm_bf16(_I64(rows), _I64(bs), _I64(n), _ptr(brp), _ptr(bci), _ptr(bv_bits), _ptr(B_bits),
                               _ptr(out), _ptr(out32))
    return out, out32


def bsr_abs_bound_bf16(brp, bci, bv_bits, B_bits, bs: int) -> np.ndarray:
    """Per output of a bf16 BSR SpMM: the sum of |a * b| over its terms, f64."""
    brp, bci, bv_bits, B_bits = _i32(brp), _i32(bci), _u16(bv_bits), _u16(B_bits)
    rows, n = (len(brp) - 1) * bs, B_bits.shape[1]
    out = np.empty((rows, n), dtype=np.float64)
    lib().oracle_bsr_abs_bound_bf16(_I64(rows), _I64(bs), _I64(n), _ptr(brp), _ptr(bci), _ptr(bv_bits), _ptr(B_bits),
                                    _ptr(out))
    return out


def bf16_mismatches(got_bits, want_bits, want_f32, bound) -> tuple[int, int]:
    """Compares bf16 outputs (bit patterns) with the oracle's: (outputs further than one bf16 ulp from the
    oracle's bits, counted where the exact sum is at least 2**-6 of the size of its terms; outputs of
    cancelling sums, |sum| below that, whose error exceeds 1e-2 * 2**-6 of the size of their terms)."""
    got = np.ascontiguousarray(got_bits).astype(np.uint16).ravel()
    want = np.ascontiguousarray(want_bits).astype(np.uint16).ravel()
    f32 = np.ascontiguousarray(want_f32, dtype=np.float32).ravel()
    S = np.ascontiguousarray(bound, dtype=np.float64).ravel()

    def ordered(bits):  # bf16 bit patterns -> integers in value order
        b = bits.astype(np.int32)
        return np.where(b & 0x8000, -(b & 0x7FFF), b)

    regular = np.abs(f32) >= S * 2.0 ** -6
    ulps = np.abs(ordered(got) - ordered(want))
    got_f32 = (got.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    tiny_bad = (~regular) & (np.abs(got_f32 - f32) > 1e-2 * 2.0 ** -6 * S + 1e-30)
    return int(np.sum(regular & (ulps > 1))), int(np.sum(tiny_bad))


def partition(lower, upper, worker, count):
    b, e = _I64(), _I64()
    lib().oracle_partition(_I64(lower), _I64(upper), _I64(worker), _I64(count), C.byref(b), C.byref(e))
    return b.value, e.value


def chunk_bounds(lower, upper, worker, factor):
    b, e = _I64(), _I64()
    lib().oracle_chunk_bounds(_I64(lower), _I64(upper), _I64(worker), _I64(factor), C.byref(b), C.byref(e))
    return b.value, e.value


def row_at_position(row_ptr, position) -> int:
    row_ptr = _i32(row_ptr)
    return int(lib().oracle_row_at_position(_ptr(row_ptr), _I64(len(row_ptr)), _I64(position)))


def _position_call(fn, row_ptr, col, val, x, extra, trace):
    row_ptr, col, val, x = _i32(row_ptr), _i32(col), _f32(val), _f32(x)
    rows, nnz = len(row_ptr) - 1, len(val)
    y = np.empty(rows, dtype=np.float32)
    tr = [np.full(max(nnz, 1), -1, dtype=np.int32) for _ in range(3)] if trace else [None] * 3
    fn(_I64(rows), _I64(nnz), *[_I64(v) for v in extra], _ptr(row_ptr), _ptr(col), _ptr(val), _ptr(x), _ptr(y),
       _ptr(tr[0]), _ptr(tr[1]), _ptr(tr[2]))
    if trace:
        return y, tr[0][:nnz], tr[1][:nnz], tr[2][:nnz]
    return y


def spmv_thread_position(row_ptr, col, val, x, chunk=1, segmented=False, trace=False):
    fn = lib().oracle_spmv_thread_position_segmented if segmented else lib().oracle_spmv_thread_position_atomic
    return _position_call(fn, row_ptr, col, val, x, [chunk], trace)


def spmv_wave_position(row_ptr, col, val, x, block=256, batch=1, trace=False):
    return _position_call(lib().oracle_spmv_wave_position, row_ptr, col, val, x, [block, batch], trace)


def spmm_thread_position(row_ptr, col, val, B, chunk=1) -> np.ndarray:
    row_ptr, col, val, B = _i32(row_ptr), _i32(col), _f32(val), _f32(B)
    rows, n, nnz = len(row_ptr) - 1, B.shape[1], len(val)
    out = np.empty((rows, n), dtype=np.float32)
    lib().oracle_spmm_thread_position(_I64(rows), _I64(nnz), _I64(n), _I64(chunk), _ptr(row_ptr), _ptr(col),
                                      _ptr(val), _ptr(B), _ptr(out))
    return out


def count_mismatches_reference(actual, expected) -> int:
    a, e = _f32(actual).ravel(), _f32(expected).ravel()
    return int(lib().oracle_count_mismatches_reference(_ptr(a), _ptr(e), _I64(a.size)))


def count_mismatches_bound(actual, expected, bound, rel=1e-5) -> int:
    a, e = _f32(actual).ravel(), _f32(expected).ravel()
    b = np.ascontiguousarray(bound, dtype=np.float64).ravel()
    return int(lib().oracle_count_mismatches_bound(_ptr(a), _ptr(e), _ptr(b), C.c_double(rel), _I64(a.size)))


# ---------------------------------------------------------------------------
# The reference's own CPU helper (benchmark/SparseBenchmarkUtils.cpp compiled
# unmodified).  Its loaders read a binary matrix named by an environment
# variable, overwrite the dense operand with a fixed pattern and compute the
# expected output; here they are driven through their MLIR C-interface
# descriptors.
# ---------------------------------------------------------------------------

class _M1(C.Structure):
    _fields_ = [("base", _P), ("data", _P), ("offset", _I64), ("sizes", _I64 * 1), ("strides", _I64 * 1)]


class _M2(C.Structure):
    _fields_ = [("base", _P), ("data", _P), ("offset", _I64), ("sizes", _I64 * 2), ("strides", _I64 * 2)]


def _m1(a):
    return _M1(a.ctypes.data, a.ctypes.data, 0, (_I64 * 1)(a.shape[0]), (_I64 * 1)(1))


def _m2(a):
    return _M2(a.ctypes.data, a.ctypes.data, 0, (_I64 * 2)(*a.shape), (_I64 * 2)(a.shape[1], 1))


def reference_available() -> bool:
    return _build.REF_LIB.exists() or _build.reference_root() is not None


def _reflib() -> C.CDLL:
    global _ref
    if _ref is None:
        path = _build.build_reference()
        if path is None:
            raise RuntimeError("the reference CPU helper is not built (oracle/_ref is empty)")
        _ref = C.CDLL(str(path))
    return _ref


def reference_csr_spmv(csr_file: Path, rows, cols, nnz):
    """Runs loadCSRSpMVBenchmarkInputs: returns (row_ptr, col, val, x == 1, expected)."""
    rp, ci = np.empty(rows + 1, np.int32), np.empty(nnz, np.int32)
    v, x, y = np.empty(nnz, np.float32), np.empty(cols, np.float32), np.empty(rows, np.float32)
    os.environ["SPARSEWAVE_BENCHMARK_CSR"] = str(csr_file)
    d = [_m1(a) for a in (rp, ci, v, x, y)]
    _reflib()._mlir_ciface_loadCSRSpMVBenchmarkInputs(*[C.byref(m) for m in d])
    return rp, ci, v, x, y


def reference_coo_spmv(coo_file: Path, rows, cols, nnz):
    """Runs loadCOOSpMVBenchmarkInputs: returns (row, col, val, x == 1, expected)."""
    ri, ci = np.empty(nnz, np.int32), np.empty(nnz, np.int32)
    v, x, y = np.empty(nnz, np.float32), np.empty(cols, np.float32), np.empty(rows, np.float32)
    os.environ["SPARSEWAVE_BENCHMARK_COO"] = str(coo_file)
    d = [_m1(a) for a in (ri, ci, v, x, y)]
    _reflib()._mlir_ciface_loadCOOSpMVBenchmarkInputs(*[C.byref(m) for m in d])
    return ri, ci, v, x, y


def reference_csr_spmm(csr_file: Path, rows, cols, nnz, n):
    """Runs loadSpMMBenchmarkInputs: returns (row_ptr, col, val, B pattern, expected)."""
    rp, ci, v = np.empty(rows + 1, np.int32), np.empty(nnz, np.int32), np.empty(nnz, np.float32)
    B, out = np.empty((cols, n), np.float32), np.empty((rows, n), np.float32)
    os.environ["SPARSEWAVE_BENCHMARK_CSR"] = str(csr_file)
    _reflib()._mlir_ciface_loadSpMMBenchmarkInputs(C.byref(_m1(rp)), C.byref(_m1(ci)), C.byref(_m1(v)),
                                                   C.byref(_m2(B)), C.byref(_m2(out)))
    return rp, ci, v, B, out


def reference_bsr_spmm(bsr_file: Path, rows, cols, nnzb, bs, n):
    """Runs loadBSRSpMMBenchmarkInputs: returns (brp, bci, bv, B pattern, expected)."""
    brp, bci = np.empty(rows // bs + 1, np.int32), np.empty(nnzb, np.int32)
    bv = np.empty(nnzb * bs * bs, np.float32)
    B, out = np.empty((cols, n), np.float32), np.empty((rows, n), np.float32)
    os.environ["SPARSEWAVE_BENCHMARK_BSR"] = str(bsr_file)
    _reflib()._mlir_ciface_loadBSRSpMMBenchmarkInputs(C.byref(_m1(brp)), C.byref(_m1(bci)), C.byref(_m1(bv)),
                                                      C.byref(_m2(B)), C.byref(_m2(out)))
    return brp, bci, bv, B, out
