"""ctypes face of libsparsewave_benchmark_utils.so (host-only): the four MLIR C-interface input loaders of the
SparseWave benchmark programs and the Matrix Market converter."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

from . import build as _build

_lib = None
_I64 = C.c_int64

LOADER_SYMBOLS = ("_mlir_ciface_loadCSRSpMVBenchmarkInputs", "_mlir_ciface_loadCOOSpMVBenchmarkInputs",
                  "_mlir_ciface_loadSpMMBenchmarkInputs", "_mlir_ciface_loadBSRSpMMBenchmarkInputs")


class Memref1(C.Structure):
    _fields_ = [("base", C.c_void_p), ("data", C.c_void_p), ("offset", _I64), ("sizes", _I64 * 1),
                ("strides", _I64 * 1)]


class Memref2(C.Structure):
    _fields_ = [("base", C.c_void_p), ("data", C.c_void_p), ("offset", _I64), ("sizes", _I64 * 2),
                ("strides", _I64 * 2)]


def memref(a: np.ndarray):
    """Descriptor of a C-contiguous numpy array of rank 1 or 2 (the array must outlive the call)."""
    if a.ndim == 1:
        return Memref1(a.ctypes.data, a.ctypes.data, 0, (_I64 * 1)(a.shape[0]), (_I64 * 1)(1))
    return Memref2(a.ctypes.data, a.ctypes.data, 0, (_I64 * 2)(*a.shape), (_I64 * 2)(a.shape[1], 1))


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        path = _build.LOADERS
        if not path.exists():
            _build.build_loaders()
        _lib = C.CDLL(str(path))
        _lib.swbu_convert_matrix_market.restype = C.c_int
        _lib.swbu_convert_matrix_market.argtypes = [C.c_char_p, C.c_char_p, _I64, C.c_char_p, C.c_char_p, C.c_size_t]
        for name in LOADER_SYMBOLS:
            getattr(_lib, name).restype = None
    return _lib


def convert_matrix_market(mtx_path, fmt: str, out_path, block_size: int = 0) -> None:
    """Matrix Market file -> SWCSR001 / SWCOO001 / SWBSR001 (`fmt` = "csr", "coo" or "bsr")."""
    err = C.create_string_buffer(512)
    st = load().swbu_convert_matrix_market(os.fsencode(Path(mtx_path)), fmt.encode(), int(block_size),
                                           os.fsencode(Path(out_path)), err, len(err))
    if st != 0:
        raise ValueError(err.value.decode())


def _call(symbol: str, env: str, path, arrays):
    os.environ[env] = str(path)
    descriptors = [memref(a) for a in arrays]
    getattr(load(), symbol)(*[C.byref(d) for d in descriptors])
    return arrays


def load_csr_spmv_inputs(path, rows: int, cols: int, nnz: int):
    """(row_ptr, col_idx, values, x == 1, expected) of an SWCSR001 file; aborts the process on a bad file."""
    a = [np.empty(rows + 1, np.int32), np.empty(nnz, np.int32), np.empty(nnz, np.float32),
         np.empty(cols, np.float32), np.empty(rows, np.float32)]
    return _call(LOADER_SYMBOLS[0], "SPARSEWAVE_BENCHMARK_CSR", path, a)


def load_coo_spmv_inputs(path, rows: int, cols: int, nnz: int):
    a = [np.empty(nnz, np.int32), np.empty(nnz, np.int32), np.empty(nnz, np.float32),
         np.empty(cols, np.float32), np.empty(rows, np.float32)]
    return _call(LOADER_SYMBOLS[1], "SPARSEWAVE_BENCHMARK_COO", path, a)


def load_spmm_inputs(path, rows: int, cols: int, nnz: int, n: int):
    a = [np.empty(rows + 1, np.int32), np.empty(nnz, np.int32), np.empty(nnz, np.float32),
         np.empty((cols, n), np.float32), np.empty((rows, n), np.float32)]
    return _call(LOADER_SYMBOLS[2], "SPARSEWAVE_BENCHMARK_CSR", path, a)


def load_bsr_spmm_inputs(path, rows: int, cols: int, nnzb: int, block_size: int, n: int):
    a = [np.empty(rows // block_size + 1, np.int32), np.empty(nnzb, np.int32),
         np.empty(nnzb * block_size * block_size, np.float32), np.empty((cols, n), np.float32),
         np.empty((rows, n), np.float32)]
    return _call(LOADER_SYMBOLS[3], "SPARSEWAVE_BENCHMARK_BSR", path, a)
