"""ctypes binding of libsparsewave_b200.so (declared in include/sparsewave_b200.h).

The library is the product; this module only loads it and declares argument
types.  Loading fails loudly when the library has not been built: there is no
Python or CPU fallback for any operator.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libsparsewave_b200.so"

SWB_OK = 0
SWB_ERR_INVALID_OPTION = -1
SWB_ERR_INVALID_SHAPE = -2
SWB_ERR_INVALID_ARGUMENT = -3
SWB_ERR_CUDA = -4
SWB_ERR_UNSUPPORTED = -5
SWB_ERR_INVALID_DATA = -6
SWB_ERR_CAPACITY = -7


class SwbOptions(C.Structure):
    _fields_ = [
        ("mapping", C.c_int32),
        ("position_reduction", C.c_int32),
        ("spmm_mapping", C.c_int32),
        ("accumulate", C.c_int32),
        ("block_size", C.c_int64),
        ("wave_size", C.c_int64),
        ("position_block_size", C.c_int64),
        ("position_chunk_size", C.c_int64),
        ("spmm_block_size", C.c_int64),
        ("spmm_tile_size", C.c_int64),
        ("spmm_position_chunk_size", C.c_int64),
        ("wave_position_batch", C.c_int64),
    ]


class SwbLaunchShape(C.Structure):
    _fields_ = [
        ("logical_grid", C.c_int64),
        ("logical_block", C.c_int64),
        ("work_units", C.c_int64),
        ("kernels", C.c_int64),
        ("physical_grid", C.c_int64),
    ]


class Memref1D(C.Structure):
    """MLIR C-interface descriptor of a rank-1 memref (any 4-byte element)."""
    _fields_ = [("base", C.c_void_p), ("data", C.c_void_p), ("offset", C.c_int64),
                ("sizes", C.c_int64 * 1), ("strides", C.c_int64 * 1)]


class Memref2D(C.Structure):
    _fields_ = [("base", C.c_void_p), ("data", C.c_void_p), ("offset", C.c_int64),
                ("sizes", C.c_int64 * 2), ("strides", C.c_int64 * 2)]


_P = C.c_void_p
_I64 = C.c_int64
_CTX = C.c_void_p
_OPT = C.POINTER(SwbOptions)

# name -> (restype, argtypes); every symbol include/sparsewave_b200.h declares.
SIGNATURES = {
    "swb_create": (C.c_int, [C.POINTER(_CTX), C.c_int]),
    "swb_destroy": (None, [_CTX]),
    "swb_last_error": (C.c_char_p, [_CTX]),
    "swb_version": (C.c_char_p, []),
    "swb_kernel_launch_count": (_I64, [_CTX]),
    "swb_device_status": (C.c_int, [_CTX, _P, C.POINTER(C.c_int32)]),
    "swb_options_default": (None, [_OPT]),
    "swb_options_parse": (C.c_int, [_CTX, _OPT, C.c_char_p]),
    "swb_options_validate": (C.c_int, [_CTX, _OPT]),
    "swb_spmv": (C.c_int, [_CTX, _OPT, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P]),
    "swb_coo_spmv": (C.c_int, [_CTX, _OPT, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P]),
    "swb_spmm": (C.c_int, [_CTX, _OPT, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P]),
    "swb_bsr_spmm_f32": (C.c_int, [_CTX, _OPT, _I64, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P]),
    "swb_bsr_spmm_bf16": (C.c_int, [_CTX, _OPT, _I64, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P]),
    "swb_bsr16_spmm_bf16_static": (C.c_int, [_I64, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P, C.POINTER(C.c_int32)]),
    "swb_bsr16_static_status": (C.c_int, [_P, C.POINTER(C.c_int32)]),
    "swb_spmv_host": (C.c_int, [_CTX, _OPT, _I64, _I64, _I64, _P, _P, _P, _P, _P]),
    "swb_spmm_host": (C.c_int, [_CTX, _OPT, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P]),
    "swb_bsr_spmm_bf16_host": (C.c_int, [_CTX, _OPT, _I64, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P]),
    "swb_csr_upload": (C.c_int, [_CTX, _I64, _I64, _I64, _P, _P, _P, C.POINTER(C.c_void_p)]),
    "swb_csr_release": (None, [_CTX, _P]),
    "swb_spmv_resident_host": (C.c_int, [_CTX, _OPT, _P, _P, _P]),
    "swb_spmm_resident_host": (C.c_int, [_CTX, _OPT, _P, _I64, _P, _P]),
    "swb_probe_stream_gather": (C.c_int, [_CTX, _I64, _P, _P, _P, _P, _P]),
    "swb_spmv_sharded": (C.c_int, [_CTX, _OPT, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P]),
    "swb_spmm_sharded": (C.c_int, [_CTX, _OPT, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P]),
    "swb_csr_upload_rows": (C.c_int, [_CTX, _I64, _I64, _P, _P, _P, _I64, _I64, C.POINTER(C.c_void_p)]),
    "swb_spmv_sharded_host": (C.c_int, [_CTX, _OPT, _P, _P, _P]),
    "swb_spmm_sharded_host": (C.c_int, [_CTX, _OPT, _P, _I64, _P, _P]),
    "swb_bsr_upload": (C.c_int, [_CTX, _I64, _I64, _I64, _I64, _P, _P, _P, C.POINTER(C.c_void_p)]),
    "swb_bsr_release": (None, [_CTX, _P]),
    "swb_bsr_spmm_bf16_resident_host": (C.c_int, [_CTX, _OPT, _P, _I64, _P, _P]),
    "swb_check_csr_host": (C.c_int, [_CTX, _I64, _I64, _I64, _P, _P]),
    "swb_spmv_memref": (C.c_int, [_CTX, _OPT, _P, _P, _P, _P, _P, _P]),
    "swb_spmm_memref": (C.c_int, [_CTX, _OPT, _P, _P, _P, _P, _P, _P]),
    "swb_bsr_spmm_memref": (C.c_int, [_CTX, _OPT, _P, _P, _P, _P, _P, _I64, _P]),
    "_mlir_ciface_sparsewave_spmv": (None, [_P, _P, _P, _P, _P]),
    "_mlir_ciface_sparsewave_spmm": (None, [_P, _P, _P, _P, _P]),
    "_mlir_ciface_sparsewave_bsr_spmm": (None, [_P, _P, _P, _P, _P, _I64]),
    "swb_bundle_launch": (C.c_int, [_CTX, C.c_char_p, _I64, C.POINTER(_P), _P]),
    "swb_partition": (None, [_I64, _I64, _I64, _I64, C.POINTER(_I64), C.POINTER(_I64)]),
    "swb_chunk_bounds": (None, [_I64, _I64, _I64, _I64, C.POINTER(_I64), C.POINTER(_I64)]),
    "swb_row_at_position": (_I64, [_P, _I64, _I64]),
    "swb_launch_shape_query": (C.c_int, [_CTX, _OPT, _I64, _I64, _I64, C.POINTER(SwbLaunchShape)]),
    "swb_spmv_position_trace": (C.c_int, [_CTX, _OPT, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "swb_comm_unique_id": (C.c_int, [_P]),
    "swb_comm_init": (C.c_int, [_CTX, _P, C.c_int, C.c_int]),
    "swb_comm_allgather": (C.c_int, [_CTX, _P, _P, _I64, _P]),
    "swb_comm_destroy": (None, [_CTX]),
    "swb_shard_rows_by_nnz": (C.c_int, [_CTX, _P, _I64, _I64, _P]),
    "swb_comm_window_create": (C.c_int, [_CTX, _I64, C.POINTER(C.c_void_p)]),
    "swb_comm_window_allgather": (C.c_int, [_CTX, _P, _P]),
    "swb_comm_window_allgather_next": (C.c_int, [_CTX, _P, _P, C.POINTER(C.c_void_p)]),
    "swb_comm_window_destroy": (None, [_CTX]),
    "swb_plan_row_panels": (C.c_int, [_I64, _I64, _P, _I64, _P]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library and declares every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m sparsewave_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib
