"""Python host layer over the C ABI.

Argument order follows the operand lists of `sparsewave.spmv`,
`sparsewave.spmm` and `sparsewave.bsr_spmm` (row offsets, column indices,
values, dense input, output; include/.../IR/SparseWaveOps.td:37-43,108-115,
149-159 in the SparseWave tree) and options are written in the reference's
own spelling, e.g. ``"spmv-mapping=wave-per-row spmv-block-size=128"``.

PyTorch tensors are used for device memory and streams only; every operator
call goes to libsparsewave_b200.so.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch

from . import _lib
from ._lib import SwbLaunchShape, SwbOptions


class SparseWaveError(RuntimeError):
    """A C-ABI call returned a non-zero status; `.status` holds it."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def make_options(text: str = "", **fields) -> SwbOptions:
    """Default options, then `text` (reference spelling), then field overrides."""
    lib = _lib.load()
    o = SwbOptions()
    lib.swb_options_default(C.byref(o))
    if text:
        st = lib.swb_options_parse(None, C.byref(o), text.encode())
        if st != 0:
            raise SparseWaveError(st, lib.swb_last_error(None).decode())
    for k, v in fields.items():
        if not hasattr(o, k):
            raise AttributeError(f"swb_options has no field {k!r}")
        setattr(o, k, v)
    return o


def _dev_ptr(t: Optional[torch.Tensor], dtype: torch.dtype, name: str) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise TypeError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise TypeError(f"{name} must be contiguous")
    return t.data_ptr() if t.numel() > 0 else (t.data_ptr() or None)


def _host_ptr(a, dtype, name: str) -> Optional[int]:
    if isinstance(a, torch.Tensor):
        if a.is_cuda:
            raise TypeError(f"{name} must be a host tensor")
        if a.dtype != dtype or not a.is_contiguous():
            raise TypeError(f"{name} must be a contiguous {dtype} tensor")
        return a.data_ptr() or None
    np_dtype = {torch.int32: np.int32, torch.float32: np.float32, torch.uint16: np.uint16,
                torch.bfloat16: np.uint16, torch.int64: np.int64}[dtype]
    if not isinstance(a, np.ndarray) or a.dtype != np_dtype or not a.flags["C_CONTIGUOUS"]:
        raise TypeError(f"{name} must be a C-contiguous numpy array of {np_dtype}")
    return a.ctypes.data or None


class Context:
    """One swb_context: one host thread, one CUDA device."""

    def __init__(self, device: int = 0):
        self._lib = _lib.load()
        self._ctx = C.c_void_p()
        st = self._lib.swb_create(C.byref(self._ctx), int(device))
        if st != 0:
            raise SparseWaveError(st, self._lib.swb_last_error(None).decode())
        self.device = int(device)

    def close(self) -> None:
        if self._ctx:
            self.window = self.window_buffers = None
            self._lib.swb_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- helpers --------------------------------------------------------------
    def _check(self, st: int) -> None:
        if st != 0:
            raise SparseWaveError(st, self._lib.swb_last_error(self._ctx).decode())

    @staticmethod
    def _opts(options) -> SwbOptions:
        if isinstance(options, SwbOptions):
            return options
        return make_options(options or "")

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    @property
    def kernel_launches(self) -> int:
        return int(self._lib.swb_kernel_launch_count(self._ctx))

    def device_status(self) -> int:
        """Status word of kernels with bounded waits (synchronises the current stream); 0 = healthy."""
        v = C.c_int32(-1)
        self._check(self._lib.swb_device_status(self._ctx, self._stream(), C.byref(v)))
        return int(v.value)

    # -- multi-GPU communicator (NCCL, bound inside the library) ---------------------
    def comm_init(self, rank: int, world: int, group=None) -> None:
        """Creates this context's NCCL communicator.  Collective over `group` (a torch.distributed
        group, used only to hand rank 0's unique id to the other ranks)."""
        import torch.distributed as dist
        ident = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            buf = (C.c_uint8 * 128)()
            st = self._lib.swb_comm_unique_id(buf)
            if st != 0:
                raise SparseWaveError(st, self._lib.swb_last_error(None).decode())
            ident = torch.tensor(list(buf), dtype=torch.uint8)
        if world > 1:
            backend = dist.get_backend(group)
            t = ident.cuda(self.device) if backend == "nccl" else ident
            dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            ident = t.cpu()
        raw = (C.c_uint8 * 128)(*ident.tolist())
        self._check(self._lib.swb_comm_init(self._ctx, raw, int(world), int(rank)))
        self.comm_world, self.comm_rank = int(world), int(rank)

    def allgather(self, send: torch.Tensor, recv: torch.Tensor) -> torch.Tensor:
        """recv[k * n : (k + 1) * n] = rank k's `send` (n elements), on the current stream."""
        if not (send.is_cuda and recv.is_cuda and send.is_contiguous() and recv.is_contiguous()):
            raise TypeError("allgather needs contiguous CUDA tensors")
        nbytes = send.numel() * send.element_size()
        if recv.numel() * recv.element_size() != nbytes * getattr(self, "comm_world", 1):
            raise ValueError("recv must hold world x send bytes")
        self._check(self._lib.swb_comm_allgather(self._ctx, send.data_ptr(), recv.data_ptr(), nbytes, self._stream()))
        return recv

    # -- all-gather as one kernel of peer stores (processes of one node) ---------------
    def window_create(self, bytes_per_rank: int) -> torch.Tensor:
        """Collective over the communicator's ranks: allocates this rank's window of comm_world *
        bytes_per_rank bytes, maps the other ranks' windows and returns a uint8 tensor over the local one.
        `window_buffers` is a (2, comm_world * bytes_per_rank) view of it and of the second buffer behind it,
        which the sharded operators fill in turn."""
        ptr = C.c_void_p()
        self._check(self._lib.swb_comm_window_create(self._ctx, int(bytes_per_rank), C.byref(ptr)))
        self.window_bytes_per_rank = int(bytes_per_rank)

        class _Window:  # device memory owned by the library, exposed through the CUDA array interface
            __cuda_array_interface__ = {"shape": (2, int(bytes_per_rank) * self.comm_world), "typestr": "|u1",
                                        "data": (int(ptr.value), False), "version": 3, "strides": None}

        self.window_buffers = torch.as_tensor(_Window(), device=torch.device("cuda", self.device))
        self.window = self.window_buffers[0]
        return self.window

    def window_allgather(self, send: torch.Tensor) -> torch.Tensor:
        """Stores `send` (window_bytes_per_rank bytes, contiguous, 16-byte aligned) into every rank's window
        at this rank's offset, on the current stream; returns the local window."""
        if getattr(self, "window", None) is None:
            raise ValueError("the context has no window (window_create)")
        if not (send.is_cuda and send.is_contiguous()) or send.numel() * send.element_size() != self.window_bytes_per_rank:
            raise ValueError("send must be a contiguous CUDA tensor of window_bytes_per_rank bytes")
        self._check(self._lib.swb_comm_window_allgather(self._ctx, send.data_ptr(), self._stream()))
        return self.window

    def window_allgather_next(self, send: torch.Tensor) -> torch.Tensor:
        """The same exchange into the window's two buffers in turn (no round trip between the ranks before the
        stores when calls take turns); returns the buffer that this call fills."""
        if getattr(self, "window", None) is None:
            raise ValueError("the context has no window (window_create)")
        if not (send.is_cuda and send.is_contiguous()) or send.numel() * send.element_size() != self.window_bytes_per_rank:
            raise ValueError("send must be a contiguous CUDA tensor of window_bytes_per_rank bytes")
        where = C.c_void_p()
        self._check(self._lib.swb_comm_window_allgather_next(self._ctx, send.data_ptr(), self._stream(), C.byref(where)))
        return self.window_buffers[0 if where.value == self.window_buffers.data_ptr() else 1]

    def window_destroy(self) -> None:
        """Collective: unmaps the peers' windows and frees this rank's."""
        if getattr(self, "window", None) is not None:
            self.window = self.window_buffers = None
            self._lib.swb_comm_window_destroy(self._ctx)

    def validate(self, options) -> None:
        self._check(self._lib.swb_options_validate(self._ctx, C.byref(self._opts(options))))

    def launch_shape(self, options, rows: int, nnz: int, n_rhs: int = 0) -> SwbLaunchShape:
        out = SwbLaunchShape()
        self._check(self._lib.swb_launch_shape_query(self._ctx, C.byref(self._opts(options)), rows, nnz, n_rhs,
                                                     C.byref(out)))
        return out

    # -- operators on device tensors ---------------------------------------------
    def spmv(self, options, row_ptr, col_idx, val, x, y=None, *, rows=None):
        """y = A @ x for CSR A; returns y (allocated when not given)."""
        rows = int(row_ptr.numel() - 1 if rows is None else rows)
        cols, nnz = int(x.numel()), int(val.numel())
        if y is None:
            y = torch.empty(rows, dtype=torch.float32, device=x.device)
        o = self._opts(options)
        self._check(self._lib.swb_spmv(
            self._ctx, C.byref(o), rows, cols, nnz,
            _dev_ptr(row_ptr, torch.int32, "row_ptr"), _dev_ptr(col_idx, torch.int32, "col_idx"),
            _dev_ptr(val, torch.float32, "val"), _dev_ptr(x, torch.float32, "x"),
            _dev_ptr(y, torch.float32, "y"), self._stream()))
        return y

    def spmv_sharded(self, options, row_ptr, col_idx, val, x_owned, cols: int, y=None, *, rows=None):
        """Row shard of y = A @ x: gathers every rank's chunk of x (this rank's is `x_owned`), then runs the
        shard's kernel; collective over the context's communicator."""
        rows = int(row_ptr.numel() - 1 if rows is None else rows)
        if y is None:
            y = torch.empty(rows, dtype=torch.float32, device=val.device)
        o = self._opts(options)
        self._check(self._lib.swb_spmv_sharded(
            self._ctx, C.byref(o), rows, int(cols), int(val.numel()),
            _dev_ptr(row_ptr, torch.int32, "row_ptr"), _dev_ptr(col_idx, torch.int32, "col_idx"),
            _dev_ptr(val, torch.float32, "val"), _dev_ptr(x_owned, torch.float32, "x_owned"),
            _dev_ptr(y, torch.float32, "y"), self._stream()))
        return y

    def spmm_sharded(self, options, row_ptr, col_idx, val, B_owned, cols: int, C_out=None, *, rows=None):
        """Row shard of C = A @ B (see spmv_sharded); B_owned is this rank's rows of B."""
        rows = int(row_ptr.numel() - 1 if rows is None else rows)
        n_rhs = int(B_owned.shape[1])
        if C_out is None:
            C_out = torch.empty((rows, n_rhs), dtype=torch.float32, device=val.device)
        o = self._opts(options)
        self._check(self._lib.swb_spmm_sharded(
            self._ctx, C.byref(o), rows, int(cols), int(val.numel()), n_rhs,
            _dev_ptr(row_ptr, torch.int32, "row_ptr"), _dev_ptr(col_idx, torch.int32, "col_idx"),
            _dev_ptr(val, torch.float32, "val"), _dev_ptr(B_owned, torch.float32, "B_owned"),
            _dev_ptr(C_out, torch.float32, "C"), self._stream()))
        return C_out

    def probe_stream_gather(self, col_idx, val, x, sink=None):
        """Roofline probe: the col/val streams and the gather of x with no row logic (swb_probe_stream_gather)."""
        if sink is None:
            sink = torch.zeros(1024, dtype=torch.float32, device=x.device)
        self._check(self._lib.swb_probe_stream_gather(
            self._ctx, int(val.numel()), _dev_ptr(col_idx, torch.int32, "col_idx"),
            _dev_ptr(val, torch.float32, "val"), _dev_ptr(x, torch.float32, "x"),
            _dev_ptr(sink, torch.float32, "sink"), self._stream()))
        return sink

    def coo_spmv(self, options, rows: int, row_idx, col_idx, val, x, y=None):
        """y = A @ x for COO A (entries in any order, duplicates accumulate)."""
        cols, nnz = int(x.numel()), int(val.numel())
        if y is None:
            y = torch.empty(rows, dtype=torch.float32, device=x.device)
        o = self._opts(options)
        self._check(self._lib.swb_coo_spmv(
            self._ctx, C.byref(o), int(rows), cols, nnz, _dev_ptr(row_idx, torch.int32, "row_idx"),
            _dev_ptr(col_idx, torch.int32, "col_idx"), _dev_ptr(val, torch.float32, "val"),
            _dev_ptr(x, torch.float32, "x"), _dev_ptr(y, torch.float32, "y"), self._stream()))
        return y

    def spmv_position_trace(self, options, row_ptr, col_idx, val, x):
        """Position-mapped SpMV that also returns (row, worker, segment_end) per position."""
        rows, cols, nnz = int(row_ptr.numel() - 1), int(x.numel()), int(val.numel())
        y = torch.empty(rows, dtype=torch.float32, device=x.device)
        tr = [torch.full((max(nnz, 1),), -1, dtype=torch.int32, device=x.device) for _ in range(3)]
        o = self._opts(options)
        self._check(self._lib.swb_spmv_position_trace(
            self._ctx, C.byref(o), rows, cols, nnz,
            _dev_ptr(row_ptr, torch.int32, "row_ptr"), _dev_ptr(col_idx, torch.int32, "col_idx"),
            _dev_ptr(val, torch.float32, "val"), _dev_ptr(x, torch.float32, "x"),
            _dev_ptr(y, torch.float32, "y"), tr[0].data_ptr(), tr[1].data_ptr(), tr[2].data_ptr(),
            self._stream()))
        return y, tr[0][:nnz], tr[1][:nnz], tr[2][:nnz]

    def spmm(self, options, row_ptr, col_idx, val, B, C_out=None, *, rows=None):
        """C = A @ B for CSR A and row-major dense B (cols x N)."""
        rows = int(row_ptr.numel() - 1 if rows is None else rows)
        cols, n_rhs, nnz = int(B.shape[0]), int(B.shape[1]), int(val.numel())
        if C_out is None:
            C_out = torch.empty((rows, n_rhs), dtype=torch.float32, device=B.device)
        o = self._opts(options)
        self._check(self._lib.swb_spmm(
            self._ctx, C.byref(o), rows, cols, nnz, n_rhs,
            _dev_ptr(row_ptr, torch.int32, "row_ptr"), _dev_ptr(col_idx, torch.int32, "col_idx"),
            _dev_ptr(val, torch.float32, "val"), _dev_ptr(B, torch.float32, "B"),
            _dev_ptr(C_out, torch.float32, "C"), self._stream()))
        return C_out

    def bsr_spmm(self, options, block_row_ptr, block_col_idx, block_values, B, block_size: int, C_out=None):
        """C = A @ B for BSR A; f32 or bf16 chosen by the dtype of block_values."""
        brows = int(block_row_ptr.numel() - 1)
        rows, cols, n_rhs = brows * block_size, int(B.shape[0]), int(B.shape[1])
        nnzb = int(block_col_idx.numel())
        dt = block_values.dtype
        if dt not in (torch.float32, torch.bfloat16):
            raise TypeError("block_values must be float32 or bfloat16")
        if int(block_values.numel()) != nnzb * block_size * block_size:
            raise SparseWaveError(_lib.SWB_ERR_INVALID_SHAPE,
                                  "block values size must equal the number of blocks times block_size squared, "
                                  f"but got {int(block_values.numel())} and {nnzb} blocks")
        if C_out is None:
            C_out = torch.empty((rows, n_rhs), dtype=dt, device=B.device)
        fn = self._lib.swb_bsr_spmm_f32 if dt == torch.float32 else self._lib.swb_bsr_spmm_bf16
        o = self._opts(options)
        self._check(fn(self._ctx, C.byref(o), rows, cols, nnzb, block_size, n_rhs,
                       _dev_ptr(block_row_ptr, torch.int32, "block_row_ptr"),
                       _dev_ptr(block_col_idx, torch.int32, "block_col_idx"),
                       _dev_ptr(block_values, dt, "block_values"), _dev_ptr(B, dt, "B"),
                       _dev_ptr(C_out, dt, "C"), self._stream()))
        return C_out

    def bundle_launch(self, operation: str, n: int, args) -> None:
        """lrrt-style launch: five device pointers (rowOffsets, columnIndices, values, rhs, output)."""
        arr = (C.c_void_p * 5)(*[a.data_ptr() if isinstance(a, torch.Tensor) else a for a in args])
        self._check(self._lib.swb_bundle_launch(self._ctx, operation.encode(), int(n), arr, self._stream()))

    # -- operators on host buffers --------------------------------------------------
    def spmv_host(self, options, row_ptr, col_idx, val, x, y):
        rows, cols, nnz = len(row_ptr) - 1, len(x), len(val)
        o = self._opts(options)
        self._check(self._lib.swb_spmv_host(
            self._ctx, C.byref(o), rows, cols, nnz, _host_ptr(row_ptr, torch.int32, "row_ptr"),
            _host_ptr(col_idx, torch.int32, "col_idx"), _host_ptr(val, torch.float32, "val"),
            _host_ptr(x, torch.float32, "x"), _host_ptr(y, torch.float32, "y")))
        return y

    def spmm_host(self, options, row_ptr, col_idx, val, B, C_out):
        rows, cols, n_rhs, nnz = len(row_ptr) - 1, B.shape[0], B.shape[1], len(val)
        o = self._opts(options)
        self._check(self._lib.swb_spmm_host(
            self._ctx, C.byref(o), rows, cols, nnz, n_rhs, _host_ptr(row_ptr, torch.int32, "row_ptr"),
            _host_ptr(col_idx, torch.int32, "col_idx"), _host_ptr(val, torch.float32, "val"),
            _host_ptr(B, torch.float32, "B"), _host_ptr(C_out, torch.float32, "C")))
        return C_out

    def bsr_spmm_bf16_host(self, options, block_row_ptr, block_col_idx, block_values, B, block_size, C_out):
        brows = len(block_row_ptr) - 1
        rows, cols, n_rhs, nnzb = brows * block_size, B.shape[0], B.shape[1], len(block_col_idx)
        o = self._opts(options)
        self._check(self._lib.swb_bsr_spmm_bf16_host(
            self._ctx, C.byref(o), rows, cols, nnzb, block_size, n_rhs,
            _host_ptr(block_row_ptr, torch.int32, "block_row_ptr"),
            _host_ptr(block_col_idx, torch.int32, "block_col_idx"),
            _host_ptr(block_values, torch.bfloat16, "block_values"), _host_ptr(B, torch.bfloat16, "B"),
            _host_ptr(C_out, torch.bfloat16, "C")))
        return C_out

    def csr_upload(self, rows: int, cols: int, row_ptr, col_idx, val) -> "ResidentCsr":
        """Checks and copies a host CSR matrix to the device once; returns a handle for the
        `*_resident_host` calls (x / B in, y / C out per call)."""
        h = C.c_void_p()
        self._check(self._lib.swb_csr_upload(self._ctx, int(rows), int(cols), len(val),
                                             _host_ptr(row_ptr, torch.int32, "row_ptr"),
                                             _host_ptr(col_idx, torch.int32, "col_idx"),
                                             _host_ptr(val, torch.float32, "val"), C.byref(h)))
        return ResidentCsr(self, h, int(rows), int(cols))

    def csr_upload_rows(self, cols: int, row_ptr, col_idx, val, row_begin: int, row_end: int) -> "ResidentCsr":
        """Keeps rows [row_begin, row_end) of a host CSR matrix on the device (offsets rebased): the shard
        of a rank, for the `*_sharded_host` calls."""
        h = C.c_void_p()
        self._check(self._lib.swb_csr_upload_rows(self._ctx, len(row_ptr) - 1, int(cols),
                                                  _host_ptr(row_ptr, torch.int32, "row_ptr"),
                                                  _host_ptr(col_idx, torch.int32, "col_idx"),
                                                  _host_ptr(val, torch.float32, "val"), int(row_begin), int(row_end),
                                                  C.byref(h)))
        return ResidentCsr(self, h, int(row_end - row_begin), int(cols))

    def bsr_upload(self, cols: int, block_row_ptr, block_col_idx, block_values, block_size: int) -> "ResidentBsr":
        """Checks and copies a host bf16 BSR matrix to the device once; returns a handle for
        `ResidentBsr.spmm_host` (B in, C out per call)."""
        rows = (len(block_row_ptr) - 1) * block_size
        h = C.c_void_p()
        self._check(self._lib.swb_bsr_upload(self._ctx, rows, int(cols), len(block_col_idx), int(block_size),
                                             _host_ptr(block_row_ptr, torch.int32, "block_row_ptr"),
                                             _host_ptr(block_col_idx, torch.int32, "block_col_idx"),
                                             _host_ptr(block_values, torch.bfloat16, "block_values"), C.byref(h)))
        return ResidentBsr(self, h, rows, int(cols))

    def check_csr_host(self, rows, cols, row_ptr, col_idx) -> None:
        self._check(self._lib.swb_check_csr_host(self._ctx, rows, cols, len(col_idx),
                                                 _host_ptr(row_ptr, torch.int32, "row_ptr"),
                                                 _host_ptr(col_idx, torch.int32, "col_idx")))


class ResidentCsr:
    """A CSR matrix kept on the device by `Context.csr_upload`."""

    def __init__(self, ctx: Context, handle, rows: int, cols: int):
        self.ctx, self._h, self.rows, self.cols = ctx, handle, rows, cols

    def spmv_host(self, options, x, y):
        o = self.ctx._opts(options)
        self.ctx._check(self.ctx._lib.swb_spmv_resident_host(self.ctx._ctx, C.byref(o), self._h,
                                                             _host_ptr(x, torch.float32, "x"),
                                                             _host_ptr(y, torch.float32, "y")))
        return y

    def spmm_host(self, options, B, C_out):
        o = self.ctx._opts(options)
        self.ctx._check(self.ctx._lib.swb_spmm_resident_host(self.ctx._ctx, C.byref(o), self._h, int(B.shape[1]),
                                                             _host_ptr(B, torch.float32, "B"),
                                                             _host_ptr(C_out, torch.float32, "C")))
        return C_out

    def spmv_sharded_host(self, options, x_owned, y):
        """This rank's chunk of x in, the exchange and the shard's kernel on the device, this rank's rows out."""
        o = self.ctx._opts(options)
        self.ctx._check(self.ctx._lib.swb_spmv_sharded_host(self.ctx._ctx, C.byref(o), self._h,
                                                            _host_ptr(x_owned, torch.float32, "x_owned"),
                                                            _host_ptr(y, torch.float32, "y")))
        return y

    def spmm_sharded_host(self, options, B_owned, C_out):
        o = self.ctx._opts(options)
        self.ctx._check(self.ctx._lib.swb_spmm_sharded_host(self.ctx._ctx, C.byref(o), self._h, int(B_owned.shape[1]),
                                                            _host_ptr(B_owned, torch.float32, "B_owned"),
                                                            _host_ptr(C_out, torch.float32, "C")))
        return C_out

    def release(self) -> None:
        if self._h:
            self.ctx._lib.swb_csr_release(self.ctx._ctx, self._h)
            self._h = None


class ResidentBsr:
    """A bf16 BSR matrix kept on the device by `Context.bsr_upload`."""

    def __init__(self, ctx: Context, handle, rows: int, cols: int):
        self.ctx, self._h, self.rows, self.cols = ctx, handle, rows, cols

    def spmm_host(self, options, B, C_out):
        o = self.ctx._opts(options)
        self.ctx._check(self.ctx._lib.swb_bsr_spmm_bf16_resident_host(self.ctx._ctx, C.byref(o), self._h, int(B.shape[1]),
                                                                      _host_ptr(B, torch.bfloat16, "B"),
                                                                      _host_ptr(C_out, torch.bfloat16, "C")))
        return C_out

    def release(self) -> None:
        if self._h:
            self.ctx._lib.swb_bsr_release(self.ctx._ctx, self._h)
            self._h = None


def bsr16_spmm_bf16_static(block_row_ptr, block_col_idx, block_values, B, C_out=None, *, wait: bool = True):
    """16x16 bf16 BSR SpMM through the entry point that allocates no device memory
    (no context; status words in the library's fixed array).  With `wait` the call
    synchronises the current stream and raises if any CTA abandoned a wait."""
    lib = _lib.load()
    rows, cols, n_rhs = int(block_row_ptr.numel() - 1) * 16, int(B.shape[0]), int(B.shape[1])
    if C_out is None:
        C_out = torch.empty((rows, n_rhs), dtype=torch.bfloat16, device=B.device)
    gave_up = C.c_int32(-1)
    st = lib.swb_bsr16_spmm_bf16_static(
        rows, cols, int(block_col_idx.numel()), n_rhs, _dev_ptr(block_row_ptr, torch.int32, "block_row_ptr"),
        _dev_ptr(block_col_idx, torch.int32, "block_col_idx"), _dev_ptr(block_values, torch.bfloat16, "block_values"),
        _dev_ptr(B, torch.bfloat16, "B"), _dev_ptr(C_out, torch.bfloat16, "C"),
        torch.cuda.current_stream(B.device).cuda_stream, C.byref(gave_up) if wait else None)
    if st != 0:
        raise SparseWaveError(st, lib.swb_last_error(None).decode())
    if wait and gave_up.value != 0:
        raise SparseWaveError(_lib.SWB_ERR_CUDA, f"{gave_up.value} CTAs abandoned a barrier wait")
    return C_out


def bsr16_static_status() -> int:
    """CTAs of the most recent static call on the current device that abandoned a wait (synchronises the
    current stream; allocates nothing)."""
    lib = _lib.load()
    gave_up = C.c_int32(-1)
    st = lib.swb_bsr16_static_status(torch.cuda.current_stream().cuda_stream, C.byref(gave_up))
    if st != 0:
        raise SparseWaveError(st, lib.swb_last_error(None).decode())
    return int(gave_up.value)


# -- context-free helpers (host arithmetic only; need no GPU) ---------------------------

def partition(lower: int, upper: int, worker: int, count: int) -> tuple[int, int]:
    b, e = C.c_int64(), C.c_int64()
    _lib.load().swb_partition(lower, upper, worker, count, C.byref(b), C.byref(e))
    return b.value, e.value


def chunk_bounds(lower: int, upper: int, worker: int, factor: int) -> tuple[int, int]:
    b, e = C.c_int64(), C.c_int64()
    _lib.load().swb_chunk_bounds(lower, upper, worker, factor, C.byref(b), C.byref(e))
    return b.value, e.value


def row_at_position(row_ptr: np.ndarray, position: int) -> int:
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
    return int(_lib.load().swb_row_at_position(row_ptr.ctypes.data, len(row_ptr), position))


def shard_rows_by_nnz(row_ptr: np.ndarray, n_shards: int) -> np.ndarray:
    """nnz-balanced contiguous row shard boundaries (n_shards + 1 entries)."""
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
    out = np.zeros(n_shards + 1, dtype=np.int64)
    lib = _lib.load()
    st = lib.swb_shard_rows_by_nnz(None, row_ptr.ctypes.data, len(row_ptr) - 1, n_shards, out.ctypes.data)
    if st != 0:
        raise SparseWaveError(st, lib.swb_last_error(None).decode())
    return out


def plan_row_panels(row_ptr: np.ndarray, panel_nnz: int = 20000000) -> np.ndarray:
    """Row panels a resident matrix is cut into for the pipelined result copy (host array of row offsets
    in, first row of each panel followed by the row count out)."""
    lib = _lib.load()
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
    out = np.zeros(9, dtype=np.int64)
    rows = len(row_ptr) - 1
    count = lib.swb_plan_row_panels(rows, int(row_ptr[-1]), row_ptr.ctypes.data, int(panel_nnz), out.ctypes.data)
    return out[:count + 1]


def launch_shape(options, rows: int, nnz: int, n_rhs: int = 0) -> SwbLaunchShape:
    """Launch geometry without a context (auto batch assumes 148 SMs)."""
    lib = _lib.load()
    o = options if isinstance(options, SwbOptions) else make_options(options or "")
    out = SwbLaunchShape()
    st = lib.swb_launch_shape_query(None, C.byref(o), rows, nnz, n_rhs, C.byref(out))
    if st != 0:
        raise SparseWaveError(st, lib.swb_last_error(None).decode())
    return out


def validate_options(options) -> None:
    lib = _lib.load()
    o = options if isinstance(options, SwbOptions) else make_options(options or "")
    st = lib.swb_options_validate(None, C.byref(o))
    if st != 0:
        raise SparseWaveError(st, lib.swb_last_error(None).decode())
