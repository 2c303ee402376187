"""Row sharding of one CSR / BSR operator over the GPUs of one node.

Not a reference feature (the reference is single GPU).  Rows are cut into
contiguous shards balanced by nnz (`swb_shard_rows_by_nnz`); rank k keeps the
row offsets of its rows rebased to zero, its slice of the column indices and
values, global column numbering, and the matching rows of the output.  The
dense operand (x for SpMV, B for SpMM) is owned in equal contiguous row chunks
and gathered into every rank's own full copy with one NCCL all-gather before
the local kernel runs; outputs stay sharded.

One process per GPU; `torch.distributed` is the plumbing (NCCL on GPUs, gloo in
the CPU tests of this host logic).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from . import api


def dense_chunk(n_rows: int, world: int) -> int:
    """Rows of the dense operand owned by each rank: ceil(n_rows / world); rank k
    owns [k * chunk, min((k + 1) * chunk, n_rows))."""
    return -(-n_rows // world)


def owned_dense_range(n_rows: int, world: int, rank: int) -> tuple[int, int]:
    c = dense_chunk(n_rows, world)
    return min(rank * c, n_rows), min((rank + 1) * c, n_rows)


@dataclass
class CsrShard:
    """Rows [row_begin, row_end) of a CSR matrix, offsets rebased to zero."""
    rank: int
    world: int
    rows_total: int
    cols: int
    row_begin: int
    row_end: int
    row_ptr: torch.Tensor
    col_idx: torch.Tensor
    values: torch.Tensor

    @property
    def rows(self) -> int:
        return self.row_end - self.row_begin

    @property
    def nnz(self) -> int:
        return int(self.values.numel())


def shard_boundaries(row_ptr, world: int) -> np.ndarray:
    """nnz-balanced row boundaries (world + 1 entries) from the full row offsets."""
    if isinstance(row_ptr, torch.Tensor):
        row_ptr = row_ptr.cpu().numpy()
    return api.shard_rows_by_nnz(row_ptr, world)


def shard_csr(row_ptr: torch.Tensor, col_idx: torch.Tensor, values: torch.Tensor, cols: int, rank: int,
              world: int, boundaries: Optional[np.ndarray] = None) -> CsrShard:
    """Cuts rank's shard out of the full matrix (tensors on any device)."""
    rows_total = int(row_ptr.numel() - 1)
    if boundaries is None:
        boundaries = shard_boundaries(row_ptr, world)
    r0, r1 = int(boundaries[rank]), int(boundaries[rank + 1])
    p0, p1 = int(row_ptr[r0]), int(row_ptr[r1])
    local_ptr = (row_ptr[r0:r1 + 1] - p0).to(torch.int32).contiguous()
    # Copies, not views: a view that starts at position p0 is 16-byte aligned only when p0 is a multiple of 4,
    # and the 128-bit loads of the vectorised kernels need that alignment (a misaligned shard silently ran the
    # scalar kernels, 1.7x slower on a 11.5 M-nonzero shard).
    return CsrShard(rank, world, rows_total, cols, r0, r1, local_ptr, col_idx[p0:p1].clone(),
                    values[p0:p1].clone())


@dataclass
class BsrShard:
    """Block rows [block_row_begin, block_row_end) of a BSR matrix, block-row offsets rebased to zero."""
    rank: int
    world: int
    cols: int
    block_size: int
    block_row_begin: int
    block_row_end: int
    block_row_ptr: torch.Tensor
    block_col_idx: torch.Tensor
    block_values: torch.Tensor  # flat [nnzb * bs * bs], row-major inside a block

    @property
    def rows(self) -> int:
        return (self.block_row_end - self.block_row_begin) * self.block_size

    @property
    def row_begin(self) -> int:
        return self.block_row_begin * self.block_size

    @property
    def row_end(self) -> int:
        return self.block_row_end * self.block_size

    @property
    def nnzb(self) -> int:
        return int(self.block_col_idx.numel())


def shard_bsr(block_row_ptr: torch.Tensor, block_col_idx: torch.Tensor, block_values: torch.Tensor, cols: int,
              block_size: int, rank: int, world: int, boundaries: Optional[np.ndarray] = None) -> BsrShard:
    """Cuts rank's block rows out of the full BSR matrix: contiguous block rows balanced by the number of
    blocks (the same boundary rule as the CSR shards, applied to the block-row offsets)."""
    if boundaries is None:
        boundaries = shard_boundaries(block_row_ptr, world)
    r0, r1 = int(boundaries[rank]), int(boundaries[rank + 1])
    p0, p1 = int(block_row_ptr[r0]), int(block_row_ptr[r1])
    per_block = block_size * block_size
    local_ptr = (block_row_ptr[r0:r1 + 1] - p0).to(torch.int32).contiguous()
    return BsrShard(rank, world, cols, block_size, r0, r1, local_ptr, block_col_idx[p0:p1].clone(),
                    block_values.reshape(-1)[p0 * per_block:p1 * per_block].clone())


def allgather_dense(owned: torch.Tensor, n_rows: int, out: Optional[torch.Tensor] = None, group=None,
                    ctx: Optional[api.Context] = None) -> torch.Tensor:
    """Gathers every rank's chunk of the dense operand (leading dimension split
    by `dense_chunk`) into a full copy on this rank; returns its first n_rows rows.
    With a context that owns a communicator (`Context.comm_init`) the exchange is the
    library's own NCCL all-gather on the current stream; otherwise torch.distributed's."""
    native = ctx is not None and getattr(ctx, "comm_world", 0) > 1
    world = ctx.comm_world if native else (dist.get_world_size(group) if dist.is_initialized() else 1)
    chunk = dense_chunk(n_rows, world)
    tail = tuple(owned.shape[1:])
    window = getattr(ctx, "window", None) if native else None
    if window is not None:
        # the library's own all-gather kernel (peer stores over NVLink) into the library-owned window
        if chunk * int(np.prod(tail, dtype=np.int64)) * owned.element_size() != ctx.window_bytes_per_rank:
            raise ValueError("the context's window was created for another operand size")
        send = owned
        if owned.shape[0] != chunk:
            send = torch.zeros((chunk,) + tail, dtype=owned.dtype, device=owned.device)
            send[:owned.shape[0]].copy_(owned)
        full = ctx.window_allgather(send.contiguous()).view(owned.dtype).view((chunk * world,) + tail)
        return full[:n_rows]
    if out is None:
        out = torch.empty((chunk * world,) + tail, dtype=owned.dtype, device=owned.device)
    if world == 1:
        out[:owned.shape[0]].copy_(owned)
        return out[:n_rows]
    send = owned
    if owned.shape[0] != chunk:  # the last rank's chunk may be short: pad to the common size
        send = torch.zeros((chunk,) + tail, dtype=owned.dtype, device=owned.device)
        send[:owned.shape[0]].copy_(owned)
    if native:
        ctx.allgather(send.contiguous().view(-1), out.view(-1))
    else:
        dist.all_gather_into_tensor(out.view(-1), send.contiguous().view(-1), group=group)
    return out[:n_rows]


def split_by_column_range(shard: CsrShard, lo: int, hi: int) -> tuple[CsrShard, CsrShard]:
    """Splits a row shard into the entries whose column lies in [lo, hi) and the rest; both keep
    every row (possibly empty), the order of the entries inside a row and global column numbers."""
    rows = shard.rows
    rp = shard.row_ptr.to(torch.int64)
    lengths = rp[1:] - rp[:-1]
    row_of = torch.repeat_interleave(torch.arange(rows, dtype=torch.int64, device=rp.device), lengths)
    inside = (shard.col_idx >= lo) & (shard.col_idx < hi)
    parts = []
    for mask in (inside, ~inside):
        counts = torch.bincount(row_of[mask], minlength=rows)
        ptr = torch.zeros(rows + 1, dtype=torch.int64, device=rp.device)
        ptr[1:] = torch.cumsum(counts, 0)
        parts.append(CsrShard(shard.rank, shard.world, shard.rows_total, shard.cols, shard.row_begin, shard.row_end,
                              ptr.to(torch.int32), shard.col_idx[mask].contiguous(), shard.values[mask].contiguous()))
    return parts[0], parts[1]


class OverlappedShardedOperator:
    """Row shard whose entries are split by column ownership: the entries in this rank's own chunk of
    the dense operand run while the all-gather of the other chunks is in flight on a second stream, the
    rest run afterwards and add to the same output (`accumulate`).  Needs the context's own communicator
    (`Context.comm_init`) and a mapping that can accumulate (position mappings for SpMV, wave-per-row-tile
    or thread-per-position for SpMM)."""

    def __init__(self, ctx: api.Context, shard: CsrShard, options):
        if getattr(ctx, "comm_world", 0) != shard.world:
            raise ValueError("OverlappedShardedOperator needs Context.comm_init over the shard's ranks")
        self.ctx, self.shard = ctx, shard
        self.lo, self.hi = owned_dense_range(shard.cols, shard.world, shard.rank)
        self.local, self.remote = split_by_column_range(shard, self.lo, self.hi)
        base = options if isinstance(options, api.SwbOptions) else api.make_options(options or "")
        self.opts_first = api.SwbOptions.from_buffer_copy(base)
        self.opts_rest = api.SwbOptions.from_buffer_copy(base)
        self.opts_rest.accumulate = 1
        self.side = torch.cuda.Stream(device=shard.row_ptr.device)
        self._full = None

    def _run(self, owned: torch.Tensor, out, call):
        s, world = self.shard, self.shard.world
        chunk = dense_chunk(s.cols, world)
        shape = (chunk * world,) + tuple(owned.shape[1:])
        if self._full is None or tuple(self._full.shape) != shape or self._full.dtype != owned.dtype:
            self._full = torch.zeros(shape, dtype=owned.dtype, device=owned.device)
        full = self._full
        main = torch.cuda.current_stream(owned.device)
        # own chunk in place, then an in-place all-gather (NCCL leaves the own chunk alone) on the side stream
        mine = full[s.rank * chunk:(s.rank + 1) * chunk]
        mine[:owned.shape[0]].copy_(owned)
        self.side.wait_stream(main)
        with torch.cuda.stream(self.side):
            self.ctx.allgather(mine.view(-1), full.view(-1))
        dense = full[:s.cols]
        out = call(self.opts_first, self.local, dense, out)      # columns this rank owns: no remote data needed
        main.wait_stream(self.side)
        return call(self.opts_rest, self.remote, dense, out)      # the rest, added to the same output

    def spmv(self, x_owned: torch.Tensor, y_local: Optional[torch.Tensor] = None):
        return self._run(x_owned, y_local, lambda o, p, d, out: self.ctx.spmv(o, p.row_ptr, p.col_idx, p.values, d,
                                                                             out, rows=p.rows))

    def spmm(self, B_owned: torch.Tensor, C_local: Optional[torch.Tensor] = None):
        return self._run(B_owned, C_local, lambda o, p, d, out: self.ctx.spmm(o, p.row_ptr, p.col_idx, p.values, d,
                                                                             out, rows=p.rows))


def window_bytes(n_rows: int, world: int, tail=(), element_size: int = 4) -> int:
    """Bytes per rank of the window that gathers an operand of n_rows rows (`Context.window_create`)."""
    return dense_chunk(n_rows, world) * int(np.prod(tail, dtype=np.int64)) * element_size


class ShardedOperator:
    """A row shard bound to a library context: gathers the dense operand, then
    runs the local kernel on this rank's rows.  With the context's own communicator (`Context.comm_init`)
    both happen inside one C-ABI call, whose gather is the library's peer-store kernel when the context has
    a window (`Context.window_create`) and ncclAllGather otherwise; without one the gather goes through
    torch.distributed (the CPU tests of this host logic run that way on gloo)."""

    def __init__(self, ctx: api.Context, shard: CsrShard, options, group=None):
        self.ctx, self.shard, self.options, self.group = ctx, shard, options, group
        self._full = None

    def _native(self) -> bool:
        """The context owns a communicator over the shard's ranks: the whole step (gather, then kernel) is
        one C-ABI call (swb_spmv_sharded / swb_spmm_sharded)."""
        return getattr(self.ctx, "comm_world", 0) == self.shard.world and self.shard.world > 1

    def _gather(self, owned: torch.Tensor, n_rows: int) -> torch.Tensor:
        world = self.shard.world
        if getattr(self.ctx, "window", None) is not None:
            return allgather_dense(owned, n_rows, None, self.group, self.ctx)
        chunk = dense_chunk(n_rows, world)
        shape = (chunk * world,) + tuple(owned.shape[1:])
        if self._full is None or tuple(self._full.shape) != shape or self._full.dtype != owned.dtype:
            self._full = torch.empty(shape, dtype=owned.dtype, device=owned.device)
        return allgather_dense(owned, n_rows, self._full, self.group, self.ctx)

    def spmv(self, x_owned: torch.Tensor, y_local: Optional[torch.Tensor] = None, *, replicated_x=None):
        """y[row_begin:row_end] = A_shard @ x.  `x_owned` is this rank's chunk of x;
        pass `replicated_x` instead when every rank already holds all of x."""
        s = self.shard
        if replicated_x is None and self._native():
            return self.ctx.spmv_sharded(self.options, s.row_ptr, s.col_idx, s.values, x_owned, s.cols, y_local,
                                         rows=s.rows)
        x = replicated_x if replicated_x is not None else self._gather(x_owned, s.cols)
        return self.ctx.spmv(self.options, s.row_ptr, s.col_idx, s.values, x, y_local, rows=s.rows)

    def spmm(self, B_owned: torch.Tensor, C_local: Optional[torch.Tensor] = None, *, replicated_B=None):
        s = self.shard
        if replicated_B is None and self._native():
            return self.ctx.spmm_sharded(self.options, s.row_ptr, s.col_idx, s.values, B_owned, s.cols, C_local,
                                         rows=s.rows)
        B = replicated_B if replicated_B is not None else self._gather(B_owned, s.cols)
        return self.ctx.spmm(self.options, s.row_ptr, s.col_idx, s.values, B, C_local, rows=s.rows)


class ShardedBsrOperator:
    """A block-row shard of a BSR matrix bound to a library context: gathers the dense operand, then runs
    the BSR SpMM on this rank's block rows (f32 or bf16 by the dtype of the block values)."""

    def __init__(self, ctx: api.Context, shard: BsrShard, options="", group=None):
        self.ctx, self.shard, self.options, self.group = ctx, shard, options, group
        self._full = None

    def spmm(self, B_owned: torch.Tensor, C_local: Optional[torch.Tensor] = None, *, replicated_B=None):
        s = self.shard
        if replicated_B is not None:
            B = replicated_B
        else:
            chunk = dense_chunk(s.cols, s.world)
            shape = (chunk * s.world,) + tuple(B_owned.shape[1:])
            if self._full is None or tuple(self._full.shape) != shape or self._full.dtype != B_owned.dtype:
                self._full = torch.empty(shape, dtype=B_owned.dtype, device=B_owned.device)
            B = allgather_dense(B_owned, s.cols, self._full, self.group, self.ctx)
        return self.ctx.bsr_spmm(self.options, s.block_row_ptr, s.block_col_idx, s.block_values, B, s.block_size,
                                 C_local)
