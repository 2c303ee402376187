"""Host logic of the multi-GPU path on CPU: two gloo ranks cut nnz-balanced row
shards, all-gather the dense operand and together reproduce the one-rank result.
(The local arithmetic here is the oracle: this test covers sharding and the
exchange step, not the kernels.)"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from sparsewave_b200 import sharding
from tests.helpers import random_csr


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, cols = 1203, 701  # cols not divisible by the world size
        rp, ci, v = random_csr(rows, cols, 9, seed=21, empty_fraction=0.3)
        x = np.random.default_rng(21).uniform(-1, 1, cols).astype(np.float32)
        B = np.random.default_rng(22).uniform(-1, 1, (cols, 3)).astype(np.float32)
        shard = sharding.shard_csr(torch.from_numpy(rp), torch.from_numpy(ci), torch.from_numpy(v), cols, rank, world)
        lo, hi = sharding.owned_dense_range(cols, world, rank)
        x_full = sharding.allgather_dense(torch.from_numpy(x[lo:hi].copy()), cols)
        B_full = sharding.allgather_dense(torch.from_numpy(B[lo:hi].copy()), cols)
        assert np.array_equal(x_full.numpy(), x) and np.array_equal(B_full.numpy(), B)
        y = oracle.csr_spmv(shard.row_ptr.numpy(), shard.col_idx.numpy(), shard.values.numpy(), x_full.numpy())
        C = oracle.csr_spmm(shard.row_ptr.numpy(), shard.col_idx.numpy(), shard.values.numpy(), B_full.numpy())
        assert np.array_equal(y, oracle.csr_spmv(rp, ci, v, x)[shard.row_begin:shard.row_end])
        assert np.array_equal(C, oracle.csr_spmm(rp, ci, v, B)[shard.row_begin:shard.row_end])
        results[rank] = (shard.row_begin, shard.row_end, shard.nnz)
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_spmv_spmm():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_rank_main, args=(world, port, results), nprocs=world, join=True)
        r = dict(results)
    assert r[0][0] == 0 and r[0][1] == r[1][0] and r[1][1] == 1203
    total = r[0][2] + r[1][2]
    assert abs(r[0][2] - total / 2) <= 64  # nnz-balanced up to one row


def _bsr_rank_main(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sparsewave_b200 import workloads as W
        a = W.random_bsr(37, 29, 4, 0.2, seed=8, dtype=torch.float32)
        B = W.dense_uniform((a.cols, 6), seed=8)
        shard = sharding.shard_bsr(a.block_row_ptr, a.block_col_idx, a.block_values, a.cols, 4, rank, world)
        lo, hi = sharding.owned_dense_range(a.cols, world, rank)
        B_full = sharding.allgather_dense(B[lo:hi].contiguous(), a.cols)
        assert torch.equal(B_full, B)
        full = oracle.bsr_spmm_f32(a.block_row_ptr.numpy(), a.block_col_idx.numpy(), a.block_values.numpy(),
                                   B.numpy(), 4)
        mine = oracle.bsr_spmm_f32(shard.block_row_ptr.numpy(), shard.block_col_idx.numpy(),
                                   shard.block_values.numpy(), B_full.numpy(), 4)
        assert np.array_equal(mine, full[shard.row_begin:shard.row_end])
        results[rank] = (shard.block_row_begin, shard.block_row_end, shard.nnzb, shard.rows)
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_bsr():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_bsr_rank_main, args=(world, port, results), nprocs=world, join=True)
        r = dict(results)
    assert r[0][0] == 0 and r[0][1] == r[1][0] and r[1][1] == 37
    assert r[0][3] + r[1][3] == 37 * 4
    assert abs(r[0][2] - r[1][2]) <= 2 * 29  # balanced by blocks up to one block row


def test_boundaries_are_deterministic_and_cover_rows():
    rp, _, _ = random_csr(5000, 100, 12, seed=5)
    for world in (1, 2, 4, 8):
        b = sharding.shard_boundaries(torch.from_numpy(rp), world)
        assert b[0] == 0 and b[-1] == 5000 and np.all(np.diff(b) >= 0)
        assert np.array_equal(b, sharding.shard_boundaries(rp, world))
        nnz = np.diff(rp[b])
        assert nnz.max() - nnz.min() <= 2 * np.diff(rp).max()
    # one indivisible long row
    rp = np.array([0, 1, 1000, 1001, 1002], np.int32)
    b = sharding.shard_boundaries(rp, 4)
    assert b[0] == 0 and b[-1] == 4 and np.all(np.diff(b) >= 0)


def test_dense_chunks():
    assert sharding.dense_chunk(701, 2) == 351
    assert sharding.owned_dense_range(701, 2, 1) == (351, 701)
    assert sharding.owned_dense_range(5, 8, 7) == (5, 5)


def test_split_by_column_ownership():
    rp, ci, v = random_csr(500, 300, 8, seed=3, empty_fraction=0.3)
    x = np.random.default_rng(0).uniform(-1, 1, 300).astype(np.float32)
    shard = sharding.shard_csr(torch.from_numpy(rp), torch.from_numpy(ci), torch.from_numpy(v), 300, 1, 2)
    lo, hi = sharding.owned_dense_range(300, 2, 1)
    own, rest = sharding.split_by_column_range(shard, lo, hi)
    assert own.nnz + rest.nnz == shard.nnz and own.rows == rest.rows == shard.rows
    assert bool(((own.col_idx >= lo) & (own.col_idx < hi)).all()) and bool(((rest.col_idx < lo) | (rest.col_idx >= hi)).all())
    parts = [oracle.csr_spmv(p.row_ptr.numpy(), p.col_idx.numpy(), p.values.numpy(), x) for p in (shard, own, rest)]
    assert np.allclose(parts[0], parts[1] + parts[2], atol=1e-5)
    for p in (own, rest):  # order inside a row is preserved: columns stay sorted
        r = p.row_ptr.numpy()
        c = p.col_idx.numpy()
        assert all(np.all(np.diff(c[r[i]:r[i + 1]]) > 0) for i in range(p.rows))


def test_split_by_column_range_keeps_every_entry_once():
    """The column-ownership split of a shard (the overlapped operator's two passes): both parts keep all rows
    and the order of the entries inside a row, and together they are the shard."""
    rows, cols = 300, 120
    rp, ci, v = random_csr(rows, cols, 8, seed=31, empty_fraction=0.25)
    shard = sharding.shard_csr(torch.from_numpy(rp), torch.from_numpy(ci), torch.from_numpy(v), cols, 0, 1)
    inside, outside = sharding.split_by_column_range(shard, 40, 80)
    assert inside.rows == outside.rows == rows and inside.nnz + outside.nnz == len(v)
    assert bool(((inside.col_idx >= 40) & (inside.col_idx < 80)).all())
    assert bool(((outside.col_idx < 40) | (outside.col_idx >= 80)).all())
    x = np.random.default_rng(31).uniform(-1, 1, cols).astype(np.float32)
    parts = [oracle.csr_spmv(p.row_ptr.numpy(), p.col_idx.numpy(), p.values.numpy(), x) for p in (inside, outside)]
    whole = oracle.csr_spmv(rp, ci, v, x)
    assert np.allclose(parts[0] + parts[1], whole, rtol=1e-5, atol=1e-5)
    for r in range(rows):  # order inside a row is the original order
        row_cols = ci[rp[r]:rp[r + 1]]
        a = inside.col_idx[inside.row_ptr[r]:inside.row_ptr[r + 1]].numpy()
        b = outside.col_idx[outside.row_ptr[r]:outside.row_ptr[r + 1]].numpy()
        assert np.array_equal(a, row_cols[(row_cols >= 40) & (row_cols < 80)])
        assert np.array_equal(b, row_cols[(row_cols < 40) | (row_cols >= 80)])


def test_window_bytes():
    assert sharding.window_bytes(4194304, 8) == 524288 * 4
    assert sharding.window_bytes(701, 2, (3,)) == 351 * 3 * 4
    assert sharding.window_bytes(16384, 4, (512,), 2) == 4096 * 512 * 2
