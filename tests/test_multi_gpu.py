"""Row-sharded SpMV / SpMM over two GPUs with the NCCL all-gather (skipped with fewer than two GPUs)."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port):
    import torch.distributed as dist

    import oracle
    from sparsewave_b200 import Context, sharding, workloads as W

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = Context(rank)
        a, x = W.config_c3(device="cuda", rows=1 << 16, max_len=4096)
        B = W.dense_uniform((a.cols, 8), seed=9, device="cuda")
        shard = sharding.shard_csr(a.row_ptr, a.col_idx, a.values, a.cols, rank, world)
        lo, hi = sharding.owned_dense_range(a.cols, world, rank)
        rp, ci, v = a.numpy()
        xh, Bh = x.cpu().numpy(), B.cpu().numpy()
        rows = slice(shard.row_begin, shard.row_end)
        op = sharding.ShardedOperator(ctx, shard, "spmv-mapping=wave-per-position")
        y = op.spmv(x[lo:hi].contiguous()).cpu().numpy()   # all-gather through torch.distributed
        ctx.comm_init(rank, world)                          # from here on: the library's own communicator
        y2 = op.spmv(x[lo:hi].contiguous()).cpu().numpy()
        assert np.all(np.abs(y2 - y) <= 1e-5 * oracle.csr_abs_bound(rp, ci, v, xh)[rows] + 1e-30)
        bound = oracle.csr_abs_bound(rp, ci, v, xh)[rows]
        assert np.all(np.abs(y - oracle.csr_spmv(rp, ci, v, xh)[rows]) <= 1e-5 * bound + 1e-30)
        # the library's own all-gather: one kernel of peer stores into an IPC window, several steps in a row
        # with a different x each (a step must not overwrite a buffer that a peer still reads); the operator's
        # steps fill the window's two buffers in turn
        ctx.window_create(sharding.window_bytes(a.cols, world))
        for step in range(5):
            xs = x * float(step + 1)
            y4 = op.spmv(xs[lo:hi].contiguous()).cpu().numpy()
            want = oracle.csr_spmv(rp, ci, v, xh * np.float32(step + 1))[rows]
            assert np.all(np.abs(y4 - want) <= 1e-5 * (step + 1) * bound + 1e-30)
            assert torch.equal(ctx.window_buffers[step & 1].view(torch.float32)[:a.cols], xs)
        # a captured graph of three steps replayed: its first step fills the buffer that its last one filled
        # (the kernel sees that on the device and waits for the peers' readers), then plain steps again, and a
        # direct all-gather (always the first buffer) in between
        xg = x[lo:hi].clone()
        yg = torch.empty(shard.rows, device="cuda")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(3):
                    op.spmv(xg, yg)
        torch.cuda.current_stream().wait_stream(side)
        for replay in range(3):
            xg.copy_(x[lo:hi] * float(replay + 2))
            graph.replay()
            want = oracle.csr_spmv(rp, ci, v, xh * np.float32(replay + 2))[rows]
            assert np.all(np.abs(yg.cpu().numpy() - want) <= 1e-5 * (replay + 2) * bound + 1e-30)
        got = ctx.window_allgather(x[lo:hi].contiguous() if (hi - lo) * 4 == ctx.window_bytes_per_rank else
                                   torch.nn.functional.pad(x[lo:hi], (0, ctx.window_bytes_per_rank // 4 - (hi - lo))))
        assert torch.equal(got.view(torch.float32)[:a.cols], x)
        seen = set()
        for k in range(3):  # the alternating form, called directly: the returned buffer holds this call's gather
            got = ctx.window_allgather_next((x[lo:hi] * float(k + 7)).contiguous())
            assert torch.equal(got.view(torch.float32)[:a.cols], x * float(k + 7))
            seen.add(got.data_ptr())
        assert len(seen) == 2
        y5 = op.spmv(x[lo:hi].contiguous()).cpu().numpy()
        assert np.all(np.abs(y5 - y) <= 1e-5 * bound + 1e-30)
        assert ctx.device_status() == 0
        ctx.window_destroy()
        ctx.window_create(sharding.window_bytes(a.cols, world, (8,)))
        opw = sharding.ShardedOperator(ctx, shard, "spmm-mapping=wave-per-row-tile spmm-tile-size=8 spmm-block-size=128")
        Cw = opw.spmm(B[lo:hi].contiguous()).cpu().numpy()
        assert np.all(np.abs(Cw - oracle.csr_spmm(rp, ci, v, Bh)[rows]) <= 1e-5 * oracle.csr_abs_bound(rp, ci, v, Bh)[rows] + 1e-30)
        assert ctx.device_status() == 0
        ctx.window_destroy()
        op = sharding.ShardedOperator(ctx, shard, "spmm-mapping=wave-per-row-tile spmm-tile-size=8 spmm-block-size=128")
        C = op.spmm(B[lo:hi].contiguous()).cpu().numpy()
        bound = oracle.csr_abs_bound(rp, ci, v, Bh)[rows]
        assert np.all(np.abs(C - oracle.csr_spmm(rp, ci, v, Bh)[rows]) <= 1e-5 * bound + 1e-30)
        # all-gather overlapped with the locally-owned columns, second part accumulated into the same output
        ov = sharding.OverlappedShardedOperator(ctx, shard, "spmv-mapping=wave-per-position")
        for _ in range(2):
            y3 = ov.spmv(x[lo:hi].contiguous()).cpu().numpy()
            assert np.all(np.abs(y3 - y) <= 2e-5 * oracle.csr_abs_bound(rp, ci, v, xh)[rows] + 1e-30)
        ov = sharding.OverlappedShardedOperator(ctx, shard, "spmm-mapping=wave-per-row-tile spmm-tile-size=8 spmm-block-size=128")
        C3 = ov.spmm(B[lo:hi].contiguous()).cpu().numpy()
        assert np.all(np.abs(C3 - C) <= 2e-5 * bound + 1e-30)
        # BSR: block rows sharded by block count, bf16 B all-gathered, tensor-core kernel on the shard
        bsr, Bb = W.config_c5(device="cuda", block_grid=64, n_rhs=128)
        bshard = sharding.shard_bsr(bsr.block_row_ptr, bsr.block_col_idx, bsr.block_values, bsr.cols, 16, rank, world)
        blo, bhi = sharding.owned_dense_range(bsr.cols, world, rank)
        Cb = sharding.ShardedBsrOperator(ctx, bshard).spmm(Bb[blo:bhi].contiguous())
        whole = ctx.bsr_spmm("", bsr.block_row_ptr, bsr.block_col_idx, bsr.block_values, Bb, 16)
        assert torch.equal(Cb, whole[bshard.row_begin:bshard.row_end])
        # the sharded step through host buffers: this rank's rows of the matrix uploaded once from the full host
        # matrix, then only this rank's chunk of x (or B) goes in and only its rows come out
        bnd = sharding.shard_boundaries(a.row_ptr, world)
        resident = ctx.csr_upload_rows(a.cols, rp, ci, v, int(bnd[rank]), int(bnd[rank + 1]))
        yh = np.empty(shard.rows, dtype=np.float32)
        for scale in (1.0, 3.0):
            resident.spmv_sharded_host("spmv-mapping=wave-per-position", np.ascontiguousarray(xh[lo:hi] * np.float32(scale)), yh)
            want = oracle.csr_spmv(rp, ci, v, xh * np.float32(scale))[rows]
            assert np.all(np.abs(yh - want) <= 1e-5 * scale * oracle.csr_abs_bound(rp, ci, v, xh)[rows] + 1e-30)
        Ch = np.empty((shard.rows, 8), dtype=np.float32)
        resident.spmm_sharded_host("spmm-mapping=wave-per-row-tile spmm-tile-size=8 spmm-block-size=128",
                                   np.ascontiguousarray(Bh[lo:hi]), Ch)
        assert np.all(np.abs(Ch - oracle.csr_spmm(rp, ci, v, Bh)[rows]) <= 1e-5 * bound + 1e-30)
        with pytest.raises(Exception):  # the host calls' result buffer is write-only
            resident.spmv_sharded_host("spmv-mapping=wave-per-position accumulate=1", np.ascontiguousarray(xh[lo:hi]), yh)
        resident.release()
        assert ctx.device_status() == 0
        # shard boundaries are the same on every rank
        b = torch.tensor(sharding.shard_boundaries(a.row_ptr, world), device="cuda")
        ref = b.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(b, ref)
        dist.barrier()
        ctx.window_destroy()  # collective tear-down, on the success path only
        ctx.close()
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharded_operators():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_rank_main, args=(2, _free_port()), nprocs=2, join=True)
