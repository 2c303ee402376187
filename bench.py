"""Benchmark of the SpMV / SpMM / BSR-SpMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5]
                    [--impl ours|reference] [--options "..."] [--rows R]

One step = one operator call over the whole synthetic workload (for N > 1: the
all-gather of the dense operand plus the local kernel on this rank's row
shard).  Rank 0 prints one JSON line.  `value` is algorithmic GB/s with the
operands resident in HBM; `e2e` is the same metric through the host-buffer
C-ABI call (H2D of the operands and D2H of the result inside the timed
region); `roofline` compares the kernel with the measured HBM copy bandwidth
and, for SpMV, with a live run of the library's stream-and-gather probe;
`parity` is the comparison of the timed step's own output with the CPU oracle
(every rank checks its rows; a mismatch makes the process exit non-zero, like
the reference runner, which accepts a timing only from a run whose output
matched: benchmark/benchmark_utils.py:707-716 in the SparseWave tree);
`cpu_baseline` times the CPU restatement of the reference loop on the host
cores.  The default command (one GPU, no --workload) also runs the other four
configurations for a few steps each, attaches them as `configs` and appends
every finished configuration to bench_results/results.jsonl.
`--impl reference` times only the CPU loop.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "SpMV/SpMM effective HBM GB/s"
L2_BYTES = 126 * 1024 * 1024

# Default options per workload: the mapping each configuration names.
WORKLOADS = {
    "c1": dict(kind="spmv", options="spmv-mapping=wave-per-row spmv-block-size=128",
               name="c1: CSR SpMV 4096x4096, 16 nnz/row, f32/i32"),
    "c2": dict(kind="spmm", options="spmm-mapping=wave-per-row-tile spmm-tile-size=4 spmm-block-size=64",
               name="c2: CSR SpMM 65536x65536, 32 nnz/row, N=4, f32/i32"),
    "c3": dict(kind="spmv", options="spmv-mapping=wave-per-position spmv-block-size=128",
               name="c3: power-law CSR SpMV 4194304x4194304, Zipf(1.8) rows in [1,65536], f32/i32"),
    "c4": dict(kind="spmm", options="spmm-mapping=wave-per-row-tile spmm-tile-size=16 spmm-block-size=256",
               name="c4: CSR SpMM 2097152x2097152, 32 banded + 32 random nnz/row, N=64, f32/i32"),
    "c5": dict(kind="bsr", options="",
               name="c5: BSR SpMM 16384x16384, 16x16 bf16 blocks at 5% density, N=512"),
}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel at the full workload size,
# from the one-pass ncu captures summarised under profiles/ (None where no capture exists).
NCU_TRAFFIC_BYTES = {"c2": 18.1e6, "c3": 0.7934e9, "c4": 16.69e9, "c5": 45.3e6}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=None,
                   help="timed steps (default: at least 100 and at least 60 ms of them)")
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default=None, choices=sorted(WORKLOADS), help="default c3")
    p.add_argument("--options", default=None, help="option string in the reference's spelling")
    p.add_argument("--rows", type=int, default=None, help="override the row count (testing)")
    p.add_argument("--no-graph", action="store_true", help="launch every step from the host instead of replaying "
                   "a CUDA graph of the steps")
    p.add_argument("--graph-steps", type=int, default=10, help="steps captured in one CUDA graph (inputs larger "
                   "than L2 only; the timed region stays exactly --steps steps)")
    p.add_argument("--no-align", action="store_true", help="N > 1 with the L2 flush: do not line the ranks up "
                   "(a 16-byte all-gather outside the event pairs) between a flush and the timed step")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-cpu", action="store_true")
    p.add_argument("--no-parity", action="store_true", help="skip the comparison of the timed output with the oracle")
    p.add_argument("--no-configs", action="store_true",
                   help="default command only: do not run the other four configurations after the headline one")
    p.add_argument("--no-library", action="store_true",
                   help="one GPU: skip the cuSPARSE (torch.sparse) column, the analogue of the reference's rocSPARSE "
                        "column; comparison only")
    p.add_argument("--results-dir", default=str(ROOT / "bench_results"),
                   help="results.jsonl (one line per finished configuration, appended) and metadata.json go here")
    p.add_argument("--overlap", action="store_true",
                   help="N > 1: run the locally-owned columns of the shard while the all-gather is in flight")
    p.add_argument("--torch-collective", action="store_true",
                   help="N > 1: all-gather through torch.distributed instead of the library's communicator")
    p.add_argument("--nccl-allgather", action="store_true",
                   help="N > 1: all-gather with ncclAllGather on the library's communicator instead of the "
                        "library's own peer-store kernel (CUDA IPC windows over NVLink)")
    p.add_argument("--replicated", action="store_true",
                   help="N > 1: dense operand already replicated, no all-gather in the step")
    return p.parse_args()


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._thread = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                f = [t.strip() for t in out.stdout.strip().split(",")]
                if len(f) >= 6:
                    self.samples.append(f)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        mhz = sorted(float(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": float(self.samples[0][1]), "reasons": reasons,
                "samples": len(self.samples),
                "window": "warm-up, timed steps and about 0.3 s more of the same steps"}


def build_workload(name: str, device, rows):
    """Returns the operands (torch tensors on `device`) and the algorithmic bytes / flops of one call."""
    from sparsewave_b200 import workloads as W
    kw = {} if rows is None else ({"block_grid": rows // 16} if name == "c5" else {"rows": rows})
    a, dense = getattr(W, f"config_{name}")(device=device, **kw)
    kind = WORKLOADS[name]["kind"]
    if kind == "spmv":
        nbytes, flops = W.spmv_bytes(a.rows, a.cols, a.nnz), 2 * a.nnz
    elif kind == "spmm":
        n = dense.shape[1]
        nbytes, flops = W.spmm_bytes(a.rows, a.cols, a.nnz, n), 2 * a.nnz * n
    else:
        n = dense.shape[1]
        nbytes = W.bsr_bytes(a.rows, a.cols, a.nnzb, 16, n)
        flops = 2 * a.nnzb * 256 * n
    return dict(kind=kind, a=a, dense=dense, bytes=nbytes, flops=flops)


def describe(wl):
    a = wl["a"]
    d = {"rows": a.rows, "cols": a.cols}
    if wl["kind"] == "bsr":
        d.update(nnzb=a.nnzb, block_size=16, n_rhs=int(wl["dense"].shape[1]))
    else:
        d.update(nnz=a.nnz)
        if wl["kind"] == "spmm":
            d.update(n_rhs=int(wl["dense"].shape[1]))
    return d


def cpu_pass(wl, host):
    """One pass of the CPU restatement of the reference loop over the whole workload (all host threads)."""
    import oracle
    if wl["kind"] == "spmv":
        return oracle.csr_spmv(host["row_ptr"], host["col_idx"], host["values"], host["dense"], parallel=True)
    if wl["kind"] == "spmm":
        return oracle.csr_spmm(host["row_ptr"], host["col_idx"], host["values"], host["dense"], parallel=True)
    return oracle.bsr_spmm_bf16(host["row_ptr"], host["col_idx"], host["values"], host["dense"], 16)[0]


def host_copies(wl):
    import torch
    a, dense = wl["a"], wl["dense"]
    if wl["kind"] == "bsr":
        return dict(row_ptr=a.block_row_ptr.cpu().numpy(), col_idx=a.block_col_idx.cpu().numpy(),
                    values=a.block_values.view(torch.uint16).cpu().numpy(),
                    dense=dense.view(torch.uint16).cpu().numpy())
    return dict(row_ptr=a.row_ptr.cpu().numpy(), col_idx=a.col_idx.cpu().numpy(), values=a.values.cpu().numpy(),
                dense=dense.cpu().numpy())


def time_cpu(wl, host, seconds=20.0, max_passes=50):
    """Passes over the whole workload until about `seconds` seconds are spent; returns (best seconds, passes)."""
    cpu_pass(wl, host)  # warm-up (page faults, thread pool)
    best, passes, t_end = float("inf"), 0, time.perf_counter() + seconds
    while passes < 3 or (time.perf_counter() < t_end and passes < max_passes):
        t0 = time.perf_counter()
        cpu_pass(wl, host)
        best = min(best, time.perf_counter() - t0)
        passes += 1
    return best, passes


# ---------------------------------------------------------------------------------------------------
# parity of a timed step's output: rows [row_begin, row_begin + rows) of the operator, checked in row
# blocks against the oracle on host copies of the same operands
# ---------------------------------------------------------------------------------------------------

def check_parity(kind, row_ptr, col_idx, values, dense, out, block_elems=1 << 24):
    """`row_ptr` (rebased to 0), `col_idx`, `values`: host arrays of the rows this process computed; `dense`:
    the whole dense operand on the host; `out`: this process's result (torch tensor, device or host).  Returns
    the parity record of those rows."""
    import torch

    import oracle
    rec = {"checked_rows": 0, "checked_outputs": 0}
    if kind == "bsr":
        got = out.detach().contiguous().view(torch.uint16).cpu().numpy()
        bits, f32 = oracle.bsr_spmm_bf16(row_ptr, col_idx, values, dense, 16)
        bound = oracle.bsr_abs_bound_bf16(row_ptr, col_idx, values, dense, 16)
        beyond_ulp, cancelling = oracle.bf16_mismatches(got, bits, f32, bound)
        got32 = (got.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        rel = np.abs(got32 - f32) / np.maximum(np.abs(f32.astype(np.float64)), 2.0 ** -6 * bound + 1e-30)
        rec.update(checked_rows=int(got.shape[0]), checked_outputs=int(got.size),
                   mismatches_north_star=int(np.sum(rel > 1e-2)), mismatches_beyond_one_bf16_ulp=beyond_ulp,
                   mismatches_cancelling_sums=cancelling, max_rel_err=float(rel.max()) if rel.size else 0.0,
                   criterion="BF16: |C - C_ref| <= 1e-2 * max(|C_ref|, 2^-6 * sum|a*b|); also counted: outputs more "
                             "than one bf16 ulp from the oracle's rounded bits")
        rec["ok"] = rec["mismatches_north_star"] == 0 and beyond_ulp == 0 and cancelling == 0
        return rec
    rows = len(row_ptr) - 1
    width = 1 if kind == "spmv" else int(dense.shape[1])
    got_all = out.detach().cpu().numpy().reshape(rows, width)
    step = max(1, block_elems // width)
    bad_ns, bad_ref, worst, checksum_got, checksum_exp = 0, 0, 0.0, 0.0, 0.0
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        p0, p1 = int(row_ptr[r0]), int(row_ptr[r1])
        rp = (row_ptr[r0:r1 + 1] - p0).astype(np.int32)
        ci, v = col_idx[p0:p1], values[p0:p1]
        if kind == "spmv":
            exp = oracle.csr_spmv(rp, ci, v, dense, parallel=True)
        else:
            exp = oracle.csr_spmm(rp, ci, v, dense, parallel=True)
        bound = oracle.csr_abs_bound(rp, ci, v, dense).reshape(r1 - r0, width)
        exp = exp.reshape(r1 - r0, width)
        got = got_all[r0:r1]
        err = np.abs(got.astype(np.float64) - exp)
        bad_ns += int(np.sum(err > 1e-5 * bound + 1e-30))
        bad_ref += oracle.count_mismatches_reference(got, exp)
        if err.size:
            worst = max(worst, float(np.max(err / (1e-5 * bound + 1e-30))))
        checksum_got += float(got.astype(np.float64).sum())
        checksum_exp += float(exp.astype(np.float64).sum())
    rec.update(checked_rows=rows, checked_outputs=rows * width, mismatches_north_star=bad_ns,
               **{"mismatches_reference_1e-4": bad_ref}, max_err_over_bound=worst,
               checksum_f64=checksum_got, checksum_f64_oracle=checksum_exp,
               criterion="|y - y_ref| <= 1e-5 * sum|a_ij * x_j| per output decides; also counted: outputs outside "
                         "the reference runner's own 1e-4 * max(1, |expected|) (rows of tens of thousands of terms "
                         "exceed it under any f32 summation order, the CPU loop's own included)")
    rec["ok"] = bad_ns == 0
    return rec


def merge_parity(rec, env):
    """Sum of the counts and maximum of the errors over the ranks (every rank checked its own rows)."""
    if env["world"] == 1:
        return rec
    import torch
    import torch.distributed as dist
    sums = ["checked_rows", "checked_outputs", "mismatches_north_star", "mismatches_reference_1e-4",
            "mismatches_beyond_one_bf16_ulp", "mismatches_cancelling_sums", "checksum_f64", "checksum_f64_oracle"]
    maxes = ["max_err_over_bound", "max_rel_err"]
    for keys, op in ((sums, dist.ReduceOp.SUM), (maxes, dist.ReduceOp.MAX)):
        present = [k for k in keys if k in rec]
        if not present:
            continue
        t = torch.tensor([float(rec[k]) for k in present], dtype=torch.float64, device=env["device"])
        dist.all_reduce(t, op=op)
        for k, v in zip(present, t.tolist()):
            rec[k] = int(v) if k.startswith(("checked", "mismatches")) else v
    ok = torch.tensor([int(rec["ok"])], dtype=torch.int32, device=env["device"])
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    rec["ok"] = bool(int(ok.item()))
    rec["ranks_checked"] = env["world"]
    return rec


# ---------------------------------------------------------------------------------------------------

def init_env(args):
    import torch
    import torch.distributed as dist

    from sparsewave_b200 import Context
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    ctx = Context(local)
    if world > 1 and not args.torch_collective:
        ctx.comm_init(rank, world)  # the library's own NCCL communicator (capturable in the step's CUDA graph)
    env = dict(rank=rank, world=world, local=local, device=device, ctx=ctx)

    def barrier():
        # Drain this rank's queue first: the library's communicator and torch.distributed's are two NCCL
        # communicators on the same GPUs, and collectives of both in flight at once can wait on each other.
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def per_rank(value):
        if world == 1:
            return [value]
        t = torch.zeros(world, dtype=torch.float64, device=device)
        t[rank] = value
        dist.all_reduce(t)
        return t.tolist()

    env.update(barrier=barrier, max_over_ranks=max_over_ranks, per_rank=per_rank)
    return env


def setup_window(args, env, nbytes):
    """The library's own exchange kernel for the all-gather of N > 1.  Creation succeeds on every rank or on
    none; before it is used, two exchanges of a rank-coded pattern are checked on every rank, and one bad rank
    sends all of them back to ncclAllGather.  Returns the description of the exchange in use."""
    import torch
    import torch.distributed as dist
    ctx, rank, world, device = env["ctx"], env["rank"], env["world"], env["device"]
    if getattr(ctx, "window", None) is not None:
        ctx.window_destroy()
    if args.nccl_allgather or args.torch_collective or args.replicated or args.overlap or nbytes % 16 != 0:
        return "torch.distributed" if args.torch_collective else "library NCCL communicator"
    try:
        ctx.window_create(nbytes)
        probe = torch.full((nbytes // 4,), float(rank + 1), dtype=torch.float32, device=device)
        for _ in range(2):
            ctx.window_allgather(probe)
        torch.cuda.synchronize()
        got = ctx.window.view(torch.float32).view(world, -1)
        good = all(bool((got[k] == float(k + 1)).all()) for k in range(world)) and ctx.device_status() == 0
        agreed = torch.tensor([int(good)], dtype=torch.int32, device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        torch.cuda.synchronize()
        if int(agreed.item()) == 1:
            return "peer-store kernel over NVLink into CUDA IPC windows"
        print("bench: the peer-window self-check failed, using ncclAllGather", file=sys.stderr)
        ctx.window_destroy()
    except Exception as exc:  # noqa: BLE001  (no CUDA IPC between these processes: same on every rank)
        print(f"bench: peer window unavailable, using ncclAllGather: {exc}", file=sys.stderr)
    return "library NCCL communicator"


def measure_workload(args, env, name, *, headline, steps_arg, warmup, clocks=None):
    """Runs one configuration: timed steps, parity of their output, and (as far as they apply) the gather
    bound, the library column, the end-to-end leg and the CPU baseline.  Returns the record of the run."""
    import torch
    import torch.distributed as dist

    from sparsewave_b200 import make_options, sharding
    ctx, rank, world, device = env["ctx"], env["rank"], env["world"], env["device"]
    barrier, max_over_ranks = env["barrier"], env["max_over_ranks"]
    spec = WORKLOADS[name]
    options = args.options if (args.options is not None and headline) else spec["options"]
    opts = make_options(options)  # parsed once; the steps pass the option block
    wl = build_workload(name, device, args.rows if headline else None)
    kind, a, dense = wl["kind"], wl["a"], wl["dense"]
    gather_kind = None
    shard = None

    # ---- this rank's share --------------------------------------------------------------
    if world > 1 and kind == "bsr":
        # block rows sharded by block count, bf16 B all-gathered (launch-sized at this configuration)
        shard = sharding.shard_bsr(a.block_row_ptr, a.block_col_idx, a.block_values, a.cols, 16, rank, world)
        op = sharding.ShardedBsrOperator(ctx, shard, opts)
        lo, hi = sharding.owned_dense_range(a.cols, world, rank)
        owned = dense[lo:hi].contiguous()
        out = torch.empty((shard.rows, dense.shape[1]), dtype=torch.bfloat16, device=device)
        full = dense if args.replicated else None
        step = lambda: op.spmm(owned, out, replicated_B=full)
        local_step = lambda: ctx.bsr_spmm(opts, shard.block_row_ptr, shard.block_col_idx, shard.block_values, dense, 16, out)
        local_input_bytes = 512 * shard.nnzb + dense.numel() * 2
        gather_kind = "library NCCL communicator"
    elif world > 1:
        shard = sharding.shard_csr(a.row_ptr, a.col_idx, a.values, a.cols, rank, world)
        overlap = args.overlap and not args.replicated and not args.torch_collective
        nbytes = sharding.window_bytes(a.cols, world, tuple(dense.shape[1:]), dense.element_size())
        gather_kind = setup_window(args, env, nbytes)
        op = sharding.OverlappedShardedOperator(ctx, shard, opts) if overlap else \
            sharding.ShardedOperator(ctx, shard, opts)
        lo, hi = sharding.owned_dense_range(a.cols, world, rank)
        owned = dense[lo:hi].contiguous()
        out = torch.empty((shard.rows,) + tuple(dense.shape[1:]), dtype=torch.float32, device=device)
        full = dense if args.replicated else None
        if overlap:
            step = (lambda: op.spmv(owned, out)) if kind == "spmv" else (lambda: op.spmm(owned, out))
        elif kind == "spmv":
            step = lambda: op.spmv(owned, out, replicated_x=full)
        else:
            step = lambda: op.spmm(owned, out, replicated_B=full)
        if kind == "spmv":
            local_step = lambda: ctx.spmv(opts, shard.row_ptr, shard.col_idx, shard.values, dense, out, rows=shard.rows)
        else:
            local_step = lambda: ctx.spmm(opts, shard.row_ptr, shard.col_idx, shard.values, dense, out, rows=shard.rows)
        local_input_bytes = 8 * shard.nnz + dense.numel() * 4
    else:
        if kind == "spmv":
            out = torch.empty(a.rows, dtype=torch.float32, device=device)
            step = lambda: ctx.spmv(opts, a.row_ptr, a.col_idx, a.values, dense, out)
        elif kind == "spmm":
            out = torch.empty((a.rows, dense.shape[1]), dtype=torch.float32, device=device)
            step = lambda: ctx.spmm(opts, a.row_ptr, a.col_idx, a.values, dense, out)
        else:
            out = torch.empty((a.rows, dense.shape[1]), dtype=torch.bfloat16, device=device)
            step = lambda: ctx.bsr_spmm(opts, a.block_row_ptr, a.block_col_idx, a.block_values, dense, 16, out)
        local_step = step
        local_input_bytes = wl["bytes"]

    # Inputs larger than L2 need no flush; smaller ones get a 256 MiB write between timed steps.
    flush = None
    if local_input_bytes <= 2 * L2_BYTES:
        flush = env.setdefault("flush", torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device))

    # The flush kernels of the ranks do not end at the same moment; a step's exchange would wait for the last of
    # them inside its event pair.  A 16-byte all-gather between the flush and the first record lines the ranks
    # up again, as consecutive steps of a real run do by themselves.
    align = None
    if flush is not None and world > 1 and getattr(ctx, "comm_world", 1) > 1 and not args.no_align:
        tick = torch.zeros(4, dtype=torch.float32, device=device)
        tock = torch.zeros(4 * world, dtype=torch.float32, device=device)
        align = lambda: ctx.allgather(tick, tock)  # noqa: E731

    def timed(fn, calls):
        """Device time of `calls` calls in ms: one event pair around all of them, or one
        pair per call with an L2 flush outside the pairs."""
        if flush is None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(calls):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1)
        pairs = []
        for _ in range(calls):
            flush.zero_()
            if align is not None:
                align()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            pairs.append((e0, e1))
        torch.cuda.synchronize()
        return sum(p[0].elapsed_time(p[1]) for p in pairs)

    def capture(fn, count):
        """`count` calls of fn as one CUDA graph.  Host launches remain for steps whose all-gather goes through
        torch.distributed (capturing that one hung here, so it is not tried); the library's own exchange is
        captured with the kernels."""
        before = ctx.kernel_launches
        g = torch.cuda.CUDAGraph()
        # relaxed: NCCL's helper threads may issue CUDA calls of their own while this thread captures
        with torch.cuda.graph(g, capture_error_mode="relaxed"):
            for _ in range(count):
                fn()
        launches = ctx.kernel_launches - before
        g.replay()
        torch.cuda.synchronize()
        return g, launches

    for _ in range(max(warmup, 3)):
        step()
    barrier()
    # A quick estimate of the step time (rank-uniform) sizes the timed region when --steps is not given: at
    # least 100 steps and at least 60 ms.
    est_ms = max_over_ranks(timed(step, 3) / 3)
    if steps_arg is not None:
        steps = steps_arg
    else:
        steps = int(min(20000, max(100, math.ceil(60.0 / max(est_ms, 1e-3)))))
        steps = (steps + 9) // 10 * 10
    # Steps captured in a CUDA graph and replayed: no host work between the kernels of a step, and with several
    # steps per graph none between steps either (the host threads of N ranks share the cores with NCCL's).
    # With the L2 flush, which stays outside the event pairs, one step per graph sits between the two records.
    per_graph = 1
    if flush is None and args.graph_steps > 1:
        per_graph = max(d for d in range(1, args.graph_steps + 1) if steps % d == 0)
    torch_collective = world > 1 and not args.replicated and args.torch_collective
    graph, launches_per_graph, run_step = None, None, step
    if not args.no_graph and not torch_collective:
        try:
            graph, launches_per_graph = capture(step, per_graph)
            run_step = graph.replay
        except Exception as exc:  # noqa: BLE001
            print(f"bench: CUDA graph capture failed, launching from the host: {exc}", file=sys.stderr)
            torch.cuda.synchronize()
            graph, per_graph = None, 1
    else:
        per_graph = 1
    barrier()
    launches0 = ctx.kernel_launches
    total_ms = timed(run_step, steps // per_graph)
    launches1 = ctx.kernel_launches
    barrier()
    total_ms = max_over_ranks(total_ms)
    ms_per_step = total_ms / steps
    gpu_launches = launches1 - launches0 if graph is None else launches_per_graph * (steps // per_graph)

    # The reference's own convention (benchmark/benchmark_utils.py:520-521): 10 warm-up dispatches, 50
    # timed ones, each with its own event pair; median / min / p95 of those (max over ranks per dispatch).
    one_graph = None
    one_step = step
    if graph is not None:
        if per_graph == 1:
            one_step = graph.replay
        else:
            one_graph, _ = capture(step, 1)
            one_step = one_graph.replay
    per_dispatch = []
    for i in range(60):
        if flush is not None:
            flush.zero_()
            if align is not None:
                align()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        one_step()
        e1.record()
        if i >= 10:
            per_dispatch.append((e0, e1))
    torch.cuda.synchronize()
    times = torch.tensor([x.elapsed_time(y) for x, y in per_dispatch], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    times = sorted(times.tolist())
    dispatch_stats = {"warmup": 10, "dispatches": 50, "median_ms": times[len(times) // 2], "min_ms": times[0],
                      "p95_ms": times[min(len(times) - 1, int(round(0.95 * (len(times) - 1))))]}
    barrier()
    if clocks is not None:
        # Keep the same steps running for about 0.3 s so that the sampler sees the clocks under this
        # load.  The count comes from the rank-reduced time, so every rank runs the same number of steps
        # (they contain a collective when N > 1).
        soak = int(min(5000, max(10, 300.0 / max(ms_per_step * per_graph, 1e-3))))
        for _ in range(soak):
            run_step()
        barrier()
        clocks.__exit__(None, None, None)

    # ---- phases of a sharded step, each as its own graph of 20 repetitions (device time, per rank) -----
    phases = None
    if world > 1 and not args.replicated and not torch_collective and kind != "bsr" and not args.overlap:
        phases = {}
        try:
            if getattr(ctx, "window", None) is not None:
                gather = lambda: ctx.window_allgather_next(owned)  # the form the sharded step uses
            else:
                chunk = sharding.dense_chunk(a.cols, world)
                send = torch.zeros((chunk,) + tuple(dense.shape[1:]), dtype=dense.dtype, device=device)
                send[:owned.shape[0]].copy_(owned)
                recv = torch.empty((chunk * world,) + tuple(dense.shape[1:]), dtype=dense.dtype, device=device)
                gather = lambda: ctx.allgather(send.view(-1), recv.view(-1))
            for label, fn in (("allgather_ms", gather), ("kernel_ms", local_step)):
                for _ in range(3):
                    fn()
                g, _ = capture(fn, 20)
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                vals = env["per_rank"](e0.elapsed_time(e1) / 20)
                phases[label] = max(vals)
                phases[label.replace("_ms", "_ms_per_rank")] = [round(v, 5) for v in vals]
                del g
                barrier()
            phases["note"] = ("each phase is a CUDA graph of 20 back-to-back repetitions, L2 warm; kernel_ms is the "
                              "local operator on this rank's shard with the dense operand in place (zero fill "
                              "included); the step's time is about allgather_ms + the largest kernel_ms")
        except Exception as exc:  # noqa: BLE001
            phases = {"unavailable": str(exc)}

    # ---- parity of the timed step's own output ------------------------------------------------------
    device_status = int(max_over_ranks(float(ctx.device_status())))  # non-zero: a bounded device-side wait gave up
    parity = None
    if not args.no_parity:
        run_step()  # the output checked is that of the graph (or host-launched step) that was timed
        torch.cuda.synchronize()
        if shard is None:
            hc = host_copies(wl)
            parity = check_parity(kind, hc["row_ptr"], hc["col_idx"], hc["values"], hc["dense"], out)
            wl["host"] = hc
        elif kind == "bsr":
            parity = check_parity(kind, shard.block_row_ptr.cpu().numpy(), shard.block_col_idx.cpu().numpy(),
                                  shard.block_values.view(torch.uint16).cpu().numpy().reshape(-1),
                                  dense.view(torch.uint16).cpu().numpy(), out)
        else:
            parity = check_parity(kind, shard.row_ptr.cpu().numpy(), shard.col_idx.cpu().numpy(),
                                  shard.values.cpu().numpy(), dense.cpu().numpy(), out)
        parity = merge_parity(parity, env)
        parity["output"] = "the result of one more run of the timed step"
        barrier()

    gbs = wl["bytes"] / (ms_per_step * 1e-3) / 1e9
    gflops = wl["flops"] / (ms_per_step * 1e-3) / 1e9
    peak, tf_peak, peak_kind = measured_peaks()
    rec = {
        "workload": spec["name"], "options": options, **describe(wl), "n_gpus": world, "steps": steps,
        "warmup": max(warmup, 3), "ms_per_step": ms_per_step, "value": gbs, "unit": "GB/s", "gflops": gflops,
        "frac_of_hbm_peak": gbs / (peak * world), "bytes_algorithmic": wl["bytes"], "flops": wl["flops"],
        "gpu_launches": int(gpu_launches), "dispatch_stats": dispatch_stats, "device_status": device_status,
        "parity": parity,
        "l2": "inputs exceed L2" if flush is None else "256 MiB flush between timed steps" + (
            "; ranks lined up by a 16-byte all-gather between the flush and the event pair" if align is not None else ""),
        "launch": (f"CUDA graph of {per_graph} step(s), replayed" if graph is not None else "host launch per step"),
    }
    if world > 1:
        rec["dense_operand"] = "replicated" if args.replicated else (
            f"all-gathered each step ({gather_kind})" + (", overlapped with the locally-owned columns" if args.overlap else ""))
        rec["phases"] = phases

    # ---- roofline of the dominant kernel (one GPU) ------------------------------------------------
    if world == 1:
        rec["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                           "traffic": NCU_TRAFFIC_BYTES.get(name), "peak_kind": peak_kind,
                           "duration": "step time (zero fill + compute kernel where the mapping has both)"}
        if kind == "bsr":
            rec["roofline"]["tensor"] = {"achieved_tflops": gflops / 1e3, "peak_tflops": tf_peak,
                                         "frac": gflops / 1e3 / tf_peak, "peak_kind": "burst (kernel timed alone)"}
        if kind == "spmv" and a.nnz >= 4 and local_input_bytes > 2 * L2_BYTES:
            # What the matrix's own col/val streams and the gather of x cost with no row logic at all, on
            # the real columns and on sequential ones: the floor of any mapping that reads x[col[p]] through
            # the cache hierarchy, against which the kernel's time is read.
            seq = (torch.arange(a.nnz, device=device, dtype=torch.int64) % a.cols).to(torch.int32)
            bound = {}
            for label, cols_used in (("real_columns", a.col_idx), ("sequential_columns", seq)):
                probe = lambda: ctx.probe_stream_gather(cols_used, a.values, dense)
                for _ in range(3):
                    probe()
                torch.cuda.synchronize()
                bound[label + "_ms"] = timed(probe, 20) / 20
            del seq
            rec["roofline"].update(
                gather_bound_ms=bound["real_columns_ms"],
                gather_bound_gbs=wl["bytes"] / (bound["real_columns_ms"] * 1e-3) / 1e9,
                stream_only_ms=bound["sequential_columns_ms"],
                frac_of_gather_bound=bound["real_columns_ms"] / ms_per_step,
                gather_bound="swb_probe_stream_gather on this matrix's col/val and x (no rows, no output): with the "
                             "real columns and, as stream_only_ms, with column = position mod cols")

    # ---- vendor library on the same operands (comparison column only) ---------------------------
    if world == 1 and not args.no_library and kind in ("spmv", "spmm"):
        try:
            A = torch.sparse_csr_tensor(a.row_ptr, a.col_idx, a.values, size=(a.rows, a.cols))
            lib_step = (lambda: torch.mv(A, dense)) if kind == "spmv" else (lambda: torch.mm(A, dense))
            for _ in range(3):
                lib_step()
            torch.cuda.synchronize()
            n_lib = max(5, min(steps, 50))
            lib_ms = timed(lib_step, n_lib) / n_lib
            rec["library_baseline"] = {"name": "cuSPARSE via torch.sparse_csr", "ms_per_step": lib_ms,
                                       "value": wl["bytes"] / (lib_ms * 1e-3) / 1e9, "unit": "GB/s",
                                       "ours_over_library": lib_ms / ms_per_step}
            del A
        except Exception as exc:  # noqa: BLE001
            rec["library_baseline"] = {"unavailable": str(exc)}

    graph = one_graph = run_step = one_step = None  # the graphs hold the captured collective
    torch.cuda.synchronize()

    # ---- end to end through the host-buffer C-ABI call --------------------------------------
    if not args.no_e2e:
        rec["e2e"] = run_e2e(args, env, wl, options, shard, min(steps, 10 if headline else 5))

    # ---- CPU baseline (rank 0, one GPU) -----------------------------------------------------
    if world == 1 and not args.no_cpu:
        import oracle
        host = wl.get("host") or host_copies(wl)
        cores = oracle.use_all_cores()
        best, passes = time_cpu(wl, host, seconds=20.0 if headline else 4.0)
        rec["cpu_baseline"] = {"value": wl["bytes"] / best / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                               "ms_per_pass": best * 1e3,
                               "sample": f"{passes} passes over the whole workload, best pass, OpenMP over rows"}
    return rec


def run_e2e(args, env, wl, options, shard, steps):
    """The same operator through the host-buffer C-ABI calls with pinned host operands.

    One GPU, CSR: the matrix is uploaded once with swb_csr_upload (what the reference's host programs do before
    their dispatch loop, benchmark/spmv.mlir.in:37-65) and every timed step copies the dense operand in
    and the result out (swb_spmv_resident_host / swb_spmm_resident_host).  `full_upload` also times the
    variant that re-sends the whole matrix every step (swb_spmv_host / swb_spmm_host).
    N GPUs, CSR: every rank keeps its rows of the matrix (swb_csr_upload_rows) and a step sends only the rank's
    own chunk of the dense operand in, exchanges the chunks on the device, runs the shard's kernel and copies
    the rank's rows out (swb_spmv_sharded_host / swb_spmm_sharded_host).  BSR: the matrix (at N > 1 the rank's block rows)
    uploaded once with swb_bsr_upload, all of B in and the rows of C out per step."""
    import torch

    from sparsewave_b200 import sharding
    ctx, rank, world = env["ctx"], env["rank"], env["world"]
    barrier, max_over_ranks = env["barrier"], env["max_over_ranks"]
    kind, a, dense = wl["kind"], wl["a"], wl["dense"]
    pin = lambda t: t.cpu().contiguous().pin_memory()

    def measure(call, count):
        for _ in range(2):
            call()
        barrier()
        t0 = time.perf_counter()
        for _ in range(count):
            call()
        torch.cuda.synchronize()
        return max_over_ranks((time.perf_counter() - t0) * 1e3) / count

    steps = max(1, steps)
    timer = "host clock around the synchronous C-ABI calls, max over ranks"
    if kind == "bsr":
        brp, bci, bv, rows = a.block_row_ptr, a.block_col_idx, a.block_values, a.rows
        if world > 1:
            brp, bci, bv, rows = shard.block_row_ptr, shard.block_col_idx, shard.block_values, shard.rows
        h = [pin(brp), pin(bci), pin(bv), pin(dense)]
        out = torch.empty((rows, dense.shape[1]), dtype=torch.bfloat16).pin_memory()
        full_ms = measure(lambda: ctx.bsr_spmm_bf16_host(options, h[0], h[1], h[2], h[3], 16, out), steps)
        full = {"value": wl["bytes"] / (full_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": full_ms,
                "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in h)),
                "d2h_bytes_per_step": int(out.numel() * out.element_size()), "matrix": "sent every step"}
        # the (shard of the) matrix uploaded once, B in and C out every step
        resident = ctx.bsr_upload(a.cols, h[0], h[1], h[2], 16)
        ms = measure(lambda: resident.spmm_host(options, h[3], out), steps)
        resident.release()
        return {"value": wl["bytes"] / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "steps": steps,
                "h2d_bytes_per_step": int(h[3].numel() * h[3].element_size()),
                "d2h_bytes_per_step": int(out.numel() * out.element_size()),
                "matrix": "uploaded once before the timed steps (swb_bsr_upload); B in and C out every step",
                "full_upload": full, "timer": timer}
    if world > 1:
        # the rank's rows are cut out of the full host matrix by the library (row range from the nnz-balanced
        # boundaries); only the rank's chunk of the dense operand crosses PCIe per step
        bnd = sharding.shard_boundaries(a.row_ptr, world)
        full = [a.row_ptr.cpu().numpy(), a.col_idx.cpu().numpy(), a.values.cpu().numpy()]
        resident = ctx.csr_upload_rows(a.cols, full[0], full[1], full[2], int(bnd[rank]), int(bnd[rank + 1]))
        del full
        lo, hi = sharding.owned_dense_range(a.cols, world, rank)
        owned = pin(dense[lo:hi])
        shape = (shard.rows,) if kind == "spmv" else (shard.rows, dense.shape[1])
        out = torch.empty(shape, dtype=torch.float32).pin_memory()
        if kind == "spmv":
            ms = measure(lambda: resident.spmv_sharded_host(options, owned, out), steps)
        else:
            ms = measure(lambda: resident.spmm_sharded_host(options, owned, out), steps)
        # the result of the last call against the device-resident step's (same kernels, same operands)
        resident.release()
        return {"value": wl["bytes"] / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "steps": steps,
                "h2d_bytes_per_step": int(owned.numel() * owned.element_size()),
                "d2h_bytes_per_step": int(out.numel() * out.element_size()),
                "bytes": "per rank (rank 0's figures; the chunks and shards are of equal size up to rounding)",
                "matrix": "this rank's rows uploaded once (swb_csr_upload_rows); per step the rank's chunk of the "
                          "dense operand in, the exchange over NVLink on the device, the rank's rows out",
                "timer": timer}
    rp, ci, v, rows = a.row_ptr, a.col_idx, a.values, a.rows
    h = [pin(rp), pin(ci), pin(v), pin(dense)]
    shape = (rows,) if kind == "spmv" else (rows, dense.shape[1])
    out = torch.empty(shape, dtype=torch.float32).pin_memory()
    resident = ctx.csr_upload(rows, a.cols, h[0], h[1], h[2])
    if kind == "spmv":
        ms = measure(lambda: resident.spmv_host(options, h[3], out), steps)
        full_ms = measure(lambda: ctx.spmv_host(options, h[0], h[1], h[2], h[3], out), min(steps, 3))
    else:
        ms = measure(lambda: resident.spmm_host(options, h[3], out), steps)
        full_ms = measure(lambda: ctx.spmm_host(options, h[0], h[1], h[2], h[3], out), min(steps, 3))
    resident.release()
    dense_bytes = h[3].numel() * h[3].element_size()
    out_bytes = out.numel() * out.element_size()
    return {"value": wl["bytes"] / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "steps": steps,
            "h2d_bytes_per_step": int(dense_bytes), "d2h_bytes_per_step": int(out_bytes),
            "matrix": "uploaded once before the timed steps (swb_csr_upload); dense operand in and result out "
                      "every step",
            "full_upload": {"value": wl["bytes"] / (full_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": full_ms,
                            "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in h)),
                            "d2h_bytes_per_step": int(out_bytes), "matrix": "sent every step"},
            "timer": timer}


# Configuration 3 names three mappings to compare; the line carries them beside the headline mapping.
C3_MAPPINGS = [
    "spmv-mapping=thread-per-position spmv-position-chunk-size=8 spmv-position-reduction=segmented spmv-block-size=256",
    "spmv-mapping=thread-per-position spmv-block-size=256",
    "spmv-mapping=block-per-row spmv-block-size=64",
    "spmv-mapping=wave-per-row spmv-block-size=128",
]


def compare_mappings(env, option_strings, steps=10):
    """The other SpMV mappings on configuration 3: a few timed steps each and the same parity check."""
    import torch

    from sparsewave_b200 import make_options
    ctx, device = env["ctx"], env["device"]
    wl = build_workload("c3", device, None)
    a, x = wl["a"], wl["dense"]
    hc = host_copies(wl)
    y = torch.empty(a.rows, dtype=torch.float32, device=device)
    out = []
    for text in option_strings:
        opts = make_options(text)
        call = lambda: ctx.spmv(opts, a.row_ptr, a.col_idx, a.values, x, y)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            call()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        parity = check_parity("spmv", hc["row_ptr"], hc["col_idx"], hc["values"], hc["dense"], y)
        out.append({"options": text, "steps": steps, "ms_per_step": ms, "value": wl["bytes"] / (ms * 1e-3) / 1e9,
                    "unit": "GB/s", "launch": "host launch per step",
                    "parity": {k: parity[k] for k in ("checked_rows", "mismatches_north_star", "max_err_over_bound", "ok")}})
    return out


def write_results(args, records, line):
    """results.jsonl (one line per finished configuration, appended) and metadata.json: the sweep files of the
    reference runner (benchmark/benchmark_utils.py:1018-1059 in the SparseWave tree) in JSON form."""
    try:
        out = Path(args.results_dir)
        out.mkdir(parents=True, exist_ok=True)
        with open(out / "results.jsonl", "a") as f:
            for r in records:
                f.write(json.dumps(r) + "\n")
        meta = {"command": " ".join(sys.argv), "when": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
                "n_gpus": line["n_gpus"], "clocks": line.get("clocks"), "metric": METRIC,
                "configs": [r["workload"] for r in records]}
        (out / "metadata.json").write_text(json.dumps(meta, indent=1))
    except OSError as exc:
        print(f"bench: results files not written: {exc}", file=sys.stderr)


def run_ours(args):
    import torch
    import torch.distributed as dist
    env = init_env(args)
    rank, world, ctx = env["rank"], env["world"], env["ctx"]
    headline = args.workload or "c3"
    default_command = args.workload is None and args.options is None and args.rows is None

    # Clocks are sampled from the warm-up on; because one nvidia-smi query takes longer than a short
    # timed region, the same steps keep running (untimed) afterwards until a few samples exist.
    clocks = ClockSampler(env["local"])
    clocks.__enter__()
    rec = measure_workload(args, env, headline, headline=True, steps_arg=args.steps, warmup=args.warmup, clocks=clocks)
    records = [rec]
    mappings = None
    if default_command and world == 1 and not args.no_configs:
        try:
            mappings = compare_mappings(env, C3_MAPPINGS)
        except Exception as exc:  # noqa: BLE001
            mappings = [{"failed": repr(exc), "parity": {"ok": False}}]
        torch.cuda.empty_cache()
        for name in ("c1", "c2", "c4", "c5"):
            try:
                records.append(measure_workload(args, env, name, headline=False, steps_arg=None, warmup=3))
            except Exception as exc:  # noqa: BLE001  (the headline stands; the failed configuration is named)
                records.append({"workload": WORKLOADS[name]["name"], "failed": repr(exc),
                                "parity": {"ok": False}, "device_status": -1})
            torch.cuda.empty_cache()

    def shutdown():
        # Orderly on every rank: drain the GPU, tear the window down together, release the library's
        # communicator, then torch.distributed's.
        torch.cuda.synchronize()
        if world > 1:
            env["barrier"]()
            ctx.window_destroy()
        ctx.close()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()

    bad = [r["workload"] for r in records
           if r.get("device_status", 0) != 0 or (r.get("parity") is not None and not r["parity"].get("ok", False))]
    bad += ["c3 with " + m.get("options", "?") for m in (mappings or []) if not m["parity"].get("ok", False)]
    if rank == 0:
        line = {
            "metric": METRIC, "value": rec["value"], "unit": "GB/s", "n_gpus": world, "steps": rec["steps"],
            "warmup": rec["warmup"], "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16" if WORKLOADS[headline]["kind"] == "bsr" else "f32",
            "data": "synthetic",
            "config": {k: rec[k] for k in ("workload", "options", "rows", "cols", "nnz", "nnzb", "block_size", "n_rhs",
                                           "bytes_algorithmic", "flops", "dense_operand", "l2", "launch") if k in rec},
            "gflops": rec["gflops"], "frac_of_hbm_peak": rec["frac_of_hbm_peak"], "gpu_launches": rec["gpu_launches"],
            "clocks": clocks.summary(), "e2e": rec.get("e2e"), "dispatch_stats": rec["dispatch_stats"],
            "device_status": rec["device_status"], "parity": rec["parity"],
        }
        if world > 1:
            line["phases"] = rec.get("phases")
            line["config"].setdefault("dense_operand", "replicated")
        else:
            line["config"]["dense_operand"] = "replicated"
            line["roofline"] = rec.get("roofline")
            line["cpu_baseline"] = rec.get("cpu_baseline")
            if "library_baseline" in rec:
                line["library_baseline"] = rec["library_baseline"]
            if len(records) > 1:
                keep = ("workload", "options", "steps", "ms_per_step", "value", "unit", "gflops", "roofline", "parity",
                        "cpu_baseline", "library_baseline", "e2e", "gpu_launches", "device_status", "l2", "launch",
                        "failed")
                line["configs"] = [{k: r[k] for k in keep if k in r} for r in records[1:]]
            if mappings is not None:
                line["mappings"] = mappings  # the other SpMV mappings on the headline matrix
        if bad:
            line["void"] = "output mismatch or device status in: " + "; ".join(bad)
        print(json.dumps(line), flush=True)
        write_results(args, records, line)
    shutdown()
    if bad:
        print("bench: a timed step's output did not match the oracle, or a bounded device wait gave up: "
              + "; ".join(bad), file=sys.stderr)
        sys.exit(1)


def run_reference(args):
    """The reference's CPU CSR loop (restated in oracle/swb_oracle.c, all host threads) on the same workload."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    import oracle
    name = args.workload or "c3"
    spec = WORKLOADS[name]
    # Launchers that start one process per GPU export OMP_NUM_THREADS=1; this arm is the only user of the
    # host cores, so it takes all the cores the process may run on.
    cores = oracle.use_all_cores()
    try:
        import torch
        device = "cuda" if torch.cuda.is_available() else "cpu"  # the GPU only generates the inputs
        wl = build_workload(name, device, args.rows)
        host = host_copies(wl)
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"could not build the workload: {e}"}))
        return
    warm = max(1, min(args.warmup, 3))
    for _ in range(warm):
        cpu_pass(wl, host)
    steps = args.steps
    if steps is None:
        t0 = time.perf_counter()
        cpu_pass(wl, host)
        steps = int(min(200, max(5, 20.0 / max(time.perf_counter() - t0, 1e-4))))
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_pass(wl, host)
    ms = (time.perf_counter() - t0) * 1e3 / steps
    gbs = wl["bytes"] / (ms * 1e-3) / 1e9
    sample = "every step is one pass over the whole workload, OpenMP over rows"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if wl["kind"] == "bsr" else "f32",
        "data": "synthetic",
        "config": {"workload": spec["name"], **describe(wl), "bytes_algorithmic": wl["bytes"], "flops": wl["flops"]},
        "gflops": wl["flops"] / (ms * 1e-3) / 1e9,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
