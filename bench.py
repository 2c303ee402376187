"""Benchmark of the SpMV / SpMM / BSR-SpMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5]
                    [--impl ours|reference] [--options "..."] [--rows R]

One step = one operator call over the whole synthetic workload (for N > 1: the
all-gather of the dense operand plus the local kernel on this rank's row
shard).  Rank 0 prints one JSON line.  `value` is algorithmic GB/s with the
operands resident in HBM; `e2e` is the same metric through the host-buffer
C-ABI call (H2D of the operands and D2H of the result inside the timed
region); `roofline` compares the kernel with the measured HBM copy bandwidth;
`cpu_baseline` times the CPU restatement of the reference loop on the host
cores.  `--impl reference` times only that CPU loop.
"""
from __future__ import annotations

import argparse
import json
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
    "c3": dict(kind="spmv", options="spmv-mapping=wave-per-position spmv-block-size=256",
               name="c3: power-law CSR SpMV 4194304x4194304, Zipf(1.8) rows in [1,65536], f32/i32"),
    "c4": dict(kind="spmm", options="spmm-mapping=wave-per-row-tile spmm-tile-size=16 spmm-block-size=256",
               name="c4: CSR SpMM 2097152x2097152, 32 banded + 32 random nnz/row, N=64, f32/i32"),
    "c5": dict(kind="bsr", options="",
               name="c5: BSR SpMM 16384x16384, 16x16 bf16 blocks at 5% density, N=512"),
}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel at the full workload size,
# from the one-pass ncu captures summarised under profiles/ (None where no capture exists).
NCU_TRAFFIC_BYTES = {"c2": 18.1e6, "c3": 1.095e9, "c4": 16.71e9, "c5": 45.3e6}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    p.add_argument("--options", default=None, help="option string in the reference's spelling")
    p.add_argument("--rows", type=int, default=None, help="override the row count (testing)")
    p.add_argument("--no-graph", action="store_true", help="launch every step from the host instead of replaying "
                   "a CUDA graph of one step")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-cpu", action="store_true")
    p.add_argument("--compare-library", action="store_true",
                   help="also time cuSPARSE (through torch.sparse) on the same operands, like the reference's "
                        "rocSPARSE column; comparison only")
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


def run_ours(args):
    import torch
    import torch.distributed as dist

    from sparsewave_b200 import Context, sharding

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    ctx = Context(local)
    if world > 1 and not args.torch_collective:
        ctx.comm_init(rank, world)  # the library's own NCCL communicator (capturable in the step's CUDA graph)
    spec = WORKLOADS[args.workload]
    options = args.options if args.options is not None else spec["options"]
    from sparsewave_b200 import make_options
    opts = make_options(options)  # parsed once; the steps pass the option block
    wl = build_workload(args.workload, device, args.rows)
    kind, a, dense = wl["kind"], wl["a"], wl["dense"]
    gather_kind = "library NCCL communicator"

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
        local_input_bytes = 512 * shard.nnzb + dense.numel() * 2
    elif world > 1:
        shard = sharding.shard_csr(a.row_ptr, a.col_idx, a.values, a.cols, rank, world)
        overlap = args.overlap and not args.replicated and not args.torch_collective
        nbytes = sharding.window_bytes(a.cols, world, tuple(dense.shape[1:]), dense.element_size())
        if not (args.nccl_allgather or args.torch_collective or args.replicated or overlap) and nbytes % 16 == 0:
            # The library's own exchange kernel.  Creation succeeds on every rank or on none; before it is
            # used, two exchanges of a rank-coded pattern are checked on every rank, and one bad rank sends
            # all of them back to ncclAllGather.
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
                    gather_kind = "peer-store kernel over NVLink into CUDA IPC windows"
                else:
                    print("bench: the peer-window self-check failed, using ncclAllGather", file=sys.stderr)
                    ctx.window_destroy()
                del probe
            except Exception as exc:  # noqa: BLE001  (no CUDA IPC between these processes: same on every rank)
                print(f"bench: peer window unavailable, using ncclAllGather: {exc}", file=sys.stderr)
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
        local_input_bytes = wl["bytes"]

    def barrier():
        # Drain this rank's queue first: the library's communicator and torch.distributed's are two NCCL
        # communicators on the same GPUs, and collectives of both in flight at once can wait on each other.
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Inputs larger than L2 need no flush; smaller ones get a 256 MiB write between timed steps.
    flush = None
    if local_input_bytes <= 2 * L2_BYTES:
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)

    def timed(fn, steps):
        """Device time of `steps` calls in ms: one event pair around all of them, or one
        pair per step with an L2 flush outside the pairs."""
        if flush is None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1)
        pairs = []
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            pairs.append((e0, e1))
        torch.cuda.synchronize()
        return sum(p[0].elapsed_time(p[1]) for p in pairs)

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # Clocks are sampled from the warm-up on; because one nvidia-smi query takes longer than a short
    # timed region, the same steps keep running (untimed) afterwards until a few samples exist.
    with ClockSampler(local) as clocks:
        for _ in range(max(args.warmup, 3)):
            step()
        barrier()
        # One step (collective + kernels) captured in a CUDA graph and replayed: a timed step is then a single
        # graph launch with no host work between its kernels (with the L2 flush, which stays outside the
        # event pairs, the replay sits between the two event records).  Host launches remain for
        # steps whose all-gather goes through torch.distributed (capturing that one hung here, so it is not
        # tried); the library's own ncclAllGather is captured with the kernels.
        eager_step, launches_per_step, graph = step, None, None
        torch_collective = world > 1 and not args.replicated and args.torch_collective
        if not args.no_graph and not torch_collective:
            try:
                before = ctx.kernel_launches
                g = torch.cuda.CUDAGraph()
                # relaxed: NCCL's helper threads may issue CUDA calls of their own while this thread captures
                with torch.cuda.graph(g, capture_error_mode="relaxed"):
                    eager_step()
                launches_per_step = ctx.kernel_launches - before
                g.replay()
                torch.cuda.synchronize()
                graph, step = g, g.replay
                g = None
            except Exception as exc:  # noqa: BLE001
                print(f"bench: CUDA graph capture failed, launching from the host: {exc}", file=sys.stderr)
                torch.cuda.synchronize()
        barrier()
        launches0 = ctx.kernel_launches
        total_ms = timed(step, args.steps)
        launches1 = ctx.kernel_launches
        barrier()
        # The reference's own convention (benchmark/benchmark_utils.py:520-521): 10 warm-up dispatches, 50
        # timed ones, each with its own event pair; median / min / p95 of those (max over ranks per dispatch).
        per_dispatch = []
        for i in range(60):
            if flush is not None:
                flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            if i >= 10:
                per_dispatch.append((e0, e1))
        torch.cuda.synchronize()
        times = torch.tensor([a.elapsed_time(b) for a, b in per_dispatch], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
        times = sorted(times.tolist())
        dispatch_stats = {"warmup": 10, "dispatches": 50, "median_ms": times[len(times) // 2], "min_ms": times[0],
                          "p95_ms": times[min(len(times) - 1, int(round(0.95 * (len(times) - 1))))]}
        barrier()
        # Keep the same steps running for about 0.3 s so that the sampler sees the clocks under this
        # load.  The step count comes from the rank-reduced time, so every rank runs the same number
        # of steps (they contain a collective when N > 1).
        soak_steps = int(min(5000, max(10, 300.0 / max(max_over_ranks(total_ms) / args.steps, 1e-3))))
        for _ in range(soak_steps):
            step()
        barrier()
    device_status = ctx.device_status()  # non-zero: a bounded device-side wait gave up, the numbers are void
    if device_status != 0:
        print(f"bench: rank {rank}: device status {device_status}: a bounded wait gave up", file=sys.stderr)
    gpu_launches = launches1 - launches0 if graph is None else launches_per_step * args.steps
    total_ms = max_over_ranks(total_ms)
    ms_per_step = total_ms / args.steps
    gbs = wl["bytes"] / (ms_per_step * 1e-3) / 1e9
    gflops = wl["flops"] / (ms_per_step * 1e-3) / 1e9

    # ---- vendor library on the same operands (comparison column only) ---------------------------
    library = None
    if args.compare_library and world == 1 and kind in ("spmv", "spmm"):
        A = torch.sparse_csr_tensor(a.row_ptr, a.col_idx, a.values, size=(a.rows, a.cols))
        lib_step = (lambda: torch.mv(A, dense)) if kind == "spmv" else (lambda: torch.mm(A, dense))
        for _ in range(3):
            lib_step()
        torch.cuda.synchronize()
        lib_ms = timed(lib_step, args.steps) / args.steps
        library = {"name": "cuSPARSE via torch.sparse_csr", "ms_per_step": lib_ms,
                   "value": wl["bytes"] / (lib_ms * 1e-3) / 1e9, "unit": "GB/s"}
        del A

    # ---- end to end through the host-buffer C-ABI call --------------------------------------
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, ctx, wl, options, rank, world, device, barrier, max_over_ranks)

    # ---- CPU baseline (rank 0, one GPU) -----------------------------------------------------
    cpu = None
    if world == 1 and not args.no_cpu:
        import oracle
        host = host_copies(wl)
        best, passes = time_cpu(wl, host)
        cpu = {"value": wl["bytes"] / best / 1e9, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
               "ms_per_pass": best * 1e3,
               "sample": f"{passes} passes over the whole workload, best pass, OpenMP over rows"}

    def shutdown():
        # Orderly on every rank: drop the graph (it holds the captured collective), drain the GPU, release
        # the library's communicator, then torch.distributed's.
        nonlocal graph, step
        graph = step = None
        torch.cuda.synchronize()
        ctx.close()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()

    if rank != 0:
        shutdown()
        return
    peak, tf_peak, peak_kind = measured_peaks()
    line = {
        "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16" if kind == "bsr" else "f32", "data": "synthetic",
        "config": {"workload": spec["name"], "options": options, **describe(wl),
                   "bytes_algorithmic": wl["bytes"], "flops": wl["flops"],
                   "dense_operand": "replicated" if (world == 1 or args.replicated) else
                   ("all-gathered each step (torch.distributed)" if args.torch_collective
                    else f"all-gathered each step ({gather_kind})" +
                    (", overlapped with the locally-owned columns" if args.overlap else "")),
                   "l2": "inputs exceed L2" if flush is None else "256 MiB flush between timed steps",
                   "launch": "CUDA graph of one step, replayed" if graph is not None else "host launch per step"},
        "gflops": gflops, "frac_of_hbm_peak": gbs / (peak * world), "gpu_launches": int(gpu_launches),
        "clocks": clocks.summary(), "e2e": e2e, "dispatch_stats": dispatch_stats, "device_status": device_status,
    }
    if world == 1:
        line["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                            "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "peak_kind": peak_kind,
                            "duration": "step time (zero fill + compute kernel where the mapping has both)"}
        if kind == "bsr":
            line["roofline"]["tensor"] = {"achieved_tflops": gflops / 1e3, "peak_tflops": tf_peak,
                                          "frac": gflops / 1e3 / tf_peak}
        line["cpu_baseline"] = cpu
        if library is not None:
            line["library_baseline"] = library
    print(json.dumps(line), flush=True)
    shutdown()


def run_e2e(args, ctx, wl, options, rank, world, device, barrier, max_over_ranks):
    """The same operator through the host-buffer C-ABI calls with pinned host operands.

    CSR: the matrix is uploaded once with swb_csr_upload (what the reference's host programs do before
    their dispatch loop, benchmark/spmv.mlir.in:37-65) and every timed step copies the dense operand in
    and the result out (swb_spmv_resident_host / swb_spmm_resident_host).  `full_upload` also times the
    variant that re-sends the whole matrix every step (swb_spmv_host / swb_spmm_host).  BSR has only the
    full-upload call."""
    import torch

    from sparsewave_b200 import sharding
    kind, a, dense = wl["kind"], wl["a"], wl["dense"]
    pin = lambda t: t.cpu().contiguous().pin_memory()

    def measure(call, steps):
        for _ in range(2):
            call()
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            call()
        torch.cuda.synchronize()
        return max_over_ranks((time.perf_counter() - t0) * 1e3) / steps

    steps = max(1, min(args.steps, 10))
    timer = "host clock around the synchronous C-ABI calls, max over ranks"
    if kind == "bsr":
        brp, bci, bv, rows = a.block_row_ptr, a.block_col_idx, a.block_values, a.rows
        if world > 1:
            s = sharding.shard_bsr(brp, bci, bv, a.cols, 16, rank, world)
            brp, bci, bv, rows = s.block_row_ptr, s.block_col_idx, s.block_values, s.rows
        h = [pin(brp), pin(bci), pin(bv), pin(dense)]
        out = torch.empty((rows, dense.shape[1]), dtype=torch.bfloat16).pin_memory()
        ms = measure(lambda: ctx.bsr_spmm_bf16_host(options, h[0], h[1], h[2], h[3], 16, out), steps)
        return {"value": wl["bytes"] / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "steps": steps,
                "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in h)),
                "d2h_bytes_per_step": int(out.numel() * out.element_size()), "matrix": "sent every step",
                "timer": timer}
    if world > 1:
        s = sharding.shard_csr(a.row_ptr, a.col_idx, a.values, a.cols, rank, world)
        rp, ci, v, rows = s.row_ptr, s.col_idx, s.values, s.rows
    else:
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


def run_reference(args):
    """The reference's CPU CSR loop (restated in oracle/swb_oracle.c, all host threads) on the same workload."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    import oracle
    spec = WORKLOADS[args.workload]
    try:
        import torch
        device = "cuda" if torch.cuda.is_available() else "cpu"  # the GPU only generates the inputs
        wl = build_workload(args.workload, device, args.rows)
        host = host_copies(wl)
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"could not build the workload: {e}"}))
        return
    for _ in range(max(1, min(args.warmup, 3))):
        cpu_pass(wl, host)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(wl, host)
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    gbs = wl["bytes"] / (ms * 1e-3) / 1e9
    cores = oracle.num_threads()
    sample = "every step is one pass over the whole workload, OpenMP over rows"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(1, min(args.warmup, 3)), "ms_per_step": ms, "higher_is_better": True,
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
