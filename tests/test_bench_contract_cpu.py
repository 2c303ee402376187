"""The reference arm of bench.py runs without a GPU: its JSON line carries the contract's keys, and ranks
other than 0 print nothing."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _run(extra_env=None, workload="c1"):
    env = dict(os.environ, **(extra_env or {}))
    p = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--workload", workload, "--steps", "2",
                        "--warmup", "1"], capture_output=True, text=True, cwd=ROOT, env=env, timeout=300)
    assert p.returncode == 0, p.stderr
    return p.stdout.strip()


def test_reference_arm_json_line():
    line = json.loads(_run().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["metric"] == "SpMV/SpMM effective HBM GB/s" and line["steps"] == 2 and line["n_gpus"] == 1
    assert line["config"]["workload"].startswith("c1") and line["config"]["nnz"] == 65536
    assert line["config"]["bytes_algorithmic"] == 8 * 65536 + 4 * 4097 + 4 * 4096 + 4 * 4096
    cpu = line["cpu_baseline"]
    assert cpu["kind"] == "port" and cpu["cores"] >= 1 and cpu["value"] == line["value"] and cpu["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["value"] > 0 and line["ms_per_step"] > 0


def test_reference_arm_other_ranks_stay_silent():
    assert _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}) == ""


def test_reference_arm_spmm_and_bsr_workloads():
    for workload, kind_key in (("c2", "n_rhs"), ("c5", "nnzb")):
        line = json.loads(_run(workload=workload).splitlines()[-1])
        assert kind_key in line["config"] and line["value"] > 0


def test_parity_record_counts_mismatches():
    """bench.check_parity on CPU tensors: the oracle's own output passes, one corrupted output is counted under
    both criteria and fails the record; bf16 BSR outputs are held to one ulp of the oracle's bits."""
    import numpy as np
    import torch

    import bench
    import oracle
    from tests.helpers import random_csr
    rp, ci, v = random_csr(300, 200, 7, seed=5)
    rng = np.random.default_rng(5)
    x = rng.uniform(-1, 1, 200).astype(np.float32)
    B = rng.uniform(-1, 1, (200, 8)).astype(np.float32)
    y = torch.from_numpy(oracle.csr_spmv(rp, ci, v, x))
    rec = bench.check_parity("spmv", rp, ci, v, x, y, block_elems=64)  # several row blocks
    assert rec["ok"] and rec["checked_rows"] == 300 and rec["mismatches_north_star"] == 0
    y[17] += 1.0
    rec = bench.check_parity("spmv", rp, ci, v, x, y)
    assert not rec["ok"] and rec["mismatches_north_star"] == 1 and rec["mismatches_reference_1e-4"] == 1
    C = torch.from_numpy(oracle.csr_spmm(rp, ci, v, B))
    rec = bench.check_parity("spmm", rp, ci, v, B, C, block_elems=256)
    assert rec["ok"] and rec["checked_outputs"] == 300 * 8
    from sparsewave_b200 import workloads as W
    a = W.random_bsr(6, 5, 16, 0.5, seed=3)
    Bb = W.dense_normal((80, 16), seed=3)
    operands = (a.block_row_ptr.numpy(), a.block_col_idx.numpy(), a.block_values.view(torch.uint16).numpy(),
                Bb.view(torch.uint16).numpy())
    bits, _ = oracle.bsr_spmm_bf16(*operands, 16)
    good = torch.from_numpy(bits.copy()).view(torch.bfloat16)
    assert bench.check_parity("bsr", *operands, good)["ok"]
    bits[3, 5] += 3  # three ulps off
    rec = bench.check_parity("bsr", *operands, torch.from_numpy(bits).view(torch.bfloat16))
    assert not rec["ok"] and rec["mismatches_beyond_one_bf16_ulp"] == 1
