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
