"""swb_runner, the native benchmark runner: argument and file errors on CPU, a timed and validated
run per mapping on the GPU (the reference's runners end with the mismatch count `[0]`,
benchmark/benchmark_utils.py:707-716)."""
import subprocess

import numpy as np
import pytest

from sparsewave_b200 import build, formats
from tests.helpers import random_csr

RUNNER = build.RUNNER


def run(*args):
    return subprocess.run([str(RUNNER), *map(str, args)], capture_output=True, text=True, timeout=300)


def test_runner_is_built():
    assert RUNNER.exists(), "python -m sparsewave_b200.build builds lib/swb_runner"


def test_argument_and_file_errors(tmp_path):
    r = run("--csr", tmp_path / "missing.csr")
    assert r.returncode == 1 and "could not open" in r.stderr
    bad = tmp_path / "bad.csr"
    bad.write_bytes(b"NOTACSR0" + b"\0" * 64)
    r = run("--csr", bad)
    assert r.returncode == 1 and "invalid CSR binary header" in r.stderr
    r = run("--operation", "sddmm", "--csr", bad)
    assert r.returncode == 1 and "--operation must be spmv or spmm" in r.stderr
    r = run()
    assert r.returncode == 1 and "--csr is required" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("operation,options", [
    ("spmv", "spmv-mapping=thread-per-row"), ("spmv", "spmv-mapping=wave-per-row spmv-block-size=128"),
    ("spmv", "spmv-mapping=block-per-row spmv-block-size=64"), ("spmv", "spmv-mapping=wave-per-position"),
    ("spmv", "spmv-mapping=thread-per-position spmv-position-chunk-size=8 spmv-position-reduction=segmented"),
    ("spmm", "spmm-mapping=thread-per-output"), ("spmm", "spmm-mapping=wave-per-row-tile spmm-tile-size=4 spmm-block-size=64"),
])
def test_timed_and_validated_run(tmp_path, operation, options):
    rp, ci, v = random_csr(4000, 3000, 12, seed=31)
    path = tmp_path / "m.csr"
    formats.write_csr_binary(path, 4000, 3000, rp, ci, v)
    r = run("--csr", path, "--operation", operation, "--options", options, "--rhs-columns", 4, "--warmup", 2,
            "--iterations", 5)
    assert r.returncode == 0, r.stderr
    lines = r.stdout.strip().splitlines()
    assert lines[-1] == "[0]"
    fields = dict(line.split("=", 1) for line in lines[:-1])
    assert len(fields["timings_us"].split(",")) == 5
    assert float(fields["min_us"]) <= float(fields["median_us"]) <= float(fields["p95_us"])
    assert float(fields["gflops"]) > 0 and int(fields["nnz"]) == len(v)


@pytest.mark.gpu
def test_option_errors_surface_the_reference_diagnostic(tmp_path):
    rp, ci, v = random_csr(100, 100, 4, seed=1)
    path = tmp_path / "m.csr"
    formats.write_csr_binary(path, 100, 100, rp, ci, v)
    r = run("--csr", path, "--options", "spmv-mapping=wave-per-row spmv-block-size=48")
    assert r.returncode == 1 and "wave-per-row requires the SpMV block size to be a multiple of 32, but got 48" in r.stderr
