"""CUDA flavour of the SparseWave lrrt bundle.

The reference's `sparsewave-bundle` writes `manifest.json` + `kernels.hsaco`
for a fixed-shape SpMM and verifies them (tools/sparsewave-bundle/
sparsewave-bundle.py:232-284, sparsewave_bundle_manifest.py:73-120,
sparsewave_bundle_verify.py:83-111).  `write_bundle` produces the same
manifest shape with a cubin for sm_100a; `verify_bundle` re-checks it;
`load_and_launch` is the executor side (CUDA driver API), used by the tests.

    python -m sparsewave_b200.bundle --output DIR --rows N [--verify]
"""
from __future__ import annotations

import argparse
import hashlib
import json
import shutil
import subprocess
from pathlib import Path

MANIFEST_VERSION = 1
CODE_OBJECT = "kernels.cubin"
TARGET = "sm_100a"
SPMM_ARGUMENT_NAMES = ("rowOffsets", "columnIndices", "values", "rhs", "output")
SUPPORTED = {"mapping": "wave-per-row-tile", "block_size": 64, "tile_size": 4, "wavefront_size": 32}
KERNEL_SOURCE = Path(__file__).resolve().parent / "spmm_bundle_kernel.cu"
SYMBOL = "spmm_kernel"


class BundleError(RuntimeError):
    pass


def grid_expression(block_size: int, wavefront_size: int) -> str:
    """Total work-items, as in sparsewave_bundle_manifest.py:64-66."""
    return f"ceil_div(n, {block_size // wavefront_size}) * {block_size}"


def validate_supported_options(mapping, block_size, tile_size, wavefront_size, chip=TARGET):
    """The bundle launch contract is fixed (sparsewave-bundle.py:158-187)."""
    requested = {"chip": (chip, TARGET), "block size": (block_size, SUPPORTED["block_size"]),
                 "wavefront size": (wavefront_size, SUPPORTED["wavefront_size"]),
                 "mapping": (mapping, SUPPORTED["mapping"]), "tile size": (tile_size, SUPPORTED["tile_size"])}
    for label, (actual, supported) in requested.items():
        if actual != supported:
            raise BundleError(f"initial lrrt bundle support requires {label} {supported}, got {actual}")


def manifest_for(cubin: Path, rows: int) -> dict:
    digest = hashlib.sha256(cubin.read_bytes()).hexdigest()
    return {
        "manifest_version": MANIFEST_VERSION,
        "target": TARGET,
        "kernels": [{
            "name": "spmm",
            "symbol": SYMBOL,
            "code_object": CODE_OBJECT,
            "args": [{"name": n, "type": "ptr", "offset": 8 * i, "size": 8}
                     for i, n in enumerate(SPMM_ARGUMENT_NAMES)],
            "kernarg_size": 40,
            "block": [SUPPORTED["block_size"], 1, 1],
            "grid": [grid_expression(SUPPORTED["block_size"], SUPPORTED["wavefront_size"]), 1, 1],
            "shared_memory_bytes": 0,
            "workspace_bytes": 0,
            "sparsewave": {
                "operation": "spmm", "mapping": SUPPORTED["mapping"], "tile_size": SUPPORTED["tile_size"],
                "wavefront_size": SUPPORTED["wavefront_size"], "cubin_sha256": digest,
                "launch_n": "output_rows", "fixed_output_rows": int(rows), "rhs_columns": 4,
            },
        }],
    }


def write_bundle(output: Path, rows: int, mapping="wave-per-row-tile", block_size=64, tile_size=4,
                 wavefront_size=32) -> dict:
    """Compiles the fixed-shape kernel to a cubin and writes the manifest next to it."""
    validate_supported_options(mapping, block_size, tile_size, wavefront_size)
    if rows <= 0:
        raise BundleError("fixed_output_rows must be positive")
    output = Path(output)
    output.mkdir(parents=True, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cubin = output / CODE_OBJECT
    subprocess.run([nvcc, "-cubin", "-gencode", "arch=compute_100a,code=sm_100a", "-O3",
                    f"-DSWB_BUNDLE_ROWS={int(rows)}", str(KERNEL_SOURCE), "-o", str(cubin)], check=True)
    manifest = manifest_for(cubin, rows)
    (output / "manifest.json").write_text(json.dumps(manifest, indent=2) + "\n")
    verify_bundle(output)
    return manifest


def verify_bundle(directory: Path) -> dict:
    """Checks the bundle the way sparsewave_bundle_verify.py does: version, target, one `spmm` kernel,
    code-object digest, symbol present, positional pointer arguments at offsets 0..32, block, grid
    expression, no shared memory or workspace, producer fields."""
    directory = Path(directory)
    manifest = json.loads((directory / "manifest.json").read_text())
    if manifest.get("manifest_version") != MANIFEST_VERSION:
        raise BundleError("unsupported manifest_version")
    if manifest.get("target") != TARGET:
        raise BundleError(f"manifest target must be '{TARGET}'")
    kernels = manifest.get("kernels")
    if not isinstance(kernels, list) or len(kernels) != 1:
        raise BundleError("expected exactly one kernel")
    kernel = kernels[0]
    if kernel.get("name") != "spmm":
        raise BundleError("initial SparseWave logical kernel name must be 'spmm'")
    if kernel.get("code_object") != CODE_OBJECT:
        raise BundleError(f"kernel code_object must be '{CODE_OBJECT}'")
    blob = (directory / CODE_OBJECT).read_bytes()
    producer = kernel.get("sparsewave", {})
    if hashlib.sha256(blob).hexdigest() != producer.get("cubin_sha256"):
        raise BundleError("code object digest does not match the manifest")
    if blob[:4] != b"\x7fELF" or kernel.get("symbol", "").encode() not in blob:
        raise BundleError("code object does not define the manifest symbol")
    expected_args = [{"name": n, "type": "ptr", "offset": 8 * i, "size": 8} for i, n in enumerate(SPMM_ARGUMENT_NAMES)]
    if kernel.get("args") != expected_args or kernel.get("kernarg_size") != 40:
        raise BundleError("manifest arguments are not the positional SpMM pointer ABI")
    if kernel.get("block") != [SUPPORTED["block_size"], 1, 1]:
        raise BundleError("manifest block does not match the supported launch contract")
    if kernel.get("grid") != [grid_expression(SUPPORTED["block_size"], SUPPORTED["wavefront_size"]), 1, 1]:
        raise BundleError("manifest grid is not the supported total-work-item expression")
    if kernel.get("shared_memory_bytes") != 0 or kernel.get("workspace_bytes") != 0:
        raise BundleError("the SpMM bundle uses no shared memory and no workspace")
    for field, expected in {"operation": "spmm", "mapping": SUPPORTED["mapping"], "tile_size": SUPPORTED["tile_size"],
                            "wavefront_size": SUPPORTED["wavefront_size"], "launch_n": "output_rows"}.items():
        if producer.get(field) != expected:
            raise BundleError(f"invalid sparsewave producer field '{field}'")
    if not isinstance(producer.get("fixed_output_rows"), int) or producer["fixed_output_rows"] <= 0:
        raise BundleError("invalid sparsewave producer field 'fixed_output_rows'")
    return manifest


def load_and_launch(directory: Path, n: int, pointers, stream: int = 0) -> None:
    """Executor side: loads the cubin with the CUDA driver API and launches the manifest's kernel with
    `n` output rows and the five device pointers (ints) in manifest order."""
    from cuda.bindings import driver
    import ctypes

    manifest = verify_bundle(directory)
    kernel = manifest["kernels"][0]
    if n != kernel["sparsewave"]["fixed_output_rows"]:
        raise BundleError("n does not match the bundle's fixed_output_rows")

    def check(result):
        err, *rest = result
        if err != driver.CUresult.CUDA_SUCCESS:
            raise BundleError(f"CUDA driver error {err}")
        return rest[0] if rest else None

    module = check(driver.cuModuleLoadData((Path(directory) / CODE_OBJECT).read_bytes()))
    function = check(driver.cuModuleGetFunction(module, kernel["symbol"].encode()))
    block = kernel["block"][0]
    waves_per_block = block // kernel["sparsewave"]["wavefront_size"]
    total_items = -(-n // waves_per_block) * block      # the manifest's grid expression
    args = (ctypes.c_void_p * 5)(*[ctypes.c_void_p(int(p)) for p in pointers])
    arg_ptrs = (ctypes.c_void_p * 5)(*[ctypes.addressof(args) + 8 * i for i in range(5)])
    check(driver.cuLaunchKernel(function, total_items // block, 1, 1, block, 1, 1, 0, stream,
                                ctypes.addressof(arg_ptrs), 0))
    check(driver.cuStreamSynchronize(stream))
    check(driver.cuModuleUnload(module))


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--output", required=True)
    p.add_argument("--rows", type=int)
    p.add_argument("--mapping", default="wave-per-row-tile")
    p.add_argument("--block-size", type=int, default=64)
    p.add_argument("--tile-size", type=int, default=4)
    p.add_argument("--wavefront-size", type=int, default=32)
    p.add_argument("--verify", action="store_true", help="only verify an existing bundle")
    a = p.parse_args(argv)
    if a.verify:
        verify_bundle(Path(a.output))
        print("bundle ok")
        return
    if a.rows is None:
        p.error("--rows is required")
    write_bundle(Path(a.output), a.rows, a.mapping, a.block_size, a.tile_size, a.wavefront_size)
    print(Path(a.output) / "manifest.json")


if __name__ == "__main__":
    main()
