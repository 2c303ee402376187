"""CUDA bundle (manifest.json + kernels.cubin) in the shape of the reference's lrrt bundle
(test/Driver/bundle_test.py:133-163 manifest fields, :350-365 unsupported launch contracts, :367-433
verification after mutation)."""
import json

import numpy as np
import pytest
import torch

import oracle
from sparsewave_b200 import bundle
from tests.helpers import random_csr


@pytest.fixture(scope="module")
def built(tmp_path_factory):
    d = tmp_path_factory.mktemp("bundle")
    return d, bundle.write_bundle(d, rows=1000)


def test_manifest_fields(built):
    _, manifest = built
    assert manifest["manifest_version"] == 1 and manifest["target"] == "sm_100a"
    k = manifest["kernels"][0]
    assert (k["name"], k["symbol"], k["code_object"]) == ("spmm", "spmm_kernel", "kernels.cubin")
    assert k["kernarg_size"] == 40 and k["block"] == [64, 1, 1] and k["grid"] == ["ceil_div(n, 2) * 64", 1, 1]
    assert k["shared_memory_bytes"] == 0 and k["workspace_bytes"] == 0
    assert k["args"] == [{"name": n, "type": "ptr", "offset": 8 * i, "size": 8}
                         for i, n in enumerate(("rowOffsets", "columnIndices", "values", "rhs", "output"))]
    assert k["sparsewave"]["launch_n"] == "output_rows" and k["sparsewave"]["fixed_output_rows"] == 1000
    assert k["sparsewave"]["mapping"] == "wave-per-row-tile" and k["sparsewave"]["tile_size"] == 4


@pytest.mark.parametrize("kw,label", [(dict(block_size=128), "block size 64"), (dict(tile_size=8), "tile size 4"),
                                      (dict(wavefront_size=64), "wavefront size 32"),
                                      (dict(mapping="thread-per-output"), "mapping wave-per-row-tile")])
def test_unsupported_launch_contract_is_rejected(tmp_path, kw, label):
    with pytest.raises(bundle.BundleError, match=f"initial lrrt bundle support requires {label}"):
        bundle.write_bundle(tmp_path, rows=10, **kw)


def test_verify_rejects_mutations(built, tmp_path):
    src, _ = built
    def mutated(edit, blob_edit=None):
        d = tmp_path / f"m{len(list(tmp_path.iterdir()))}"
        d.mkdir()
        blob = (src / "kernels.cubin").read_bytes()
        (d / "kernels.cubin").write_bytes(blob_edit(blob) if blob_edit else blob)
        m = json.loads((src / "manifest.json").read_text())
        edit(m)
        (d / "manifest.json").write_text(json.dumps(m))
        return d
    bundle.verify_bundle(src)
    cases = [
        (lambda m: m.update(target="gfx1101"), None, "target"),
        (lambda m: m["kernels"][0].update(block=[128, 1, 1]), None, "block"),
        (lambda m: m["kernels"][0].update(grid=["ceil_div(n, 64) * 64", 1, 1]), None, "grid"),
        (lambda m: m["kernels"][0]["args"][3].update(offset=32), None, "arguments"),
        (lambda m: m["kernels"][0].update(workspace_bytes=16), None, "workspace"),
        (lambda m: m["kernels"][0]["sparsewave"].update(tile_size=8), None, "tile_size"),
        (lambda m: m["kernels"][0]["sparsewave"].update(fixed_output_rows=0), None, "fixed_output_rows"),
        (lambda m: None, lambda b: b + b"x", "digest"),
        (lambda m: m["kernels"][0].update(symbol="other_kernel"), None, "symbol"),
    ]
    for edit, blob_edit, word in cases:
        with pytest.raises(bundle.BundleError, match=word):
            bundle.verify_bundle(mutated(edit, blob_edit))


@pytest.mark.gpu
def test_bundle_runs_and_matches_the_oracle(built, ctx):
    d, _ = built
    rp, ci, v = random_csr(1000, 700, 20, seed=77)
    B = np.random.default_rng(77).uniform(-1, 1, (700, 4)).astype(np.float32)
    t = [torch.from_numpy(a).cuda() for a in (rp, ci, v, B)]
    out = torch.full((1000, 4), float("nan"), device="cuda")
    torch.cuda.synchronize()
    bundle.load_and_launch(d, 1000, [x.data_ptr() for x in t] + [out.data_ptr()])
    expected = oracle.csr_spmm(rp, ci, v, B)
    bound = oracle.csr_abs_bound(rp, ci, v, B)
    assert np.all(np.abs(out.cpu().numpy() - expected) <= 1e-5 * bound + 1e-30)
    # the library's bundle-style entry point gives the same result
    out2 = torch.empty_like(out)
    ctx.bundle_launch("spmm", 1000, t + [out2])
    assert float((out - out2).abs().max()) <= 1e-5 * float(bound.max())
