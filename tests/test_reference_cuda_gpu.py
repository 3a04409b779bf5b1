"""Second checker on the GPU box: the reference's own CUDA library (fp32, cuBLAS), built from the
reference tree by oracle/build_ref.py into oracle/_ref/ and run in a subprocess.  Skipped when that
build is not present."""
import os
import subprocess
import sys

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libcudaBERT_ref.so")


def _run_reference(weight_dir, large, ids, seg, mask, tmp_path):
    inp, out = str(tmp_path / "in.npz"), str(tmp_path / "out.npy")
    arrays = dict(ids=ids, seg=seg)
    if mask is not None:
        arrays["mask"] = mask
    np.savez(inp, **arrays)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "run_ref_cuda.py"), weight_dir, str(int(large)),
                        inp, out], capture_output=True, text=True, timeout=300)
    if r.returncode != 0:
        pytest.fail("reference CUDA library failed: rc=%d\n%s\n%s" % (r.returncode, r.stdout[-1500:], r.stderr[-1500:]))
    return np.load(out)


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="oracle/_ref is not built")
@pytest.mark.parametrize("name", ["c0", "c0_affine", "edge_holes", "edge_s17"])
def test_fp32_mode_matches_reference_cuda_library(models, weight_dirs, tmp_path, name):
    wname = cases.CASES[name]["weights"]
    large = cases.WEIGHT_SETS[wname][0]
    ids, seg, mask = cases.case_inputs(name)
    ref = _run_reference(weight_dirs(wname), large, ids, seg, mask, tmp_path)
    gold = cases.load_golden(name)["pooled"]
    ours = models(wname, "fp32").encode([ids, seg, mask])
    # the two reference implementations (bundled PyTorch model on CPU, CUDA library on this GPU)
    # agree with each other, and the fp32 mode agrees with both, within the fp32 tolerance
    assert np.abs(ref - gold).max() <= 1e-3
    assert np.abs(ours - ref).max() <= 1e-3
