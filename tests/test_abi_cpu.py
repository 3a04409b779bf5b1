"""Host-side checks that need no GPU: the library loads, exports every symbol the public header
declares, fails cleanly without a device, and the oracle's FP8 helper behaves."""
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def pybert():
    from cudabert_b200 import build
    build.build()
    from cudabert_b200.cuda_bert import pybert as pb
    return pb


def test_library_exports_every_declared_symbol(pybert):
    with open(os.path.join(ROOT, "include", "cudabert.h")) as f:
        text = f.read()
    names = [n for n in re.findall(r"CUDABERT_API\s+[^;(]*?([A-Za-z_][A-Za-z_0-9]*)\s*\(", text)
             if n != "__attribute__"]
    assert len(names) >= 25
    for ref_name in ("init_model", "release_model", "Cuda_Inference", "Cuda_Bert", "test"):
        assert ref_name in names
    missing = [n for n in names if not hasattr(pybert.lib, n)]
    assert not missing, missing


def test_reference_binding_surface(pybert):
    """Names the reference's pybert.py exposes (cuda_bert/pybert.py:12-38)."""
    for n in ("lib", "Retval", "init_model", "release_model", "load_model", "unload_model", "inference", "bert"):
        assert hasattr(pybert, n)
    assert [f[0] for f in pybert.Retval._fields_] == ["tensor", "Pooled_Output"]
    assert pybert.filling_inputs([1, 2, 3, 9], 7) == [1, 2, 3, 1, 2, 3, 9]


def test_no_device_is_an_error_not_a_crash(pybert):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError) as e:
        pybert.load_model(False, "/nonexistent")
    assert "init_model failed" in str(e.value)
    assert pybert.status(None) != 0


def test_config_and_wrapper_surface():
    from cudabert_b200.config import Engin_Config
    c = Engin_Config()
    # defaults of the reference (config.py:3-39)
    assert (c.gpu, c.is_large, c.max_seq_length, c.batch_size) == ([0], True, 200, 128)
    assert (c.start_split, c.end_split, c.split_size, c.queue_size, c.alert_size) == (50, 180, 2, 100, 1000000)
    assert c.hiddensize == 1024
    c.is_large = False
    assert c.hiddensize == 768
    assert c.cubert_pth.endswith("cuda_bert") and os.path.isdir(c.cubert_pth)


def test_fp8_roundtrip_properties():
    from oracle import bert_oracle
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((64, 96)) * 0.02).astype(np.float32)
    q = bert_oracle.fp8_e4m3_roundtrip(w)
    assert q.shape == w.shape and q.dtype == np.float32
    i = np.unravel_index(np.abs(w).argmax(), w.shape)
    assert abs(q[i] - w[i]) <= 1e-7          # the largest magnitude maps to +-448 exactly
    big = np.abs(w) > np.abs(w).max() * 2.0 ** -6   # normal range of e4m3 under this scale
    assert (np.abs(q - w)[big] <= np.abs(w)[big] * 2.0 ** -4 * 1.001).all()
    assert np.array_equal(bert_oracle.fp8_e4m3_roundtrip(q), q)   # idempotent
    t = {"bert_encoder_layer_0_output_dense_kernel": w, "bert_pooler_dense_kernel": w, "x_bias": w[0]}
    out = bert_oracle.quantize_encoder_weights_fp8(t)
    assert np.array_equal(out["bert_pooler_dense_kernel"], w) and not np.array_equal(
        out["bert_encoder_layer_0_output_dense_kernel"], w)


def test_reference_application_import_lines():
    """The import block of the reference's sample application (apps/example.py:6-10) works unchanged
    and names the same module objects as the package's own import root."""
    import subprocess
    import sys
    code = (
        "from cuda_bert.engine import Engine\n"
        "from cuda_bert.config import Engin_Config\n"
        "from cuda_bert.cuda_model import Cuda_BERT\n"
        "import cudabert_b200.engine, cudabert_b200.config, cudabert_b200.cuda_model\n"
        "assert Engine is cudabert_b200.engine.Engine\n"
        "assert Engin_Config is cudabert_b200.config.Engin_Config\n"
        "assert Cuda_BERT is cudabert_b200.cuda_model.Cuda_BERT\n"
        "from cuda_bert.cuda_bert import pybert\n"
        "import cudabert_b200.cuda_bert.pybert as packaged\n"
        "assert pybert is packaged\n"
        "e = Engine(Engin_Config())\n"
        "for n in ('set_cuda_model', 'set_finetune_layer', 'set_tokenlizer_function', 'set_output_function', 'run'):\n"
        "    assert callable(getattr(e, n))\n"
        "print('ok')\n")
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stderr
