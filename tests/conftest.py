import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _has_cuda():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.fixture(scope="session")
def weight_dirs(tmp_path_factory):
    """name of a weight set in tests/golden/cases.py -> directory of .npy files (made on demand)."""
    import cases
    from cudabert_b200 import synth
    made = {}

    def get(name):
        if name not in made:
            d = tmp_path_factory.mktemp("w_" + name)
            synth.write_weight_dir(str(d), cases.get_weights(name))
            made[name] = str(d)
        return made[name]

    return get


@pytest.fixture(scope="session")
def models(weight_dirs):
    """(weight set, precision) -> Cuda_BERT replica on cuda:0, cached for the session."""
    import cases
    from cudabert_b200.config import Engin_Config
    from cudabert_b200.cuda_model import Cuda_BERT
    cache = {}

    def get(wname, precision):
        key = (wname, precision)
        if key not in cache:
            cfg = Engin_Config()
            cfg.is_large = cases.WEIGHT_SETS[wname][0]
            cfg.model_npy_pth = weight_dirs(wname)
            cfg.batch_size = 0
            cfg.max_seq_length = 0
            cfg.precision = precision
            cache[key] = Cuda_BERT(0, cfg)
        return cache[key]

    yield get
    for m in cache.values():
        m.close()
