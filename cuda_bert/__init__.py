"""Import root of the reference's application code.

The reference's repository root is itself the package ``cuda_bert``: its sample application does
``from cuda_bert.engine import Engine``, ``from cuda_bert.config import Engin_Config`` and
``from cuda_bert.cuda_model import Cuda_BERT`` (apps/example.py:6-10), and the binding lives in
the inner directory ``cuda_bert/cuda_bert/pybert.py`` (config.py:36-37).  This package keeps
those import lines working unchanged: every ``cuda_bert.<name>`` resolves to the module object
``cudabert_b200.<name>`` (one copy of each module, whichever name imported it first).
"""
import importlib
import importlib.abc
import importlib.util
import sys

_IMPL = "cudabert_b200"


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """``cuda_bert.a.b`` -> the module ``cudabert_b200.a.b``."""

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(__name__ + "."):
            return None
        real = _IMPL + fullname[len(__name__):]
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        return importlib.util.spec_from_loader(fullname, self, origin=real)

    def create_module(self, spec):
        return importlib.import_module(spec.origin)

    def exec_module(self, module):
        pass  # already executed under its own name


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
