"""``Cuda_BERT``: one encoder replica on one GPU behind the reference's wrapper API
(cuda_model.py:4-41): ``Cuda_BERT(id_gpu, config).encode([ids, seg, mask]) -> float32[B, H]``."""
import importlib
import sys

import numpy as np


def _load_pybert(cubert_pth):
    """The reference puts ``config.cubert_pth`` on sys.path and imports ``pybert``
    (cuda_model.py:10-11); the packaged module is used when that directory is this package's."""
    try:
        from .cuda_bert import pybert
        import os
        if cubert_pth is None or os.path.abspath(cubert_pth) == os.path.abspath(os.path.dirname(pybert.__file__)):
            return pybert
    except ImportError:
        if cubert_pth is None:
            raise
    sys.path.insert(0, cubert_pth)
    return importlib.import_module("pybert")


class Cuda_BERT(object):
    def __init__(self, id_gpu, config):
        self.id_gpu = id_gpu
        self.max_batchsize = config.batch_size
        self.max_seq_length = config.max_seq_length
        self._pybert = _load_pybert(getattr(config, "cubert_pth", None))

        if config.is_large:
            self.hidden_size = 1024
        else:
            self.hidden_size = 768

        self.model = self._pybert.load_model(config.is_large, config.model_npy_pth, id_gpu,
                                             config.batch_size, config.max_seq_length,
                                             precision=getattr(config, "precision", None))
        self.cu_encode = self._pybert.bert

    @staticmethod
    def _i32(a):
        return np.ascontiguousarray(a, dtype=np.int32)

    def encode(self, input_tensor):
        '''
        Input_tensor:
            inputs_id, segments_id, mask:
            numpy.array [batchsize, seq_length]   (mask may be None: every position valid)
        '''
        indexed_tokens = self._i32(input_tensor[0])
        segments_ids = self._i32(input_tensor[1])
        attention_mask = None if input_tensor[2] is None else self._i32(input_tensor[2])
        batchsize = indexed_tokens.shape[0]
        seq_length = indexed_tokens.shape[1]
        output = np.ones([batchsize, self.hidden_size]).astype(np.float32)
        self.cu_encode(self.model, output, indexed_tokens, segments_ids,
                       batchsize, seq_length, attention_mask)
        self._pybert.check(self.model)
        return output

    def classify(self, input_tensor):
        """Pooler + Linear(H -> C) + Softmax on the device (needs classifier_kernel/bias.npy)."""
        indexed_tokens = self._i32(input_tensor[0])
        segments_ids = self._i32(input_tensor[1])
        attention_mask = None if input_tensor[2] is None else self._i32(input_tensor[2])
        batchsize, seq_length = indexed_tokens.shape
        c = self._pybert.num_classes(self.model)
        output = np.zeros([batchsize, c], np.float32)
        self._pybert.classify(self.model, output, indexed_tokens, segments_ids, batchsize, seq_length, c,
                              attention_mask)
        self._pybert.check(self.model)
        return output

    def close(self):
        if getattr(self, "model", None):
            self._pybert.unload_model(self.model)
            self.model = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
