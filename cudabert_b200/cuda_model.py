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

        if getattr(config, "weight_cache_pth", None):
            import os
            os.makedirs(config.weight_cache_pth, exist_ok=True)
            os.environ["CUDABERT_WEIGHT_CACHE"] = str(config.weight_cache_pth)   # read by the library at every load
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


class Cuda_BERT_Pool(object):
    """Several replicas inside ONE process, one host thread per replica (ctypes releases the GIL
    during a call): ``encode`` / ``classify`` cut the batch into contiguous row shards, run them
    concurrently and gather the rows on the host in the original order.  It is the in-process form
    of the engine's multi-GPU mode (reference: one OS process per GPU id, engine.py:385-397): batch
    sharding over independent replicas, no collective, nothing shared between GPUs.  ``gpus`` may
    name a GPU more than once (two replicas on one device share it through their own streams)."""

    def __init__(self, gpus, config):
        from concurrent.futures import ThreadPoolExecutor
        if not gpus:
            raise ValueError("Cuda_BERT_Pool needs at least one GPU id")
        self.replicas = [Cuda_BERT(g, config) for g in gpus]
        self.hidden_size = self.replicas[0].hidden_size
        self._threads = ThreadPoolExecutor(max_workers=len(self.replicas))

    def _shards(self, input_tensor):
        rows = np.asarray(input_tensor[0]).shape[0]
        n = min(len(self.replicas), rows)
        bounds = [rows * i // n for i in range(n + 1)]
        return [[None if t is None else np.asarray(t)[bounds[i]:bounds[i + 1]] for t in input_tensor]
                for i in range(n)]

    def _run(self, method, input_tensor):
        shards = self._shards(input_tensor)
        futures = [self._threads.submit(getattr(r, method), s) for r, s in zip(self.replicas, shards)]
        return np.concatenate([f.result() for f in futures], axis=0)

    def encode(self, input_tensor):
        return self._run("encode", input_tensor)

    def classify(self, input_tensor):
        return self._run("classify", input_tensor)

    def close(self):
        for r in self.replicas:
            r.close()
        self._threads.shutdown(wait=True)
