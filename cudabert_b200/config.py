"""Engine configuration.  ``Engin_Config`` offers the attribute names callers of the reference set
(config.py:3-39) so that their scripts run unchanged; defaults and their meaning are listed in
``_DEFAULTS`` below.  Additions: ``precision``, ``weight_cache_pth``, ``native_batcher``, ``native_reader``, ``reader_threads``, ``replica_mode``,
``resume_without_dead_gpu`` and ``mp_start_method``."""
import os

_PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))

# name -> (default, meaning)
_DEFAULTS = {
    "gpu": ([0], "CUDA device ids; one independent replica (and worker process) per id"),
    "is_large": (True, "BERT-large (24 x 1024, 16 heads) instead of BERT-base (12 x 768, 12 heads)"),
    "max_seq_length": (200, "tokenizer output length: longer inputs are truncated, shorter ones padded"),
    "batch_size": (128, "lines per batch and bucket"),
    "queue_size": (100, "kept for callers that set it; the queues between the stages are bounded internally"),
    "alert_size": (1000000, "lines the writer may hold back before it asks the reader to flush its buckets"),
    "start_split": (50, "first inner boundary of the length buckets"),
    "end_split": (180, "last inner boundary of the length buckets"),
    "split_size": (2, "distance between inner bucket boundaries"),
    "skip_first_line": (False, "drop a header line of the input file"),
    "model_npy_pth": ("./model_npy", "directory of .npy weights: the encoder, the pooler, the fine-tune head"),
    "cubert_pth": (os.path.join(_PACKAGE_DIR, "cuda_bert"), "directory that holds pybert.py and libcudaBERT.so"),
    "precision": (None, '"fp32", "bf16" or "fp8"; None = environment CUDABERT_PRECISION, else bf16'),
    "weight_cache_pth": (None, "directory for device-ready copies of the weights (one file per model directory and mode), "
                               "written at the first load and read by later ones; None = environment CUDABERT_WEIGHT_CACHE, else no cache"),
    "native_batcher": (True, "bucket and trim in the library's batcher; False = the Python classes"),
    "native_reader": (True, "with a tokenizer.Tokenlizer as tokenizer function: read, tokenise and bucket in native threads"),
    "reader_threads": (0, "tokenizer threads of the native reader; 0 = up to 16, one core left free"),
    "replica_mode": ("auto", '"process": one OS process per replica (the reference\'s way); "thread": one thread per replica '
                             'inside this process (needs a tokenizer.Tokenlizer); "auto": threads for more than two GPUs when possible'),
    "resume_without_dead_gpu": (True, "if a replica's process dies, resume after the last written line on the rest"),
    "mp_start_method": (None, 'multiprocessing start method; use "spawn" when the parent already holds a CUDA context'),
}


class Engin_Config(object):
    def __init__(self):
        for name, (default, _) in _DEFAULTS.items():
            setattr(self, name, list(default) if isinstance(default, list) else default)

    @property
    def hiddensize(self):
        """Width of the pooler output.  The reference computes it once in its constructor, so it goes
        stale when ``is_large`` is changed afterwards; here it always follows ``is_large``."""
        return 1024 if self.is_large else 768

    @staticmethod
    def describe():
        """One line per setting: name, default, meaning."""
        return "\n".join("%-24s %-14r %s" % (k, v[0], v[1]) for k, v in _DEFAULTS.items())
