"""ctypes binding of libcudaBERT.so.

Same public names and call signatures as the reference's binding (cuda_bert/pybert.py:12-38):
``lib``, ``Retval``, ``init_model``, ``release_model``, ``load_model``, ``unload_model``,
``inference``, ``bert``, plus ``classify`` (commented out in the reference, pybert.py:40-42).
Differences, on purpose:

* no tokenizer is imported or downloaded at import time (reference: pybert.py:2,68);
* ``Retval`` holds two device pointers as ``c_void_p`` (the reference declares them as numpy
  ndpointers of the removed ``numpy.float``, pybert.py:6-8, which cannot work with numpy >= 1.24);
* a missing library raises ``ImportError`` with the build command; there is no CPU fallback;
* failures never kill the process: ``load_model`` raises ``RuntimeError`` with the library's
  message, ``status`` / ``last_error`` report per-handle errors, ``check`` raises on them.
"""
from ctypes import (CDLL, RTLD_GLOBAL, POINTER, Structure, byref, c_bool, c_char_p, c_double, c_float, c_int,
                    c_long, c_size_t, c_void_p)
import os

import numpy
from numpy.ctypeslib import ndpointer


class Retval(Structure):
    _fields_ = [("tensor", c_void_p),
                ("Pooled_Output", c_void_p)]


lib_dir = os.path.abspath(os.path.dirname(__file__))
_lib_path = os.path.join(lib_dir, "libcudaBERT.so")
if not os.path.exists(_lib_path):
    raise ImportError("%s is missing: build it with `python -m cudabert_b200.build` "
                      "(nvcc, sm_100a); there is no fallback path" % _lib_path)
lib = CDLL(_lib_path, RTLD_GLOBAL)

_i32 = ndpointer(numpy.int32, flags="C_CONTIGUOUS")
_f32 = ndpointer(numpy.float32, flags="C_CONTIGUOUS")


class _OptionalI32:
    """int32 ndarray or None (-> NULL): the mask argument may be omitted."""

    @classmethod
    def from_param(cls, obj):
        if obj is None:
            return None
        return _i32.from_param(obj)


init_model = lib.init_model
init_model.argtypes = [c_bool, c_int, c_int, c_int, c_char_p]
init_model.restype = c_void_p

release_model = lib.release_model
release_model.argtypes = [c_void_p]
release_model.restype = None

init_ex = lib.cudabert_init_ex
init_ex.argtypes = [c_bool, c_int, c_int, c_int, c_char_p, c_int, c_int]
init_ex.restype = c_void_p

status = lib.cudabert_status
status.argtypes = [c_void_p]
status.restype = c_int

_last_error = lib.cudabert_last_error
_last_error.argtypes = [c_void_p]
_last_error.restype = c_char_p

PRECISIONS = {"fp32": 0, "bf16": 1, "fp8": 2}


def last_error(model=None):
    msg = _last_error(model)
    return msg.decode("utf-8", "replace") if msg else ""


def check(model):
    """Raise RuntimeError if the last call on this handle failed."""
    if status(model) != 0:
        raise RuntimeError("cudaBERT: " + last_error(model))


def load_model(is_large_model, model_dir, num_gpu=0, max_batchsize=0, max_seq_length=0,
               precision=None, num_layers=0):
    '''
        max_batchsize and max_seq_length pre-size the activation memory;
        larger batches grow it on demand.
        precision: None (environment CUDABERT_PRECISION, default bf16), "fp32", "bf16" or "fp8".
    '''
    prec = -1 if precision is None else PRECISIONS[precision]
    model = init_ex(is_large_model, num_gpu, max_batchsize, max_seq_length,
                    bytes(model_dir, encoding='utf-8'), prec, num_layers)
    if not model:
        raise RuntimeError("cudaBERT: init_model failed: " + last_error(None))
    return model


def unload_model(model):
    release_model(model)


inference = lib.Cuda_Inference
inference.argtypes = [c_void_p, _i32, _i32, c_int, c_int, _OptionalI32]
inference.restype = Retval

bert = lib.Cuda_Bert
bert.argtypes = [c_void_p, _f32, _i32, _i32, c_int, c_int, _OptionalI32]
bert.restype = None

classify = lib.Cuda_Classify
classify.argtypes = [c_void_p, _f32, _i32, _i32, c_int, c_int, c_int, _OptionalI32]
classify.restype = None

# length-bucketing batcher of the engine's reader stage (host only)
from ctypes import c_longlong as _c_ll
batcher_create = lib.cudabert_batcher_create
batcher_create.argtypes = [_i32, c_int, c_int, c_int]
batcher_create.restype = c_void_p
batcher_destroy = lib.cudabert_batcher_destroy
batcher_destroy.argtypes = [c_void_p]
batcher_destroy.restype = None
batcher_put = lib.cudabert_batcher_put
batcher_put.argtypes = [c_void_p, _c_ll, _i32, _i32, _i32, c_int]
batcher_put.restype = c_int
batcher_flush = lib.cudabert_batcher_flush
batcher_flush.argtypes = [c_void_p]
batcher_flush.restype = c_int
batcher_ready = lib.cudabert_batcher_ready
batcher_ready.argtypes = [c_void_p]
batcher_ready.restype = c_int
batcher_pending = lib.cudabert_batcher_pending
batcher_pending.argtypes = [c_void_p]
batcher_pending.restype = _c_ll
batcher_next = lib.cudabert_batcher_next
batcher_next.argtypes = [c_void_p, POINTER(c_int), POINTER(c_int), POINTER(_c_ll)]
batcher_next.restype = c_int
batcher_pop = lib.cudabert_batcher_pop
batcher_pop.argtypes = [c_void_p, ndpointer(numpy.int64, flags="C_CONTIGUOUS"), _i32, _i32, _i32]
batcher_pop.restype = c_int

# BERT tokenizer of the engine's reader stage (host only)
tokenizer_create = lib.cudabert_tokenizer_create
tokenizer_create.argtypes = [c_char_p, c_int]
tokenizer_create.restype = c_void_p
tokenizer_destroy = lib.cudabert_tokenizer_destroy
tokenizer_destroy.argtypes = [c_void_p]
tokenizer_destroy.restype = None
tokenizer_vocab_size = lib.cudabert_tokenizer_vocab_size
tokenizer_vocab_size.argtypes = [c_void_p]
tokenizer_vocab_size.restype = c_int
tokenizer_tokenize = lib.cudabert_tokenizer_tokenize
tokenizer_tokenize.argtypes = [c_void_p, c_char_p, _i32, c_int]
tokenizer_tokenize.restype = c_int
tokenizer_encode_pair = lib.cudabert_tokenizer_encode_pair
tokenizer_encode_pair.argtypes = [c_void_p, c_char_p, c_char_p, c_int, _i32, _i32, _i32]
tokenizer_encode_pair.restype = c_int

# native reader stage: file -> tokenizer threads -> batcher
_i64 = ndpointer(numpy.int64, flags="C_CONTIGUOUS")
reader_create = lib.cudabert_reader_create
reader_create.argtypes = [c_char_p, c_void_p, c_int, _i32, c_int, c_int, c_int, _c_ll, _c_ll]
reader_create.restype = c_void_p
reader_destroy = lib.cudabert_reader_destroy
reader_destroy.argtypes = [c_void_p]
reader_destroy.restype = None
reader_next = lib.cudabert_reader_next
reader_next.argtypes = [c_void_p, POINTER(c_int), POINTER(c_int), POINTER(_c_ll)]
reader_next.restype = c_int
reader_pop = lib.cudabert_reader_pop
reader_pop.argtypes = [c_void_p, _i64, _i32, _i32, _i32, _i64]
reader_pop.restype = c_int
reader_raw = lib.cudabert_reader_raw
reader_raw.argtypes = [c_void_p, c_char_p, _c_ll]
reader_raw.restype = _c_ll
reader_flush = lib.cudabert_reader_flush
reader_flush.argtypes = [c_void_p]
reader_flush.restype = c_int
reader_rejected = lib.cudabert_reader_rejected
reader_rejected.argtypes = [c_void_p, POINTER(_c_ll)]
reader_rejected.restype = _c_ll
reader_lines = lib.cudabert_reader_lines
reader_lines.argtypes = [c_void_p]
reader_lines.restype = _c_ll

attention_kernel_for = lib.cudabert_attention_kernel_for
attention_kernel_for.argtypes = [c_int]
attention_kernel_for.restype = c_int


def attention_kernel_name(seq_length):
    """Name of the attention kernel a 16-bit forward pass of this padded length runs."""
    return {1: "attention_f16_kernel", 2: "attention_tc_kernel",
            3: "attention_f16_persist_kernel"}.get(attention_kernel_for(int(seq_length)), "unknown")


hidden_size = lib.cudabert_hidden_size
hidden_size.argtypes = [c_void_p]
hidden_size.restype = c_int

num_classes = lib.cudabert_num_classes
num_classes.argtypes = [c_void_p]
num_classes.restype = c_int

forward_dev = lib.cudabert_forward_dev
forward_dev.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int]
forward_dev.restype = c_int

classify_dev = lib.cudabert_classify_dev
classify_dev.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int]
classify_dev.restype = c_int

probs_dev = lib.cudabert_probs_dev
probs_dev.argtypes = [c_void_p]
probs_dev.restype = c_void_p

sync = lib.cudabert_sync
sync.argtypes = [c_void_p]
sync.restype = c_int

# test hook: makes one bounded device-side wait run out (limit in microseconds) and returns the status
test_wait_timeout = lib.cudabert_test_wait_timeout
test_wait_timeout.argtypes = [c_void_p, c_int]
test_wait_timeout.restype = c_int

pooled_dev = lib.cudabert_pooled_dev
pooled_dev.argtypes = [c_void_p]
pooled_dev.restype = c_void_p

copy_to_host = lib.cudabert_copy_to_host
copy_to_host.argtypes = [c_void_p, c_void_p, c_size_t]
copy_to_host.restype = c_int

stream = lib.cudabert_stream
stream.argtypes = [c_void_p]
stream.restype = c_void_p

launch_count = lib.cudabert_launch_count
launch_count.argtypes = [c_void_p]
launch_count.restype = c_long
graph_captures = lib.cudabert_graph_captures
graph_captures.argtypes = [c_void_p]
graph_captures.restype = c_long
graph_replays = lib.cudabert_graph_replays
graph_replays.argtypes = [c_void_p]
graph_replays.restype = c_long

profile_enable = lib.cudabert_profile_enable
profile_enable.argtypes = [c_void_p, c_int]
profile_enable.restype = None
profile_reset = lib.cudabert_profile_reset
profile_reset.argtypes = [c_void_p]
profile_reset.restype = None
_profile_get = lib.cudabert_profile_get
_profile_get.argtypes = [c_void_p, c_int, POINTER(c_double), POINTER(c_long)]
_profile_get.restype = c_int

KERNEL_CLASSES = ["embed_layernorm", "gemm_qkv", "attention", "gemm_attn_out", "layernorm", "gemm_ffn1",
                  "gemm_ffn2", "gemm_pooler", "other"]


def profile_get(model):
    """{kernel class: (total device ms, launches)} accumulated since profile_reset."""
    out = {}
    for i, name in enumerate(KERNEL_CLASSES):
        ms, n = c_double(0), c_long(0)
        _profile_get(model, i, byref(ms), byref(n))
        out[name] = (ms.value, n.value)
    return out


# single kernels on device pointers (integers), used by the per-kernel parity tests
k_gemm_tcgen05 = lib.cudabert_k_gemm_tcgen05
k_gemm_tcgen05.argtypes = [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                        c_void_p, c_void_p]
k_gemm_tcgen05.restype = c_int
k_gemm_f32 = lib.cudabert_k_gemm_f32
k_gemm_f32.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p]
k_gemm_f32.restype = c_int
k_gemm_f32_tensor = lib.cudabert_k_gemm_f32_tensor
k_gemm_f32_tensor.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p]
k_gemm_f32_tensor.restype = c_int
k_gemm_ln_folded = lib.cudabert_k_gemm_ln_folded
k_gemm_ln_folded.argtypes = [c_void_p] * 8 + [c_int] * 5 + [c_void_p, c_void_p]
k_gemm_ln_folded.restype = c_int
k_attention = lib.cudabert_k_attention
k_attention.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]
k_attention.restype = c_int
k_attention_noalloc = lib.cudabert_k_attention_noalloc
k_attention_noalloc.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]
k_attention_noalloc.restype = c_int
NOALLOC_MAX_BATCH = 4096
k_embed_layernorm = lib.cudabert_k_embed_layernorm
k_embed_layernorm.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_int, c_int, c_int, c_int]
k_embed_layernorm.restype = c_int
k_layernorm = lib.cudabert_k_layernorm
k_layernorm.argtypes = [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int]
k_layernorm.restype = c_int


def filling_inputs(words, seq_length):
    """Tile a short seed list up to seq_length keeping its last element last (reference:
    pybert.py:44-53)."""
    length = (len(words) - 1)
    total = length - 1
    end_word = words[-1]
    words = list(words[:-1])
    while total < seq_length - 2:
        total = total + 1
        words.append(words[total % length])
    words.append(end_word)
    return words


def batch_inputs(input, batchsize):
    return [input for _ in range(batchsize)]


def warp_inputs(indexed_tokens, segments_ids, attention_masks):
    c_index = numpy.array(indexed_tokens).astype(numpy.int32)
    c_seg = numpy.array(segments_ids).astype(numpy.int32)
    c_mask = numpy.array(attention_masks).astype(numpy.int32)
    return c_index, c_seg, c_mask


def test(is_large, model_dir, batchsize, seq_length, num_gpu=0, iters=100):
    """Timing loop of the reference's pybert.test (pybert.py:70-98) on its 11-token seed; the
    token ids are the ones its C test uses (cuda_bert/cuda_bert.cu:94-96), so no tokenizer or
    vocabulary download is needed."""
    import time
    indexed = [2040, 2001, 3958, 27227, 1029, 3958, 103, 2001, 1037, 13997, 11510]
    segments_ids = [0, 0, 0, 0, 0, 1, 1, 1, 1, 1, 1]
    attention_mask = [1, 1, 1, 1, 1, 1, 1, 1, 0, 0, 0]
    ids, seg, mask = warp_inputs(batch_inputs(filling_inputs(indexed, seq_length), batchsize),
                                 batch_inputs(filling_inputs(segments_ids, seq_length), batchsize),
                                 batch_inputs(filling_inputs(attention_mask, seq_length), batchsize))
    model = load_model(is_large, model_dir, num_gpu=num_gpu)
    start = time.time()
    for _ in range(iters):
        inference(model, ids, seg, batchsize, seq_length, mask)
    end = time.time()
    check(model)
    print("Batchsize: {} Seq_length: {} Use_Time: {}".format(batchsize, seq_length, (end - start) / iters))
    unload_model(model)
