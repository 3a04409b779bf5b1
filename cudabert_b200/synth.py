"""Seeded synthetic weights and inputs in the reference's on-disk and call formats.

No pretrained checkpoint or dataset ships with the reference (its README run used an
unshipped 100k-line TSV and a fine-tuned checkpoint), so tests and the benchmark use
seeded random tensors with the documented shapes and value distributions:

* weights follow ``init_bert_weights`` of the reference's bundled model
  (apps/pytorch_pretrained_bert/modeling.py:437-448): every Linear/Embedding matrix
  ~ N(0, 0.02), LayerNorm gamma = 1, beta = 0, Linear bias = 0.  ``affine=True``
  additionally randomises biases/gamma/beta so that bias and beta bugs cannot hide
  behind zeros.
* the weight directory layout is the one ``convert_pytorch_model_to_npys.py:27-66``
  writes and ``cuda_bert/utils/load_model.cc:15-37`` / ``utils/bert.cu:17-69`` read: one
  float32 C-order ``.npy`` per tensor, dense kernels stored ``[in, out]``.
* inputs follow the call contract of ``Cuda_Bert`` (cuda_bert/cuda_bert.cu:55-70):
  int32 ``ids``, ``seg``, ``mask`` of shape ``[B, S]``.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import numpy as np

VOCAB_SIZE = 30522
MAX_POSITIONS = 512
TYPE_VOCAB = 2
HEAD_DIM = 64
CLS_ID = 101


def model_dims(is_large: bool) -> Dict[str, int]:
    """Hard-coded dims, as in cuda_bert/utils/manager.cu:8-15."""
    if is_large:
        return dict(layers=24, hidden=1024, heads=16, ffn=4096)
    return dict(layers=12, hidden=768, heads=12, ffn=3072)


def make_weights(is_large: bool, seed: int, affine: bool = False,
                 num_layers: Optional[int] = None, num_classes: int = 2) -> Dict[str, np.ndarray]:
    """Return {file stem -> float32 array} for a whole encoder + pooler + classifier head."""
    d = model_dims(is_large)
    L = d["layers"] if num_layers is None else num_layers
    H, F = d["hidden"], d["ffn"]
    rng = np.random.default_rng(seed)

    def mat(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))

    def bias(n):
        return mat(n) if affine else np.zeros(n, np.float32)

    def gamma(n):
        return (1.0 + mat(n)).astype(np.float32) if affine else np.ones(n, np.float32)

    w: Dict[str, np.ndarray] = {}
    w["bert_embeddings_word_embeddings"] = mat(VOCAB_SIZE, H)
    w["bert_embeddings_position_embeddings"] = mat(MAX_POSITIONS, H)
    w["bert_embeddings_token_type_embeddings"] = mat(TYPE_VOCAB, H)
    w["bert_embeddings_LayerNorm_gamma"] = gamma(H)
    w["bert_embeddings_LayerNorm_beta"] = bias(H)
    for i in range(L):
        p = "bert_encoder_layer_%d_" % i
        for nm in ("query", "key", "value"):
            w[p + "attention_self_%s_kernel" % nm] = mat(H, H)
            w[p + "attention_self_%s_bias" % nm] = bias(H)
        w[p + "attention_output_dense_kernel"] = mat(H, H)
        w[p + "attention_output_dense_bias"] = bias(H)
        w[p + "attention_output_LayerNorm_gamma"] = gamma(H)
        w[p + "attention_output_LayerNorm_beta"] = bias(H)
        w[p + "intermediate_dense_kernel"] = mat(H, F)
        w[p + "intermediate_dense_bias"] = bias(F)
        w[p + "output_dense_kernel"] = mat(F, H)
        w[p + "output_dense_bias"] = bias(H)
        w[p + "output_LayerNorm_gamma"] = gamma(H)
        w[p + "output_LayerNorm_beta"] = bias(H)
    w["bert_pooler_dense_kernel"] = mat(H, H)
    w["bert_pooler_dense_bias"] = bias(H)
    # fine-tune head of the sample app (apps/finetune.py:16-44): Linear(H -> C) + Softmax
    w["classifier_kernel"] = mat(H, num_classes)
    w["classifier_bias"] = bias(num_classes)
    return w


def write_weight_dir(path: str, weights: Dict[str, np.ndarray]) -> str:
    os.makedirs(path, exist_ok=True)
    for name, arr in weights.items():
        np.save(os.path.join(path, name + ".npy"), np.ascontiguousarray(arr, dtype=np.float32))
    return path


def make_lengths(rng: np.random.Generator, batch: int, seq: int, dist: str) -> np.ndarray:
    """Valid lengths per row.

    ``full``            every position valid
    ``uniform:a:b``     integer uniform in [a, b]
    ``tnormal:m:s:a:b`` round(N(m, s)) resampled until inside [a, b] (truncated normal)
    """
    parts = dist.split(":")
    if parts[0] == "full":
        return np.full(batch, seq, np.int64)
    if parts[0] == "uniform":
        a, b = int(parts[1]), min(int(parts[2]), seq)
        return rng.integers(a, b + 1, size=batch)
    if parts[0] == "tnormal":
        m, s, a, b = float(parts[1]), float(parts[2]), int(parts[3]), min(int(parts[4]), seq)
        out = np.rint(rng.normal(m, s, size=batch)).astype(np.int64)
        bad = (out < a) | (out > b)
        while bad.any():
            out[bad] = np.rint(rng.normal(m, s, size=int(bad.sum()))).astype(np.int64)
            bad = (out < a) | (out > b)
        return out
    raise ValueError("unknown length distribution %r" % dist)


def make_inputs(seed: int, batch: int, seq: int, dist: str = "full"
                ) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """ids uniform in [1000, vocab) with [CLS] at position 0; seg 0 for the first half of
    the row and 1 after; mask 1 up to the row's valid length (ids under padding stay
    random: they are masked)."""
    rng = np.random.default_rng(seed)
    ids = rng.integers(1000, VOCAB_SIZE, size=(batch, seq)).astype(np.int32)
    ids[:, 0] = CLS_ID
    seg = np.zeros((batch, seq), np.int32)
    seg[:, seq // 2:] = 1
    lens = make_lengths(rng, batch, seq, dist)
    mask = (np.arange(seq)[None, :] < lens[:, None]).astype(np.int32)
    return ids, seg, mask


# The five workloads of the benchmark specification (model size, precision, shape, lengths).
CONFIGS = {
    0: dict(large=False, precision="fp32", batch=8, seq=128, dist="uniform:32:128", lines=8),
    1: dict(large=True, precision="bf16", batch=128, seq=200, dist="uniform:16:200", lines=100000),
    2: dict(large=False, precision="bf16", batch=256, seq=128, dist="tnormal:60:25:8:128", lines=1000000),
    3: dict(large=True, precision="bf16", batch=32, seq=512, dist="full", lines=32),
    4: dict(large=True, precision="fp8", batch=1024, seq=64, dist="uniform:8:64", lines=1024),
}


def weight_seed(cfg: int) -> int:
    return 1000 + cfg


def input_seed(cfg: int) -> int:
    return 2000 + cfg
