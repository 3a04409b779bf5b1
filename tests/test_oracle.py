"""The CPU restatement in oracle/ against the golden outputs of the real reference model."""
import numpy as np
import pytest
import torch

import cases
from oracle import bert_oracle

FP32_TOL = 2e-5      # two fp32 evaluations of the same network in a different op order
FP64_TOL = 1e-9      # fp64 restatement vs fp64 run of the reference module


@pytest.mark.parametrize("name", list(cases.CASES.keys()))
def test_oracle_matches_reference_outputs(name):
    large, dims = cases.case_dims(name)
    w = cases.get_weights(cases.CASES[name]["weights"])
    ids, seg, mask = cases.case_inputs(name)
    gold = cases.load_golden(name)
    layers, pooled = bert_oracle.bert_forward(w, ids, seg, mask, dims["heads"], dims["layers"],
                                              return_all=True)
    tol = FP32_TOL if name != "edge_zero_row" else 2e-4   # -10000 + score rounds at 1e-3 in fp32
    assert np.abs(pooled - gold["pooled"]).max() <= tol
    assert np.abs(layers[0][:, :, :8] - gold["embed8"]).max() <= tol
    assert np.abs(layers[1][:, :, :8] - gold["layer0_8"]).max() <= tol
    assert np.abs(layers[-1][:, :, :8] - gold["last8"]).max() <= 10 * tol
    assert np.abs(layers[-1][:, 0, :] - gold["cls_hidden"]).max() <= 10 * tol
    probs = bert_oracle.classify(bert_oracle.Weights(w), torch.from_numpy(pooled)).numpy()
    assert np.abs(probs - gold["probs"]).max() <= tol


@pytest.mark.parametrize("name", ["c0", "edge_zero_row", "edge_holes"])
def test_oracle_fp64_matches_reference_fp64(name):
    large, dims = cases.case_dims(name)
    w = cases.get_weights(cases.CASES[name]["weights"])
    ids, seg, mask = cases.case_inputs(name)
    gold = cases.load_golden(name)
    _, pooled = bert_oracle.bert_forward(w, ids, seg, mask, dims["heads"], dims["layers"],
                                         dtype=torch.float64)
    assert np.abs(pooled - gold["pooled64"]).max() <= FP64_TOL


def test_fp16_activation_range_and_bf16_weight_set():
    """The 16-bit modes keep activations in fp16 between kernels (largest finite value 65504; the
    kernels saturate instead of overflowing).  On the synthetic workloads every such tensor stays
    below 100, three orders of magnitude inside the range.  And the bf16 weight set really is
    bf16: every rounded dense weight survives the trip through the library's container format
    (fp16 holding 4096 x the bf16 value) unchanged."""
    import torch
    import cases
    from cudabert_b200 import synth
    from oracle import bert_oracle
    for name in ("c0_affine", "c1_small"):
        wname = cases.CASES[name]["weights"]
        dims = synth.model_dims(cases.WEIGHT_SETS[wname][0])
        ids, seg, mask = cases.case_inputs(name)
        mx = bert_oracle.activation_maxima(cases.get_weights(wname), ids[:2], seg[:2], mask[:2], dims["heads"],
                                           min(dims["layers"], 6))
        assert set(mx) == {"layernorm_out", "qkv", "context", "dense_out", "gelu_out"}
        assert max(mx.values()) < 100.0, mx
    w = cases.get_weights("base_affine")
    rounded = bert_oracle.round_encoder_weights_bf16(w)
    k = "bert_encoder_layer_3_intermediate_dense_kernel"
    assert not np.array_equal(rounded[k], w[k]) and np.array_equal(rounded["bert_pooler_dense_kernel"], w["bert_pooler_dense_kernel"])
    t = torch.from_numpy(rounded[k])
    assert torch.equal(t.bfloat16().float(), t)
    assert torch.equal((t * 4096.0).half().float() / 4096.0, t)
