"""Generate the golden fixtures by running the REAL reference implementation.

Run where a checkout of the reference is present (``--reference``)::

    python tests/golden/make_golden.py [--reference /path/to/cudaBERT]

It imports the reference's bundled ``pytorch_pretrained_bert.BertModel``
(apps/pytorch_pretrained_bert/modeling.py:563-647) unmodified, loads the seeded synthetic
weights of ``tests/golden/cases.py`` into its ``state_dict`` (dense kernels transposed back
to ``nn.Linear.weight`` layout, the inverse of convert_pytorch_model_to_npys.py:62-63),
and stores for every case

* ``pooled``      fp32 pooler ``[B, H]`` of the fp32 model       (what the reference returns)
* ``pooled64``    pooler of the same module run in fp64          (tighter truth)
* ``probs``       Linear(H -> 2) + Softmax on ``pooled``         (apps/finetune.py:16-24)
* ``embed8`` / ``layer0_8`` / ``last8``  the first 8 features of every token after the
  embeddings, after encoder layer 0 and after the last layer (localises a mismatch)
* ``cls_hidden``  final hidden state of token 0 ``[B, H]``

Fixtures are a few KB to a few tens of KB each; the weights are never stored (they are a
function of the seed).  Nothing here runs on the GPU box: tests only read the ``.npz``.
"""
from __future__ import annotations

import argparse
import copy
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import cases  # noqa: E402


def load_reference_model(reference_root: str):
    sys.path.insert(0, os.path.join(reference_root, "apps"))
    from pytorch_pretrained_bert.modeling import BertConfig, BertModel  # type: ignore
    return BertConfig, BertModel


def to_state_dict(weights, layers):
    """npy-layout names -> BertModel.state_dict() names."""
    sd = {}
    g = lambda k: torch.from_numpy(np.asarray(weights[k]))
    sd["embeddings.word_embeddings.weight"] = g("bert_embeddings_word_embeddings")
    sd["embeddings.position_embeddings.weight"] = g("bert_embeddings_position_embeddings")
    sd["embeddings.token_type_embeddings.weight"] = g("bert_embeddings_token_type_embeddings")
    sd["embeddings.LayerNorm.weight"] = g("bert_embeddings_LayerNorm_gamma")
    sd["embeddings.LayerNorm.bias"] = g("bert_embeddings_LayerNorm_beta")
    for i in range(layers):
        s = "bert_encoder_layer_%d_" % i
        d = "encoder.layer.%d." % i
        for a, b in (("attention_self_query", "attention.self.query"),
                     ("attention_self_key", "attention.self.key"),
                     ("attention_self_value", "attention.self.value"),
                     ("attention_output_dense", "attention.output.dense"),
                     ("intermediate_dense", "intermediate.dense"),
                     ("output_dense", "output.dense")):
            sd[d + b + ".weight"] = g(s + a + "_kernel").t().contiguous()
            sd[d + b + ".bias"] = g(s + a + "_bias")
        for a, b in (("attention_output_LayerNorm", "attention.output.LayerNorm"),
                     ("output_LayerNorm", "output.LayerNorm")):
            sd[d + b + ".weight"] = g(s + a + "_gamma")
            sd[d + b + ".bias"] = g(s + a + "_beta")
    sd["pooler.dense.weight"] = g("bert_pooler_dense_kernel").t().contiguous()
    sd["pooler.dense.bias"] = g("bert_pooler_dense_bias")
    return sd


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CUDABERT_REFERENCE") or os.path.join(
        os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))), "reference"),
                    help="checkout of the reference project (default: $CUDABERT_REFERENCE, else the directory "
                         "'reference' beside this repository)")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    BertConfig, BertModel = load_reference_model(args.reference)
    torch.set_num_threads(os.cpu_count() or 1)

    by_weights = {}
    for name, c in cases.CASES.items():
        if args.only and name not in args.only.split(","):
            continue
        by_weights.setdefault(c["weights"], []).append(name)

    for wname, names in by_weights.items():
        large, dims = cases.WEIGHT_SETS[wname][0], None
        dims = cases.synth.model_dims(large)
        weights = cases.get_weights(wname)
        cfg = BertConfig(cases.synth.VOCAB_SIZE, hidden_size=dims["hidden"],
                         num_hidden_layers=dims["layers"], num_attention_heads=dims["heads"],
                         intermediate_size=dims["ffn"])
        model = BertModel(cfg).eval()
        missing = model.load_state_dict(to_state_dict(weights, dims["layers"]), strict=True)
        model64 = copy.deepcopy(model).double()
        wc = torch.from_numpy(weights["classifier_kernel"])
        bc = torch.from_numpy(weights["classifier_bias"])
        for name in names:
            ids, seg, mask = cases.case_inputs(name)
            ids_t = torch.from_numpy(ids).long()
            seg_t = torch.from_numpy(seg).long()
            mask_t = None if mask is None else torch.from_numpy(mask).long()
            with torch.no_grad():
                layers_out, pooled = model(ids_t, seg_t, mask_t, output_all_encoded_layers=True)
                embed = model.embeddings(ids_t, seg_t)
                _, pooled64 = model64(ids_t, seg_t, mask_t, output_all_encoded_layers=False)
                head = torch.nn.Linear(dims["hidden"], wc.shape[1])
                head.weight.copy_(wc.t())
                head.bias.copy_(bc)
                probs = torch.softmax(head(pooled), dim=-1)
            np.savez_compressed(
                cases.golden_path(name),
                pooled=pooled.numpy().astype(np.float32),
                pooled64=pooled64.numpy().astype(np.float64),
                probs=probs.numpy().astype(np.float32),
                embed8=embed[:, :, :8].numpy().astype(np.float32),
                layer0_8=layers_out[0][:, :, :8].numpy().astype(np.float32),
                last8=layers_out[-1][:, :, :8].numpy().astype(np.float32),
                cls_hidden=layers_out[-1][:, 0, :].numpy().astype(np.float32),
            )
            print("wrote", name, pooled.shape, "maxabs(fp32-fp64)=%.3g"
                  % float(np.abs(pooled.numpy() - pooled64.numpy()).max()))
        del model, model64
        cases.drop_weights(wname)


if __name__ == "__main__":
    main()
