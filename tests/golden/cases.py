"""Shared table of parity cases: the generator of the golden fixtures, the CPU tests of the
oracle and the GPU parity tests all read it, so they agree on seeds and shapes.

Every case is a down-scaled or exact instance of one of the five benchmark workloads, or
an edge case of the call contract of ``Cuda_Bert`` (cuda_bert/cuda_bert.cu:55-70): ragged
and length-1 rows, ``mask == nullptr``, a row whose mask is all zero, a mask with holes.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from cudabert_b200 import synth  # noqa: E402

GOLDEN_DIR = os.path.dirname(os.path.abspath(__file__))

# weight sets: name -> (is_large, seed, affine)
WEIGHT_SETS = {
    "base_init": (False, synth.weight_seed(0), False),   # workload 0 as specified
    "base_affine": (False, 1100, True),
    "large_affine": (True, 1101, True),
}

# name -> dict(weights, batch, seq, dist, seed, mask_mode)
CASES = {
    "c0": dict(weights="base_init", batch=8, seq=128, dist="uniform:32:128", seed=synth.input_seed(0)),
    "c0_affine": dict(weights="base_affine", batch=8, seq=128, dist="uniform:32:128", seed=2100),
    "c1_small": dict(weights="large_affine", batch=4, seq=200, dist="uniform:16:200", seed=2101),
    "c2_small": dict(weights="base_affine", batch=16, seq=128, dist="tnormal:60:25:8:128", seed=2102),
    "c3_small": dict(weights="large_affine", batch=2, seq=512, dist="full", seed=2103),
    "c4_small": dict(weights="large_affine", batch=16, seq=64, dist="uniform:8:64", seed=2104),
    "edge_s17": dict(weights="base_affine", batch=3, seq=17, dist="uniform:1:17", seed=2105),
    "edge_b1s1": dict(weights="base_affine", batch=1, seq=1, dist="full", seed=2106),
    "edge_nomask": dict(weights="base_affine", batch=2, seq=40, dist="full", seed=2107, mask_mode="none"),
    "edge_zero_row": dict(weights="base_affine", batch=3, seq=33, dist="uniform:5:33", seed=2108,
                          mask_mode="zero_row"),
    "edge_holes": dict(weights="base_affine", batch=2, seq=50, dist="uniform:20:50", seed=2109,
                       mask_mode="holes"),
}

_weight_cache = {}


def get_weights(name: str):
    if name not in _weight_cache:
        large, seed, affine = WEIGHT_SETS[name]
        _weight_cache[name] = synth.make_weights(large, seed, affine)
    return _weight_cache[name]


def drop_weights(name: str):
    _weight_cache.pop(name, None)


def case_inputs(name: str):
    """Return (ids, seg, mask-or-None) for a case."""
    c = CASES[name]
    ids, seg, mask = synth.make_inputs(c["seed"], c["batch"], c["seq"], c["dist"])
    mode = c.get("mask_mode", "prefix")
    if mode == "none":
        mask = None
    elif mode == "zero_row":
        mask[1, :] = 0
    elif mode == "holes":
        rng = np.random.default_rng(c["seed"] + 7)
        holes = rng.random(mask.shape) < 0.25
        holes[:, 0] = False
        mask = (mask * (~holes)).astype(np.int32)
    return ids, seg, mask


def case_dims(name: str):
    large = WEIGHT_SETS[CASES[name]["weights"]][0]
    return large, synth.model_dims(large)


def golden_path(name: str) -> str:
    return os.path.join(GOLDEN_DIR, name + ".npz")


def load_golden(name: str):
    return dict(np.load(golden_path(name)))
