"""The library's environment switches (read once per process): each setting runs the same cases in a
child process.  Switches that only change how the work is scheduled must give the same bits as the
default; switches that pick another kernel or tile shape must stay within a small distance of it."""
import os
import subprocess
import sys

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE_CASES = ["c0_affine", "c2_small", "edge_s17", "edge_b1s1", "edge_nomask", "edge_zero_row", "edge_holes"]
LARGE_CASES = ["c1_small", "c3_small", "c4_small"]
SWITCHES = ("CUDABERT_PACK", "CUDABERT_GRAPH", "CUDABERT_PDL", "CUDABERT_LAST_LAYER", "CUDABERT_ATTENTION",
            "CUDABERT_GEMM_PAIR", "CUDABERT_GEMM_SMALL_TILES", "CUDABERT_PRECISION", "CUDABERT_LN",
            "CUDABERT_FP8_OPERAND", "CUDABERT_ATTENTION_TILES", "CUDABERT_FP32_GEMM", "CUDABERT_LN_FOLD", "SWITCH_CHILD_PRECISION")


@pytest.fixture(scope="module")
def run_with(weight_dirs, tmp_path_factory):
    specs = ["%s:0:%s" % (weight_dirs("base_affine"), ",".join(BASE_CASES)),
             "%s:1:%s" % (weight_dirs("large_affine"), ",".join(LARGE_CASES))]
    folder = tmp_path_factory.mktemp("switches")
    cache = {}

    def run(**switches):
        key = tuple(sorted(switches.items()))
        if key not in cache:
            env = {k: v for k, v in os.environ.items() if k not in SWITCHES}
            env.update(switches)
            out = str(folder / ("out_%d.npz" % len(cache)))
            r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "switch_child.py"), out] + specs,
                               env=env, capture_output=True, text=True, timeout=600)
            assert r.returncode == 0, "%s: rc=%d\n%s\n%s" % (switches, r.returncode, r.stdout[-1500:], r.stderr[-1500:])
            cache[key] = dict(np.load(out))
        return cache[key]

    return run


@pytest.mark.parametrize("switch", ["CUDABERT_PACK=0", "CUDABERT_GRAPH=0", "CUDABERT_PDL=0", "CUDABERT_PDL=1",
                                    "CUDABERT_LAST_LAYER=full", "CUDABERT_LN=block"])
def test_scheduling_switches_keep_every_bit(run_with, switch):
    """Padded instead of packed rows, no graphs, dependent launch off or forced on, the last layer
    computed for every token, the other LayerNorm kernel: none of these may change a single bit of the
    pooler output."""
    default = run_with()
    name, value = switch.split("=")
    other = run_with(**{name: value})
    for case in BASE_CASES + LARGE_CASES:
        np.testing.assert_array_equal(other[case], default[case], err_msg="%s, case %s" % (switch, case))


@pytest.mark.parametrize("switch", ["CUDABERT_ATTENTION=tc", "CUDABERT_ATTENTION=persist", "CUDABERT_ATTENTION=mma",
                                    "CUDABERT_GEMM_PAIR=0", "CUDABERT_GEMM_SMALL_TILES=1", "CUDABERT_LN_FOLD=1"])
def test_kernel_choice_switches_stay_close(run_with, switch):
    """Another attention kernel or GEMM tile shape rounds at other places, and twelve or twenty-four
    layers of bf16 activations amplify that: the output stays within the bf16 mode's budget against the
    golden fp32 output (2e-2 of its scale), and within 1.5e-2 of the default's output."""
    default = run_with()
    name, value = switch.split("=")
    other = run_with(**{name: value})
    worst = {}
    for case in BASE_CASES + LARGE_CASES:
        gold = cases.load_golden(case)["pooled"]
        worst[case] = (float(np.abs(other[case] - gold).max() / np.abs(gold).max()),
                       float(np.abs(other[case] - default[case]).max() / np.abs(default[case]).max()))
    print(switch, {k: (round(a, 4), round(b, 4)) for k, (a, b) in worst.items()})
    for case, (to_gold, to_default) in worst.items():
        assert to_gold <= 2e-2, "%s, case %s vs golden: %g" % (switch, case, to_gold)
        assert to_default <= 1.5e-2, "%s, case %s vs default: %g" % (switch, case, to_default)


def test_attention_tile_switch_keeps_every_bit(run_with):
    """The tcgen05 attention kernel either gives every sequence its own 128-query tiles or cuts the
    packed rows into tiles that hold rows of several sequences.  A row walks the key blocks of its
    own sequence in the same order either way: with the kernel forced for every length, the two
    must agree in every bit (sequences of one and of several key blocks, masks with holes, a row
    without valid key)."""
    packed = run_with(CUDABERT_ATTENTION="tc", CUDABERT_ATTENTION_TILES="packed")
    sequence = run_with(CUDABERT_ATTENTION="tc", CUDABERT_ATTENTION_TILES="sequence")
    for case in BASE_CASES + LARGE_CASES:
        np.testing.assert_array_equal(packed[case], sequence[case], err_msg=case)


def test_fp32_gemm_switch_stays_at_fp32_level(run_with):
    """fp32 mode multiplies on the tensor cores (operands split into three bf16 planes, fp32
    accumulation) unless CUDABERT_FP32_GEMM=cuda sends the products to the CUDA cores.  Both are fp32
    computations of the same model; the tensor core's fp32 accumulator rounds less carefully than
    an FFMA chain, which shows as about 1e-4 on the pooler output, a tenth of the mode's budget of 1e-3.
    Both meet that budget against the golden output."""
    tensor = run_with(SWITCH_CHILD_PRECISION="fp32")
    cuda = run_with(SWITCH_CHILD_PRECISION="fp32", CUDABERT_FP32_GEMM="cuda")
    worst = {}
    for case in BASE_CASES + LARGE_CASES:
        gold = cases.load_golden(case)["pooled"]
        worst[case] = (float(np.abs(tensor[case] - cuda[case]).max()), float(np.abs(tensor[case] - gold).max()),
                       float(np.abs(cuda[case] - gold).max()))
    print({k: tuple("%.2g" % x for x in v) for k, v in worst.items()})
    for case, (between, t_gold, c_gold) in worst.items():
        assert between <= 4e-4, "%s: tensor-core and CUDA-core fp32 GEMMs differ by %g" % (case, between)
        assert t_gold <= 1e-3 and c_gold <= 1e-3, "%s: %g / %g against the golden output" % (case, t_gold, c_gold)


def test_fp8_operand_switch_keeps_every_bit(run_with):
    """FP8 mode reads the E4M3 weight bytes in the GEMM (converter warps widen them to fp16 in shared
    memory); CUDABERT_FP8_OPERAND=widened expands them to fp16 once at load instead.  Both feed the
    tensor core the same fp16 values in the same order: not a bit may differ."""
    in_kernel = run_with(SWITCH_CHILD_PRECISION="fp8")
    widened = run_with(SWITCH_CHILD_PRECISION="fp8", CUDABERT_FP8_OPERAND="widened")
    for case in BASE_CASES + LARGE_CASES:
        np.testing.assert_array_equal(widened[case], in_kernel[case], err_msg=case)
