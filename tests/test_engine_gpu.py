"""The file-to-file Engine with real replicas: reader -> native batcher -> one worker process per
GPU (each loads its own model) -> writer.  Every output line must carry what a direct call on
that line alone returns: per-row results do not depend on which batch, bucket or GPU a line went
through.  The two-GPU case runs where two devices are visible."""
import numpy as np
import pytest

import cases
from cudabert_b200.config import Engin_Config
from cudabert_b200.cuda_model import Cuda_BERT
from cudabert_b200.engine import Engine

pytestmark = pytest.mark.gpu

MAX_SEQ = 48
N_OUT = 6


class Head:
    """Stands in for the application's fine-tune layer: keeps the first N_OUT pooler values."""
    def __init__(self, is_large):
        pass

    def init_finetune_layer(self, id_gpu):
        pass

    def run(self, pooled):
        return pooled[:, :N_OUT]


def tokenize(max_seq_length, line, index):
    toks = [int(t) for t in line.split()]
    n = min(len(toks), max_seq_length)
    ids = toks[:n] + [0] * (max_seq_length - n)
    mask = [1] * n + [0] * (max_seq_length - n)
    seg = [0] * (n // 2) + [1] * (n - n // 2) + [0] * (max_seq_length - n)
    return index, line.strip(), ids, mask, seg


def output_line(raw, output):
    return raw + "\t" + " ".join("%.6e" % v for v in output)


def _config(gpus, weight_dir):
    c = Engin_Config()
    c.gpu = gpus
    c.is_large = False
    c.max_seq_length = MAX_SEQ
    c.batch_size = 16
    c.start_split, c.end_split, c.split_size = 8, 40, 8
    c.model_npy_pth = weight_dir
    c.precision = "bf16"
    c.mp_start_method = "spawn"     # the parent process already holds a CUDA context
    return c


@pytest.mark.parametrize("n_gpus", [1, 2])
def test_engine_run_matches_direct_calls(tmp_path, weight_dirs, n_gpus):
    import torch
    if torch.cuda.device_count() < n_gpus:
        pytest.skip("needs %d GPUs" % n_gpus)
    wdir = weight_dirs("base_affine")
    rng = np.random.default_rng(11)
    lines = []
    for _ in range(150):
        n = int(rng.integers(2, MAX_SEQ + 1))
        lines.append(" ".join(str(int(x)) for x in [101] + list(rng.integers(1000, 30000, n - 1))))
    src, dst = str(tmp_path / "in.tsv"), str(tmp_path / "out.tsv")
    with open(src, "w") as f:
        f.write("\n".join(lines) + "\n")
    cfg = _config(list(range(n_gpus)), wdir)
    eng = Engine(cfg)
    eng.set_cuda_model(Cuda_BERT)
    eng.set_finetune_layer(Head)
    eng.set_tokenlizer_function(tokenize)
    eng.set_output_function(output_line)
    eng.run(src, dst)
    out = open(dst).read().splitlines()
    assert len(out) == len(lines)

    direct = Cuda_BERT(0, cfg)
    try:
        for i in list(range(0, 150, 7)) + [149]:
            _, raw, ids, mask, seg = tokenize(MAX_SEQ, lines[i], i)
            n = sum(mask)
            want = direct.encode([np.array([ids[:n]]), np.array([seg[:n]]), np.array([mask[:n]])])[0, :N_OUT]
            raw_out, vals = out[i].split("\t")
            assert raw_out == raw
            got = np.array([float(v) for v in vals.split()], np.float32)
            # printed with 7 significant digits; the arithmetic itself is batch-invariant
            np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-7)
    finally:
        direct.close()


@pytest.mark.parametrize("gpus", [[0, 0], [0, 1], [0, 0, 0]])
def test_replica_pool_in_one_process(weight_dirs, gpus):
    """Thread-per-replica pool: rows sharded over the replicas and gathered in order give exactly
    what one replica returns for the whole batch, for batches smaller than the pool too."""
    import torch
    from cudabert_b200.cuda_model import Cuda_BERT_Pool
    if torch.cuda.device_count() <= max(gpus):
        pytest.skip("needs %d GPUs" % (max(gpus) + 1))
    cfg = _config([0], weight_dirs("base_affine"))
    ids, seg, mask = cases.case_inputs("c0_affine")
    single = Cuda_BERT(0, cfg)
    pool = Cuda_BERT_Pool(gpus, cfg)
    try:
        want = single.encode([ids, seg, mask])
        for call in range(3):      # repeated calls reuse the threads and the handles
            np.testing.assert_array_equal(pool.encode([ids, seg, mask]), want, err_msg="whole batch, call %d" % call)
        np.testing.assert_array_equal(pool.encode([ids[:2], seg[:2], mask[:2]]), want[:2], err_msg="two rows")
        np.testing.assert_array_equal(pool.encode([ids[:1], seg[:1], None]), single.encode([ids[:1], seg[:1], None]),
                                      err_msg="one row, no mask")
        np.testing.assert_array_equal(pool.classify([ids, seg, mask]), single.classify([ids, seg, mask]),
                                      err_msg="classify")
    finally:
        pool.close()
        single.close()


@pytest.mark.parametrize("gpus", [[0], [0, 0], [0, 1]])
def test_engine_thread_mode_matches_direct_calls(tmp_path, weight_dirs, gpus):
    """replica_mode "thread": native reader and tokenizer, one thread per replica, writer, all in this
    process (two replicas may share a GPU).  Every output line carries what a direct call on that
    line alone returns."""
    import torch
    from cudabert_b200.tokenizer import Tokenlizer
    if torch.cuda.device_count() <= max(gpus):
        pytest.skip("needs %d GPUs" % (max(gpus) + 1))
    words = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] + ["w%d" % i for i in range(1200)]
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("\n".join(words) + "\n", encoding="utf-8")
    rng = np.random.default_rng(5)
    lines = []
    for _ in range(300):
        a = " ".join(words[5 + int(x)] for x in rng.integers(0, 1200, int(rng.integers(1, 20))))
        b = " ".join(words[5 + int(x)] for x in rng.integers(0, 1200, int(rng.integers(1, 20))))
        lines.append(a + "\t" + b)
    src, dst = str(tmp_path / "in.tsv"), str(tmp_path / "out.tsv")
    with open(src, "w", encoding="utf-8") as f:
        f.write("\n".join(lines) + "\n")
    cfg = _config(gpus, weight_dirs("base_affine"))
    cfg.replica_mode = "thread"
    tok = Tokenlizer(str(vocab))
    eng = Engine(cfg)
    eng.set_cuda_model(Cuda_BERT)
    eng.set_finetune_layer(Head)
    eng.set_tokenlizer_function(tok)
    eng.set_output_function(output_line)
    eng.run(src, dst)
    out = open(dst, encoding="utf-8").read().splitlines()
    assert len(out) == len(lines)
    direct = Cuda_BERT(0, cfg)
    try:
        for i in list(range(0, 300, 11)) + [299]:
            _, raw, ids, mask, seg = tok(MAX_SEQ, lines[i], i)
            n = int(mask.sum())
            want = direct.encode([ids[None, :n], seg[None, :n], mask[None, :n]])[0, :N_OUT]
            raw_out, vals = out[i].rsplit("\t", 1)
            assert raw_out == raw
            got = np.array([float(v) for v in vals.split()], np.float32)
            np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-7)
    finally:
        direct.close()
