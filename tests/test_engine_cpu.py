"""The Engine pipeline on CPU with a stand-in for the GPU replica: bucketing by length, right-trim,
two worker processes pulling from one queue (the multi-GPU mode is batch sharding over
independent replicas), restoration of the input order, back-pressure, and detection of a worker
that dies.  Failures are injected on the host only."""
import os

import numpy as np
import pytest

from cudabert_b200.config import Engin_Config
from cudabert_b200.engine import Engine, batch_container, queue_manager
from cudabert_b200.utils import Tagged_line, optimize_batch

MAX_SEQ = 64


class FakeReplica:
    """encode() returns per line [sum of valid ids, valid length, gpu id]: depends on the trimmed
    content only, so any bucketing or ordering mistake shows in the output file."""
    def __init__(self, id_gpu, config):
        self.id_gpu = id_gpu

    def encode(self, tensor):
        ids, seg, mask = tensor
        assert ids.dtype == np.int32 and ids.shape == seg.shape == mask.shape
        assert mask[:, -1].max() == 1, "batch was not trimmed to its longest line"
        return np.stack([(ids * mask).sum(1), mask.sum(1), np.full(len(ids), self.id_gpu)], 1).astype(np.float32)


class DyingReplica(FakeReplica):
    def encode(self, tensor):
        if self.id_gpu == 1:
            os._exit(7)          # the replica process disappears mid-run
        return super().encode(tensor)


class Head:
    def __init__(self, is_large):
        pass

    def init_finetune_layer(self, id_gpu):
        pass

    def run(self, pooled):
        return pooled[:, :2]


def tokenize(max_seq_length, line, index):
    toks = [int(t) for t in line.split()]
    n = min(len(toks), max_seq_length)
    ids = toks[:n] + [0] * (max_seq_length - n)
    mask = [1] * n + [0] * (max_seq_length - n)
    return index, line.strip(), ids, mask, [0] * max_seq_length


def output_line(raw, output):
    return "%s\t%d\t%d" % (raw, int(output[0]), int(output[1]))


def _write_input(path, n_lines, seed=0):
    rng = np.random.default_rng(seed)
    lines = []
    for _ in range(n_lines):
        n = int(rng.integers(1, MAX_SEQ + 1))
        lines.append(" ".join(str(int(x)) for x in rng.integers(1, 1000, n)))
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
    return lines


def _config(gpus):
    c = Engin_Config()
    c.gpu = gpus
    c.is_large = False
    c.max_seq_length = MAX_SEQ
    c.batch_size = 8
    c.start_split, c.end_split, c.split_size = 8, 56, 8
    return c


@pytest.mark.parametrize("gpus,alert", [([0], 1000000), ([0, 1], 1000000), ([0, 1], 16)])
def test_engine_orders_output_and_shards_batches(tmp_path, gpus, alert):
    src, dst = str(tmp_path / "in.tsv"), str(tmp_path / "out.tsv")
    lines = _write_input(src, 301)
    cfg = _config(gpus)
    cfg.alert_size = alert
    eng = Engine(cfg)
    eng.set_cuda_model(FakeReplica)
    eng.set_finetune_layer(Head)
    eng.set_tokenlizer_function(tokenize)
    eng.set_output_function(output_line)
    eng.run(src, dst)
    out = open(dst).read().splitlines()
    assert len(out) == len(lines)
    for raw, got in zip(lines, out):
        toks = [int(t) for t in raw.split()]
        assert got == "%s\t%d\t%d" % (raw, sum(toks), len(toks))


def test_engine_reports_a_dead_replica(tmp_path):
    src, dst = str(tmp_path / "in.tsv"), str(tmp_path / "out.tsv")
    _write_input(src, 200)
    eng = Engine(_config([0, 1]))
    eng.set_cuda_model(DyingReplica)
    eng.set_finetune_layer(Head)
    eng.set_tokenlizer_function(tokenize)
    eng.set_output_function(output_line)
    with pytest.raises(RuntimeError, match="gpu1 died with exit code 7"):
        eng.run(src, dst)


def test_generate_splits_and_bucketing():
    cfg = Engin_Config()          # reference defaults: 50..180 step 2, max 200 (engine.py:225-232)
    eng = Engine(cfg)
    eng.generate_splits()
    assert eng.seq_length_split[:3] == [0, 50, 52] and eng.seq_length_split[-2:] == [180, 200]
    assert len(eng.seq_length_split) == 68
    tl = Tagged_line(3, "x", [5, 6, 7, 0, 0], [1, 1, 1, 0, 0], [0, 0, 1, 0, 0])
    assert tl.length == 3
    tl2 = Tagged_line(4, "y", [5, 6, 0, 0, 0], [1, 1, 0, 0, 0], [0, 0, 0, 0, 0])
    ids, seg, mask = optimize_batch([tl, tl2])
    assert ids.shape == (2, 3) and ids.dtype == np.int32
    assert mask.tolist() == [[1, 1, 1], [1, 1, 0]] and seg.tolist() == [[0, 0, 1], [0, 0, 0]]
    bc = batch_container(0, 8, 2)
    bc.put(tl)
    assert bc.prepare == []
    bc.put(tl2)
    assert len(bc.prepare) == 1 and bc.min_index == 3
    assert bc.pop().tensor[0].shape == (2, 3) and bc.min_index > 10 ** 9
