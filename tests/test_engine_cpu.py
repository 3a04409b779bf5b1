"""The Engine pipeline on CPU with a stand-in for the GPU replica: bucketing by length, right-trim,
two worker processes pulling from one queue (the multi-GPU mode is batch sharding over
independent replicas), restoration of the input order, back-pressure, and detection of a worker
that dies.  Failures are injected on the host only."""
import os

import numpy as np
import pytest

from cudabert_b200.config import Engin_Config
from cudabert_b200.engine import Engine, batch_container, native_queue_manager, queue_manager
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


@pytest.mark.parametrize("native", [True, False])
@pytest.mark.parametrize("gpus,alert", [([0], 1000000), ([0, 1], 1000000), ([0, 1], 16)])
def test_engine_orders_output_and_shards_batches(tmp_path, gpus, alert, native):
    src, dst = str(tmp_path / "in.tsv"), str(tmp_path / "out.tsv")
    lines = _write_input(src, 301)
    cfg = _config(gpus)
    cfg.alert_size = alert
    cfg.native_batcher = native
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


def test_engine_with_spawned_stages(tmp_path):
    """Start method "spawn" (what a parent that already holds a CUDA context needs): everything the
    stages receive has to survive pickling, the native batcher included."""
    src, dst = str(tmp_path / "in.tsv"), str(tmp_path / "out.tsv")
    lines = _write_input(src, 120)
    cfg = _config([0, 1])
    cfg.mp_start_method = "spawn"
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


def test_engine_resumes_without_a_dead_replica(tmp_path):
    """The replica on gpu 1 disappears at its first batch: the run is cut back to the last written
    line and finished on gpu 0 alone; every line is in the output exactly once and in order."""
    src, dst = str(tmp_path / "in.tsv"), str(tmp_path / "out.tsv")
    lines = _write_input(src, 300)
    cfg = _config([0, 1])
    eng = Engine(cfg)
    eng.set_cuda_model(DyingReplica)
    eng.set_finetune_layer(Head)
    eng.set_tokenlizer_function(tokenize)
    eng.set_output_function(output_line)
    eng.run(src, dst)
    assert cfg.gpu == [0]
    out = open(dst).read().splitlines()
    assert len(out) == len(lines)
    for raw, got in zip(lines, out):
        toks = [int(t) for t in raw.split()]
        assert got == "%s\t%d\t%d" % (raw, sum(toks), len(toks))


class DyingTwiceReplica(FakeReplica):
    """gpu 1 disappears in mid-run (after a few batches, so that lines are already written); gpu 2
    disappears while the RESUMED run loads its model, before the writer has seen a batch."""
    def __init__(self, id_gpu, config):
        super().__init__(id_gpu, config)
        self.calls = 0
        if 1 not in config.gpu:          # a resumed run
            if id_gpu == 2:
                os._exit(9)
            import time
            time.sleep(1.0)              # the surviving replica is still loading when gpu 2 is found dead

    def encode(self, tensor):
        self.calls += 1
        if self.id_gpu == 1 and self.calls == 4:
            os._exit(7)
        if self.id_gpu == 1:
            import time
            time.sleep(0.05)     # let the other replicas' lines reach the file first
        return super().encode(tensor)


def test_engine_keeps_written_lines_when_a_second_replica_dies_at_start_up(tmp_path):
    """Two failures in a row: the second strikes before the resumed run's writer has written
    anything.  The lines the first attempt wrote must survive, and the output must be complete."""
    src, dst = str(tmp_path / "in.tsv"), str(tmp_path / "out.tsv")
    lines = _write_input(src, 600)
    cfg = _config([0, 1, 2])
    eng = Engine(cfg)
    eng.set_cuda_model(DyingTwiceReplica)
    eng.set_finetune_layer(Head)
    eng.set_tokenlizer_function(tokenize)
    eng.set_output_function(output_line)
    eng.run(src, dst)
    assert cfg.gpu == [0]
    out = open(dst).read().splitlines()
    assert len(out) == len(lines)
    for raw, got in zip(lines, out):
        toks = [int(t) for t in raw.split()]
        assert got == "%s\t%d\t%d" % (raw, sum(toks), len(toks))


def test_engine_reports_a_dead_replica(tmp_path):
    src, dst = str(tmp_path / "in.tsv"), str(tmp_path / "out.tsv")
    _write_input(src, 200)
    cfg = _config([0, 1])
    cfg.resume_without_dead_gpu = False
    eng = Engine(cfg)
    eng.set_cuda_model(DyingReplica)
    eng.set_finetune_layer(Head)
    eng.set_tokenlizer_function(tokenize)
    eng.set_output_function(output_line)
    with pytest.raises(RuntimeError, match="gpu1 died with exit code 7"):
        eng.run(src, dst)


def test_engine_stops_when_its_only_replica_dies(tmp_path):
    src, dst = str(tmp_path / "in.tsv"), str(tmp_path / "out.tsv")
    _write_input(src, 50)
    eng = Engine(_config([1]))
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


class _ListQueue:
    """Unbounded stand-in for the managers' input queue, so that one process can drive them."""
    def __init__(self):
        self.items = []

    def put(self, x):
        self.items.append(x)


@pytest.mark.parametrize("seed,batch,flush_every", [(0, 8, 0), (1, 3, 37), (2, 1, 0), (3, 16, 5)])
def test_native_batcher_matches_the_python_buckets(seed, batch, flush_every):
    """Same stream into the Python buckets (the reference's algorithm, engine.py:12-130) and into
    the native batcher: identical batches (line numbers, trimmed arrays) in identical order,
    including forced flushes in mid-stream and lines whose mask has holes (a mask without any 1
    makes the reference's own trimming fail; the native batcher keeps such a row whole)."""
    rng = np.random.default_rng(seed)
    bounds = [0, 8, 16, 24, 40, MAX_SEQ]
    managers = [queue_manager(bounds, [0], None, batch), native_queue_manager(bounds, [0], None, batch, None, MAX_SEQ)]
    for m in managers:
        m.input_queue = _ListQueue()
    for i in range(400):
        n = int(rng.integers(1, MAX_SEQ + 1))
        ids = rng.integers(1, 1000, MAX_SEQ).tolist()
        seg = rng.integers(0, 2, MAX_SEQ).tolist()
        mask = [1] * n + [0] * (MAX_SEQ - n)
        if i % 41 == 7 and n > 1:
            mask[n // 2] = 0                      # a hole: the length is still set by the last 1
        for a in (ids, seg):
            a[n:] = [0] * (MAX_SEQ - n)
        for m in managers:
            m.put(Tagged_line(i, "line %d" % i, list(ids), list(mask), list(seg)))
            if flush_every and i % flush_every == flush_every - 1:
                m.force_enqueue()
    for m in managers:
        m.force_enqueue()
    py, nat = (m.input_queue.items for m in managers)
    assert len(py) == len(nat) and sum(len(b.lines_list) for b in nat) == 400
    for a, b in zip(py, nat):
        assert [l.num_line for l in a.lines_list] == [l.num_line for l in b.lines_list]
        assert [l.line_data for l in a.lines_list] == [l.line_data for l in b.lines_list]
        for x, y in zip(a.tensor, b.tensor):
            assert x.dtype == y.dtype == np.int32 and x.shape == y.shape
            np.testing.assert_array_equal(x, y)


def test_native_batcher_rejects_bad_arguments():
    from cudabert_b200.cuda_bert import pybert
    good = np.array([0, 8, 16], np.int32)
    assert not pybert.batcher_create(np.array([0, 8, 4], np.int32), 3, 4, 16)     # not ascending
    assert not pybert.batcher_create(good, 1, 4, 16) and not pybert.batcher_create(good, 3, 0, 16)
    b = pybert.batcher_create(good, 3, 2, 16)
    row = np.ones(16, np.int32)
    assert pybert.batcher_put(b, 0, row, row, row, 17) == -1 and pybert.batcher_put(b, 0, row, row, row, 0) == -1
    assert pybert.batcher_put(b, 0, row, row, np.zeros(16, np.int32), 16) == 16   # no 1 in the mask: whole row
    assert pybert.batcher_ready(b) == 0 and pybert.batcher_pending(b) == 1
    assert pybert.batcher_flush(b) == 1
    idx = np.zeros(2, np.int64)
    out = [np.zeros((2, 16), np.int32) for _ in range(3)]
    assert pybert.batcher_pop(b, idx, *out) == 1 and pybert.batcher_pop(b, idx, *out) == 0
    assert pybert.batcher_pending(b) == 0
    pybert.batcher_destroy(b)


# ---------------------------------------------------------------- one process, one thread per replica
def _word_vocab(tmp_path):
    words = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] + ["w%d" % i for i in range(200)]
    path = tmp_path / "vocab.txt"
    path.write_text("\n".join(words) + "\n", encoding="utf-8")
    return str(path), words


def _text_lines(path, n_lines, words, seed=3):
    rng = np.random.default_rng(seed)
    lines = []
    for _ in range(n_lines):
        a = " ".join(words[5 + int(x)] for x in rng.integers(0, 200, int(rng.integers(1, 30))))
        b = " ".join(words[5 + int(x)] for x in rng.integers(0, 200, int(rng.integers(0, 30))))
        lines.append(a + ("\t" + b if b else ""))
    with open(path, "w", encoding="utf-8") as f:
        f.write("\n".join(lines) + "\n")
    return lines


class FlakyReplica(FakeReplica):
    """gpu 1 cannot load its model; gpu 2 fails at its third batch: exceptions, not crashes."""
    def __init__(self, id_gpu, config):
        super().__init__(id_gpu, config)
        self.calls = 0
        if id_gpu == 1:
            raise RuntimeError("no such device")

    def encode(self, tensor):
        self.calls += 1
        if self.id_gpu == 2 and self.calls == 3:
            raise RuntimeError("replica lost")
        return super().encode(tensor)


@pytest.mark.parametrize("replica,gpus,left", [(FakeReplica, [0, 1, 2, 3], [0, 1, 2, 3]), (FlakyReplica, [0, 1, 2], [0]),
                                               (FakeReplica, [5], [5])])
def test_engine_thread_mode(tmp_path, replica, gpus, left):
    """replica_mode "thread": native reader -> one thread per replica -> writer, all in this process.
    Every line comes out once, in order, with what the replica computes for its own tokens, also
    when a replica fails to start and another fails in mid-run (their batches go to the survivors)."""
    from cudabert_b200.tokenizer import Tokenlizer
    vocab, words = _word_vocab(tmp_path)
    src, dst = str(tmp_path / "in.tsv"), str(tmp_path / "out.tsv")
    lines = _text_lines(src, 700, words)
    cfg = _config(gpus)
    cfg.replica_mode = "thread"
    cfg.alert_size = 64            # also exercises the flush request
    tok = Tokenlizer(vocab)
    eng = Engine(cfg)
    eng.set_cuda_model(replica)
    eng.set_finetune_layer(Head)
    eng.set_tokenlizer_function(tok)
    eng.set_output_function(output_line)
    eng.run(src, dst)
    assert cfg.gpu == left
    out = open(dst, encoding="utf-8").read().splitlines()
    assert len(out) == len(lines)
    for i, (raw, got) in enumerate(zip(lines, out)):
        _, raw_line, ids, mask, _ = tok(MAX_SEQ, raw, i)
        assert got == "%s\t%d\t%d" % (raw_line, int((ids * mask).sum()), int(mask.sum()))


def test_engine_thread_mode_stops_when_no_replica_is_left(tmp_path):
    from cudabert_b200.tokenizer import Tokenlizer
    vocab, words = _word_vocab(tmp_path)
    src, dst = str(tmp_path / "in.tsv"), str(tmp_path / "out.tsv")
    _text_lines(src, 200, words)
    cfg = _config([1])
    cfg.replica_mode = "thread"
    eng = Engine(cfg)
    eng.set_cuda_model(FlakyReplica)
    eng.set_finetune_layer(Head)
    eng.set_tokenlizer_function(Tokenlizer(vocab))
    eng.set_output_function(output_line)
    with pytest.raises(RuntimeError, match="last replica"):
        eng.run(src, dst)


def test_engine_mode_selection(tmp_path):
    """Threads need the native reader (a Python tokenizer would hold the interpreter lock); "auto"
    takes them from three replicas on."""
    from cudabert_b200.tokenizer import Tokenlizer
    vocab, _ = _word_vocab(tmp_path)
    eng = Engine(_config([0, 1, 2]))
    eng.set_tokenlizer_function(tokenize)
    assert not eng._wants_threads()
    eng.config.replica_mode = "thread"
    with pytest.raises(ValueError):
        eng._wants_threads()
    eng.config.replica_mode = "auto"
    eng.set_tokenlizer_function(Tokenlizer(vocab))
    assert eng._wants_threads()
    eng.config.gpu = [0, 1]
    assert not eng._wants_threads()
    eng.config.replica_mode = "process"
    eng.config.gpu = [0, 1, 2, 3]
    assert not eng._wants_threads()
