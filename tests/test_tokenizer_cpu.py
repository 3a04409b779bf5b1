"""The native tokenizer against golden vectors made by the reference's own Python tokenizer
(tests/golden/make_tokenizer_golden.py): word-piece ids of hand-made sentences in several scripts and
of random strings over many Unicode blocks, and the fixed-length features of tab-separated lines,
lower-cased and cased."""
import json
import os
import pickle

import numpy as np
import pytest

from cudabert_b200.tokenizer import Tokenlizer, WordPieceTokenizer

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tokenizer_golden.json")


@pytest.fixture(scope="module")
def golden(tmp_path_factory):
    with open(GOLDEN, encoding="utf-8") as f:
        g = json.load(f)
    vf = tmp_path_factory.mktemp("vocab") / "vocab.txt"
    vf.write_text("\n".join(g["vocab"]) + "\n", encoding="utf-8")
    g["vocab_file"] = str(vf)
    return g


@pytest.mark.parametrize("mode", ["lower", "cased"])
def test_word_piece_ids_match_the_reference(golden, mode):
    tok = WordPieceTokenizer(golden["vocab_file"], do_lower_case=(mode == "lower"))
    assert tok.vocab_size == len(set(golden["vocab"]))
    bad = []
    for text, want in golden["cases"][mode]["tokenize"]:
        got = tok.tokenize(text).tolist()
        if got != want:
            bad.append((text, got, want))
    assert not bad, "%d of %d texts differ, first: %r" % (len(bad), len(golden["cases"][mode]["tokenize"]), bad[0])


@pytest.mark.parametrize("mode", ["lower", "cased"])
def test_line_features_match_the_reference(golden, mode):
    fn = Tokenlizer(golden["vocab_file"], do_lower_case=(mode == "lower"))
    fn = pickle.loads(pickle.dumps(fn))        # what a spawned reader process receives
    for k, (max_seq, line, ids_valid, n0) in enumerate(golden["cases"][mode]["features"]):
        index, raw, ids, mask, seg = fn(max_seq, line, k)
        n = len(ids_valid)
        assert index == k and raw == "\t".join(line.replace("\0", "").rstrip().split("\t"))
        assert ids.dtype == mask.dtype == seg.dtype == np.int32 and ids.shape == (max_seq,)
        assert ids.tolist() == ids_valid + [0] * (max_seq - n), (line, max_seq)
        assert mask.tolist() == [1] * n + [0] * (max_seq - n)
        assert seg.tolist() == [0] * n0 + [1] * (n - n0) + [0] * (max_seq - n)


def test_tokenizer_rejects_bad_arguments(tmp_path, golden):
    from cudabert_b200.cuda_bert import pybert
    assert not pybert.tokenizer_create(str(tmp_path / "missing.txt").encode(), 1)
    no_specials = tmp_path / "v.txt"
    no_specials.write_text("hello\nworld\n")
    assert not pybert.tokenizer_create(str(no_specials).encode(), 1)
    with pytest.raises(ValueError):
        WordPieceTokenizer(str(no_specials)).tokenize("hello")
    tok = WordPieceTokenizer(golden["vocab_file"])
    with pytest.raises(ValueError):
        tok.encode_pair("a", None, 2)
    # invalid UTF-8 is dropped, not fatal
    h = pybert.tokenizer_create(golden["vocab_file"].encode(), 1)
    out = np.zeros(8, np.int32)
    assert pybert.tokenizer_tokenize(h, b"\xff\xfe\xc3", out, 8) == 0
    assert pybert.tokenizer_tokenize(h, b"a b c d e f g h i j k l", out, 8) == 12   # reports the full count
    pybert.tokenizer_destroy(h)


def test_tokenizer_feeds_the_engine(tmp_path, golden):
    """Tokenlizer as Engine's tokenizer function with spawned stages (the fake replica of the engine
    tests returns the id sum and valid length of every line)."""
    from cudabert_b200.engine import Engine
    from test_engine_cpu import FakeReplica, Head, output_line, _config
    lines = [l for _, l, _, _ in golden["cases"]["lower"]["features"][:60] if "\n" not in l and "\r" not in l
             and "\x0b" not in l and "\x0c" not in l and "\x1c" not in l and "\x1d" not in l and "\x1e" not in l
             and "\x85" not in l and " " not in l and " " not in l]
    src, dst = tmp_path / "in.tsv", tmp_path / "out.tsv"
    src.write_text("\n".join(lines) + "\n", encoding="utf-8")
    cfg = _config([0, 1])
    cfg.mp_start_method = "spawn"
    eng = Engine(cfg)
    eng.set_cuda_model(FakeReplica)
    eng.set_finetune_layer(Head)
    fn = Tokenlizer(golden["vocab_file"])
    eng.set_tokenlizer_function(fn)
    eng.set_output_function(output_line)
    eng.run(str(src), str(dst))
    out = dst.read_text(encoding="utf-8").splitlines()
    read_back = src.read_text(encoding="utf-8").splitlines()
    assert len(out) == len(read_back)
    for k, line in enumerate(read_back):
        _, raw, ids, mask, _ = fn(cfg.max_seq_length, line + "\n", k)
        assert out[k] == "%s\t%d\t%d" % (raw, int((ids * mask).sum()), int(mask.sum()))


@pytest.mark.parametrize("threads,native", [(1, True), (4, True), (0, False)])
def test_engine_with_native_reader(tmp_path, golden, threads, native):
    """Engine.run with the tokenizer threads + batcher inside the library (and, for comparison, with
    the same tokenizer called line by line from the Python reader loop): every line comes out once,
    in order, with the features the tokenizer gives for it.  Lines hold a header, tabs, trailing
    blanks, NUL bytes and several scripts."""
    from cudabert_b200.engine import Engine
    from test_engine_cpu import FakeReplica, Head, output_line, _config
    texts = [t for t, _ in golden["cases"]["lower"]["tokenize"]]
    body = []
    for i in range(0, len(texts) - 1, 2):
        clean = lambda s: "".join(ch for ch in s if ch not in "\t\n\r\x0b\x0c\x1c\x1d\x1e\x85  ")
        a, b = clean(texts[i]), clean(texts[i + 1])
        body.append(a + "\t" + b + ("  " if i % 3 == 0 else ""))
        body.append(a + ("\0" if i % 5 == 0 else "") + ("\t" if i % 2 else ""))
    src, dst = tmp_path / "in.tsv", tmp_path / "out.tsv"
    src.write_bytes(("a header line\n" + "\n".join(body) + "\n").encode("utf-8"))
    cfg = _config([0, 1])
    cfg.mp_start_method = "spawn"
    cfg.skip_first_line = True
    cfg.native_reader = native
    cfg.reader_threads = threads
    cfg.alert_size = 40           # the writer will ask for flushes
    eng = Engine(cfg)
    eng.set_cuda_model(FakeReplica)
    eng.set_finetune_layer(Head)
    fn = Tokenlizer(golden["vocab_file"])
    eng.set_tokenlizer_function(fn)
    eng.set_output_function(output_line)
    eng.run(str(src), str(dst))
    out = dst.read_bytes().decode("utf-8").split("\n")[:-1]
    assert len(out) == len(body)
    for k, line in enumerate(body):
        _, raw, ids, mask, _ = fn(cfg.max_seq_length, line, k)
        assert out[k] == "%s\t%d\t%d" % (raw, int((ids * mask).sum()), int(mask.sum())), k


def test_native_reader_ends_lines_like_python_text_mode(tmp_path, golden):
    """"\\n", "\\r\\n" and a lone "\\r" all end a line, so the native reader numbers the lines of a file
    exactly as the Python reader (text mode, universal newlines) does."""
    from ctypes import byref, c_int, c_longlong, create_string_buffer
    from cudabert_b200.cuda_bert import pybert
    data = b"alpha one\tbeta\nsecond line\r\nthird\rfourth \t x\n\nlast without newline"
    path = tmp_path / "mixed.tsv"
    path.write_bytes(data)
    with open(path, "r", encoding="utf-8") as f:
        want = ["\t".join(l.replace("\0", "").rstrip().split("\t")) for l in f]
    assert len(want) == 6
    tok = Tokenlizer(golden["vocab_file"])
    tok._native()
    bounds = np.array([0, 8, 32], np.int32)
    reader = pybert.reader_create(str(path).encode(), tok._handle, 32, bounds, 3, 4, 2, 0, 0)
    assert reader
    got = {}
    rows, seq, first = c_int(0), c_int(0), c_longlong(0)
    try:
        while pybert.reader_next(reader, byref(rows), byref(seq), byref(first)) == 1:
            index = np.empty(rows.value, np.int64)
            offsets = np.empty(rows.value + 1, np.int64)
            t = [np.empty((rows.value, seq.value), np.int32) for _ in range(3)]
            assert pybert.reader_pop(reader, index, t[0], t[1], t[2], offsets) == rows.value
            raw = create_string_buffer(int(offsets[-1]) + 1)
            pybert.reader_raw(reader, raw, int(offsets[-1]))
            for i, n in enumerate(index.tolist()):
                got[n] = raw.raw[offsets[i]:offsets[i + 1]].decode("utf-8")
        assert pybert.reader_rejected(reader, None) == 0
        assert pybert.reader_lines(reader) == 6
    finally:
        pybert.reader_destroy(reader)
    assert [got[i] for i in range(6)] == want
