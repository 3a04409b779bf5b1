"""BERT tokenisation for the engine's reader stage, backed by the library's native tokenizer
(csrc/tokenizer.cc).  ``Tokenlizer`` is a drop-in for the reference application's
``tokenlizer_line`` (apps/tokenlizer.py:136-147): called as ``(max_seq_length, line, index)`` on a
tab-separated ``text_a \\t text_b`` line it returns ``(index, raw line, ids, mask, segment ids)``,
the tuple ``Engine.set_tokenlizer_function`` expects, with the arrays as int32 numpy rows."""
import numpy as np


class WordPieceTokenizer(object):
    """``tokenize(text) -> int32 ids`` and ``encode_pair(a, b, max_seq_length) -> (ids, mask, seg)``.
    The native handle is made on first use in each process, so instances can be pickled."""

    def __init__(self, vocab_file, do_lower_case=True):
        self.vocab_file = vocab_file
        self.do_lower_case = bool(do_lower_case)
        self._handle = None

    def __getstate__(self):
        return {"vocab_file": self.vocab_file, "do_lower_case": self.do_lower_case, "_handle": None}

    def _native(self):
        from .cuda_bert import pybert
        if self._handle is None:
            self._handle = pybert.tokenizer_create(self.vocab_file.encode("utf-8"), int(self.do_lower_case))
            if not self._handle:
                raise ValueError("cannot use %r as a vocabulary: unreadable, or without [UNK] / [CLS] / [SEP]"
                                 % (self.vocab_file,))
        return pybert

    def __del__(self):
        if getattr(self, "_handle", None):
            try:
                from .cuda_bert import pybert
                pybert.tokenizer_destroy(self._handle)
            except ImportError:   # interpreter shutdown
                pass
            self._handle = None

    @property
    def vocab_size(self):
        return self._native().tokenizer_vocab_size(self._handle)

    def tokenize(self, text):
        lib = self._native()
        raw = text.replace("\0", "").encode("utf-8")
        out = np.empty(max(16, len(raw) + 1), np.int32)   # a word piece consumes at least one byte
        n = lib.tokenizer_tokenize(self._handle, raw, out, out.shape[0])
        if n < 0:
            raise ValueError("tokenizer rejected the text")
        return out[:n].copy()

    def encode_pair(self, text_a, text_b, max_seq_length):
        lib = self._native()
        ids, mask, seg = (np.empty(max_seq_length, np.int32) for _ in range(3))
        b = None if not text_b else text_b.replace("\0", "").encode("utf-8")
        n = lib.tokenizer_encode_pair(self._handle, text_a.replace("\0", "").encode("utf-8"), b, max_seq_length,
                                      ids, mask, seg)
        if n < 0:
            raise ValueError("tokenizer rejected the text (max_seq_length must be at least 3)")
        return ids, mask, seg


class Tokenlizer(WordPieceTokenizer):
    """The reader stage's per-line function (apps/tokenlizer.py:122-147): splits the line at tabs
    into text_a and, if present, text_b."""

    def __call__(self, max_seq_length, line, index):
        fields = line.replace("\0", "").rstrip().split("\t")
        ids, mask, seg = self.encode_pair(fields[0], fields[1] if len(fields) > 1 else None, max_seq_length)
        return index, "\t".join(fields), ids, mask, seg
