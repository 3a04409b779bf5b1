"""Containers that travel between the engine's stages.  Class, method and attribute names are the
ones code written against the reference uses (utils.py:3-67): ``Tagged_line`` (one tokenised input
line), ``Batch_Packed`` (a bucket's lines plus their stacked arrays) and ``optimize_batch``;
``Batch_Blob`` is the compact form of a batch that the native reader produces."""
import numpy as np

_FEATURES = ("input_ids", "segment_ids", "input_mask")   # order of Batch_Packed.tensor


class Tagged_line(object):
    """One line: its number in the input file, the raw text, the three token arrays, its valid
    length and, once a replica has seen it, its output row."""

    __slots__ = ("num_line", "line_data", "input_ids", "input_mask", "segment_ids", "length", "output")

    def __init__(self, num_line, line_data, input_ids, input_mask, segment_ids, measure=True):
        self.num_line, self.line_data = num_line, line_data
        self.input_ids, self.input_mask, self.segment_ids = input_ids, input_mask, segment_ids
        self.output = None
        self.length = 512        # what the reference leaves when the mask holds no 1 (utils.py:43-56)
        if measure:              # the native batcher measures the line itself
            self._get_length()

    def _get_length(self):
        """Valid length = 1 + position of the last mask entry equal to 1."""
        ones = np.flatnonzero(np.asarray(self.input_mask) == 1)
        if ones.size:
            self.length = int(ones[-1]) + 1

    def get_tensor(self, index):
        """0: ids, 1: segment ids, 2: mask."""
        return getattr(self, _FEATURES[index])

    def drop_features(self):
        """Forget the token arrays once they are inside a batch tensor: what travels on to the
        replica and the writer is the line number, the raw line and, later, the output."""
        self.input_ids = self.input_mask = self.segment_ids = None

    def __getstate__(self):
        return tuple(getattr(self, name) for name in self.__slots__)

    def __setstate__(self, state):
        for name, value in zip(self.__slots__, state):
            setattr(self, name, value)


def optimize_batch(tg_line_list):
    """[ids, segment ids, mask], each int32 [lines, L] with L the longest valid length among the
    lines: the bucket is right-trimmed to its own need (reference: utils.py:3-13)."""
    width = max(line.length for line in tg_line_list)
    stacked = []
    for which in range(len(_FEATURES)):
        rows = np.ones((len(tg_line_list), width), dtype=np.int32)
        for r, line in enumerate(tg_line_list):
            rows[r] = np.asarray(line.get_tensor(which)[:width], dtype=np.int32)
        stacked.append(rows)
    return stacked


class Batch_Packed(object):
    """A batch on its way through the pipeline: ``lines_list`` (Tagged_lines), ``tensor``
    ([ids, segment ids, mask], each [lines, L]) and, after the replica, ``output`` ([lines, ...])."""

    def __init__(self, lines_list, tensor):
        self.lines_list, self.tensor, self.output = lines_list, tensor, None

    def set_output(self, output):
        self.output = output

    def write_line(self):
        """Hand every line its own output row."""
        for line, row in zip(self.lines_list, self.output):
            line.output = row

    def results(self):
        """(line number, raw line, output row) of every line, for the writer."""
        for line, row in zip(self.lines_list, self.output):
            yield line.num_line, line.line_data, row

    def drop_tensor(self):
        """The replica is done with the token arrays; the writer does not need them."""
        self.tensor = None


class Batch_Blob(Batch_Packed):
    """A batch as the native reader delivers it: line numbers as one array and the raw text of all
    lines as one byte string with offsets, instead of one Python object per line.  Pickling it costs a
    few buffer copies, where a list of Tagged_lines costs several microseconds per line in each of the
    three hops between the stages.  ``lines_list`` is built on demand for code that wants the objects."""

    def __init__(self, index, text, offsets, tensor):
        self.index, self.text, self.offsets = index, text, offsets
        self.tensor, self.output = tensor, None
        self._lines = None

    def _raw(self, i):
        return self.text[self.offsets[i]:self.offsets[i + 1]].decode("utf-8", "replace")

    @property
    def lines_list(self):
        if self._lines is None:
            self._lines = [Tagged_line(int(n), self._raw(i), None, None, None, measure=False)
                           for i, n in enumerate(self.index)]
        return self._lines

    def write_line(self):
        for line, row in zip(self.lines_list, self.output):
            line.output = row

    def results(self):
        text, offsets = self.text, self.offsets.tolist()
        for i, (n, row) in enumerate(zip(self.index.tolist(), self.output)):
            yield n, text[offsets[i]:offsets[i + 1]].decode("utf-8", "replace"), row

    @staticmethod
    def _narrow(a):
        """Token arrays cross the process boundary in the smallest unsigned type that holds them
        (ids of a 30 522-word vocabulary in 16 bits, segment ids and mask in 8): a third of the bytes
        through the pipe.  __setstate__ widens them to int32 again."""
        lo, hi = (int(a.min()), int(a.max())) if a.size else (0, 0)
        if lo < 0 or hi > 0xFFFF:
            return a
        return a.astype(np.uint8 if hi <= 0xFF else np.uint16)

    def __getstate__(self):
        tensor = None if self.tensor is None else [None if t is None else self._narrow(t) for t in self.tensor]
        return self.index, self.text, self.offsets, tensor, self.output

    def __setstate__(self, state):
        self.index, self.text, self.offsets, tensor, self.output = state
        self.tensor = None if tensor is None else [None if t is None else t.astype(np.int32, copy=False)
                                                   for t in tensor]
        self._lines = None
