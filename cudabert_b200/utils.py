"""Line and batch containers of the engine: same names and fields as the reference's utils.py
(utils.py:3-67)."""
import numpy as np


def optimize_batch(tg_line_list):
    """Right-trim a bucket to its own longest valid length and stack it into three int32 arrays
    [ids, segment ids, mask] of shape [n, max_length] (reference: utils.py:3-13)."""
    max_length = max(tg_line.length for tg_line in tg_line_list)
    batch = []
    for i in range(3):
        new = np.ones([len(tg_line_list), max_length], dtype=np.int32)
        for j, tg_line in enumerate(tg_line_list):
            new[j] = np.asarray(tg_line.get_tensor(i)[0:max_length], dtype=np.int32)
        batch.append(new)
    return batch


class Batch_Packed(object):
    '''
        lines_list : list of Tagged_lines
        Tensor : [input_id, seg_id, mask], each [batchsize, seq]
        output : [batchsize, output_custom]
    '''
    def __init__(self, lines_list, tensor):
        self.lines_list = lines_list
        self.tensor = tensor
        self.output = None

    def set_output(self, output):
        self.output = output

    def write_line(self):
        for i in range(len(self.lines_list)):
            self.lines_list[i].output = self.output[i]


class Tagged_line(object):
    """A single set of features of data."""

    def __init__(self, num_line, line_data, input_ids, input_mask, segment_ids, measure=True):
        self.num_line = num_line
        self.line_data = line_data
        self.input_ids = input_ids
        self.input_mask = input_mask
        self.segment_ids = segment_ids
        self.length = 512
        if measure:          # the native batcher measures the line itself
            self._get_length()
        self.output = None

    def drop_features(self):
        """Forget the token arrays once they are inside a batch tensor: what travels on to the
        replica and the writer is the line number, the raw line and, later, the output."""
        self.input_ids = self.input_mask = self.segment_ids = None

    def _get_length(self):
        """ Useful length of the ids: 1 + index of the last mask entry equal to 1
        (stays 512 when the mask has none, as in the reference, utils.py:49-56)."""
        mask = np.asarray(self.input_mask)
        ones = np.nonzero(mask == 1)[0]
        if ones.size:
            self.length = int(ones[-1]) + 1

    def get_tensor(self, index):
        if index == 0:
            return self.input_ids
        if index == 1:
            return self.segment_ids
        if index == 2:
            return self.input_mask
