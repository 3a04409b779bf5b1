"""File-to-file inference pipeline with the reference's ``Engine`` API (engine.py:169-403):

    engine = Engine(config)
    engine.set_cuda_model(Cuda_BERT)            # class: (id_gpu, config) -> .encode(tensor)
    engine.set_finetune_layer(Finetune_Layer)   # class: (is_large) -> .init_finetune_layer(gpu), .run(np[B,H])
    engine.set_tokenlizer_function(fn)          # (max_seq_length, line, index) -> (idx, raw, ids, mask, seg)
    engine.set_output_function(fn)              # (raw_line, output) -> str
    engine.run(input_file, output_file)

Stages, one OS process each as in the reference (engine.py:385-397): a reader that tokenises,
buckets lines by valid length (boundaries [0, start_split, start_split+split_size, ..., end_split,
max_seq_length], engine.py:225-232) and right-trims every batch to its own longest line
(utils.py:3-13); the bucketing itself runs in the library's native
batcher unless ``config.native_batcher`` is False; one worker per GPU id in ``config.gpu`` holding an independent replica (batch
sharding, no collective: workers pull whole batches from a shared queue); a writer that restores
the input order in a sliding window and applies back-pressure through ``alert_size``
(engine.py:303-375).

With a ``tokenizer.Tokenlizer`` as tokenizer function and more than two GPUs (or
``config.replica_mode = "thread"``) the same pipeline runs inside ONE process instead: the native
reader's tokenizer threads fill the buckets, one host thread per GPU drives its replica (the
library call releases the GIL), and the writer takes finished batches from an in-process queue --
no pickling and no pipes, which is what lets eight replicas be fed at their own rate (``_run_threads``).

Differences from the reference, on purpose: workers block on the queue instead of busy-polling
``empty()`` (engine.py:253-264); every stage is joined and a stage that dies is detected by the
parent instead of being waited for forever on a sentinel count (engine.py:312, 401): a dead replica
is dropped and the run resumes after the last line written, anything else stops the run with an
error; the standard ``logging`` module replaces the reference's colour logger.
"""
import copy
import os
import logging
import multiprocessing as mp
import queue as pyqueue
import sys
import time

from .utils import optimize_batch, Batch_Blob, Batch_Packed, Tagged_line

_DONE = "__stage_done__"


def get_mylogger():
    logger = logging.getLogger("cuda_bert.engine")
    if not logger.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter("%(asctime)s %(levelname)s %(message)s"))
        logger.addHandler(h)
        logger.setLevel(logging.INFO)
    return logger


class batch_container(object):
    """ Bucket of lines whose valid length lies in (base_length, top_length]. """
    def __init__(self, base_length, top_length, batchsize):
        self.base_length = base_length
        self.top_length = top_length
        self.prepare = []
        self.temp = []
        self.min_index = sys.maxsize
        self.batchsize = batchsize

    def put(self, tg_line):
        self.temp.append(tg_line)
        if len(self.temp) == self.batchsize:
            self._batch()

    def _batch(self):
        """ Batch the collected lines and keep the batch ready for the input queue """
        if len(self.temp) == 0:
            return
        batch_tensor = optimize_batch(self.temp)
        self.prepare.append(Batch_Packed(list(self.temp), batch_tensor))
        self.temp.clear()
        self.reset_min_index()

    def force_enqueue(self):
        """ Flush a partly filled bucket: memory pressure in the writer, or end of file """
        self._batch()

    def pop(self):
        ret = self.prepare.pop(0)
        self.reset_min_index()
        return ret

    def reset_min_index(self):
        if len(self.prepare) != 0:
            self.min_index = self.prepare[0].lines_list[0].num_line
        else:
            self.min_index = sys.maxsize
        return self.min_index


class queue_manager(object):
    """ Buckets for every length range plus the queues between the stages """
    def __init__(self, seq_length_split, list_gpu, logger, batchsize, ctx=None):
        ctx = ctx or mp.get_context()
        self.num_containers = len(seq_length_split) - 1
        self.boardlines = seq_length_split
        self.output_queue = ctx.Queue()
        self.force_queue = ctx.Queue(1)
        self.input_queue = ctx.Queue(10)
        self.logger = logger
        self.containers = [batch_container(self.boardlines[i], self.boardlines[i + 1], batchsize)
                           for i in range(self.num_containers)]

    def put(self, line):
        """ Find the bucket of the line's length and add it; ship batches that became ready """
        num_queue = 0
        while num_queue < self.num_containers - 1 and line.length > self.boardlines[num_queue + 1]:
            num_queue += 1
        self.containers[num_queue].put(line)
        self.enqueue(False)

    def force_enqueue(self):
        for container in self.containers:
            container.force_enqueue()
        while self.enqueue(True) != -1:
            pass

    def enqueue(self, is_force):
        """ Ship the ready batch that starts at the smallest line number (keeps the writer's
        window short); returns -1 when no bucket holds a ready batch """
        target = None
        for container in self.containers:
            if container.prepare and (target is None or container.reset_min_index() < target.min_index):
                target = container
        if target is None:
            return -1
        min_index = target.min_index
        self.input_queue.put(target.pop())   # bounded queue: blocks while the GPUs are busy
        return min_index

    def get(self, timeout=None):
        return self.input_queue.get(timeout=timeout)


class native_queue_manager(queue_manager):
    """ queue_manager whose buckets live in the library's native batcher (csrc/batcher.cc): the
    same put / enqueue / force_enqueue / get interface and the same batches, batch order and
    right-trimming, without the per-line Python list handling and the per-batch numpy stacking.
    The batcher itself is created in the process that first puts a line (the reader stage), so
    the manager can be handed to spawned processes. """
    def __init__(self, seq_length_split, list_gpu, logger, batchsize, ctx=None, max_seq_length=512):
        ctx = ctx or mp.get_context()
        self.boardlines = list(seq_length_split)
        self.num_containers = len(seq_length_split) - 1
        self.output_queue = ctx.Queue()
        self.force_queue = ctx.Queue(1)
        self.input_queue = ctx.Queue(10)
        self.logger = logger
        self.batchsize = batchsize
        self.max_seq_length = max_seq_length
        if (self.num_containers < 1 or batchsize < 1 or max_seq_length < 1 or
                any(b > a for b, a in zip(self.boardlines, self.boardlines[1:]))):
            raise ValueError("bad bucket boundaries %r / batch size %r" % (seq_length_split, batchsize))
        self._batcher = None
        self._lines = {}   # line number -> Tagged_line, until its batch leaves

    def __getstate__(self):
        state = dict(self.__dict__)
        state["_batcher"] = None    # a pointer of the creating process; each process makes its own
        state["_lines"] = {}
        return state

    def _native(self):
        from .cuda_bert import pybert
        if self._batcher is None:
            import numpy as np
            bounds = np.ascontiguousarray(self.boardlines, dtype=np.int32)
            self._batcher = pybert.batcher_create(bounds, len(bounds), self.batchsize, self.max_seq_length)
            if not self._batcher:
                raise ValueError("the native batcher rejected boundaries %r" % (self.boardlines,))
        return pybert

    def __del__(self):
        if getattr(self, "_batcher", None):
            try:
                from .cuda_bert import pybert
                pybert.batcher_destroy(self._batcher)
            except ImportError:   # interpreter shutdown: the process's memory goes with it
                pass
            self._batcher = None

    def _row(self, values):
        import numpy as np
        a = np.ascontiguousarray(values, dtype=np.int32)
        return a[:self.max_seq_length] if a.shape[0] > self.max_seq_length else a

    def put(self, line):
        lib = self._native()
        ids, seg, mask = self._row(line.input_ids), self._row(line.segment_ids), self._row(line.input_mask)
        n = min(ids.shape[0], seg.shape[0], mask.shape[0])
        length = lib.batcher_put(self._batcher, line.num_line, ids, seg, mask, n)
        if length < 0:
            raise ValueError("line %d: the batcher rejected a row of %d entries" % (line.num_line, n))
        line.length = length
        self._lines[line.num_line] = line
        self.enqueue(False)

    def force_enqueue(self):
        self._native().batcher_flush(self._batcher)
        while self.enqueue(True) != -1:
            pass

    def enqueue(self, is_force):
        from ctypes import byref, c_int, c_longlong
        import numpy as np
        lib = self._native()
        rows, seq, first = c_int(0), c_int(0), c_longlong(0)
        if lib.batcher_next(self._batcher, byref(rows), byref(seq), byref(first)) != 1:
            return -1
        index = np.empty(rows.value, np.int64)
        tensor = [np.empty((rows.value, seq.value), np.int32) for _ in range(3)]
        got = lib.batcher_pop(self._batcher, index, tensor[0], tensor[1], tensor[2])
        assert got == rows.value
        lines = [self._lines.pop(int(i)) for i in index]
        for tl in lines:
            tl.drop_features()    # they are in `tensor` now; pickling them again per line is the reader's main cost
        self.input_queue.put(Batch_Packed(lines, tensor))   # bounded queue: blocks while the GPUs are busy
        return int(first.value)


class Engine(object):
    def __init__(self, config):
        self.handle = None
        self.finetune_layer = None
        self.cuda_model = None
        self.tokenlizer_line = None
        self.output_line = None
        self.input_file = None
        self.output_file = None
        self.config = config
        self.logger = get_mylogger()
        self.poll_seconds = 0.2

    def _init(self):
        self.generate_splits()
        assert(self.cuda_model is not None)
        assert(self.finetune_layer is not None)
        assert(self.tokenlizer_line is not None)
        assert(self.output_line is not None)
        assert(self.config.gpu != [])
        self._ctx = mp.get_context(getattr(self.config, "mp_start_method", None))
        if getattr(self.config, "native_batcher", True):
            self.handle = native_queue_manager(self.seq_length_split, self.config.gpu, self.logger,
                                               self.config.batch_size, self._ctx, self.config.max_seq_length)
        else:
            self.handle = queue_manager(self.seq_length_split, self.config.gpu,
                                        self.logger, self.config.batch_size, self._ctx)

    def set_cuda_model(self, cuda_model):
        self.cuda_model = cuda_model

    def set_finetune_layer(self, finetune_layer):
        self.finetune_layer = finetune_layer

    def set_tokenlizer_function(self, tokenlizer_line):
        self.tokenlizer_line = tokenlizer_line

    def set_output_function(self, output_line):
        self.output_line = output_line

    def generate_splits(self):
        '''
        Boundaries of the length buckets over [0, max_length].
        Too sparse : wasted computation on padding.  Too dense : more lines wait in the writer.
        '''
        ret = [0]
        for i in range(self.config.start_split,
                       self.config.end_split + self.config.split_size,
                       self.config.split_size):
            ret.append(i)
        ret.append(self.config.max_seq_length)
        self.seq_length_split = ret

    # ------------------------------------------------------------------ stages
    def _engine_model(self, id_gpu):
        config = self.config
        handle = self.handle
        user_layer = self.finetune_layer(config.is_large)
        user_layer.init_finetune_layer(id_gpu)
        model = self.cuda_model(id_gpu, config)
        start = time.time()
        total_length = 0
        # A thread keeps the next batches ready (reading the pipe and unpickling take about a
        # millisecond per batch, during which the GPU would idle; the replica's call releases the GIL).
        import threading
        ahead = pyqueue.Queue(maxsize=2)

        def prefetch():
            while True:
                item = handle.get()
                ahead.put(item)
                if item == _DONE:
                    return
        threading.Thread(target=prefetch, daemon=True).start()
        while True:
            packed_batch = ahead.get()
            if packed_batch == _DONE:
                break
            output = model.encode(packed_batch.tensor)
            packed_batch.output = user_layer.run(output)
            total_length += packed_batch.tensor[0].shape[0]
            packed_batch.drop_tensor()       # the writer wants line numbers, raw lines and outputs only
            handle.output_queue.put(packed_batch)
        handle.output_queue.put(_DONE)
        stats = ""
        if getattr(model, "model", None) is not None and hasattr(getattr(model, "_pybert", None), "graph_replays"):
            stats = "; CUDA graphs: %d captured, %d passes replayed" % (model._pybert.graph_captures(model.model),
                                                                       model._pybert.graph_replays(model.model))
        self.logger.info("engine_model on gpu %s done: %d lines in %.2f s%s", id_gpu, total_length,
                         time.time() - start, stats)

    def _generate_tagged_line(self, user_output):
        return Tagged_line(
                num_line=user_output[0],
                line_data=user_output[1],
                input_ids=user_output[2],
                input_mask=user_output[3],
                segment_ids=user_output[4],
                measure=not isinstance(self.handle, native_queue_manager))

    def _engine_preprocess_native(self, input_file, start_line):
        """ The reader stage on the library's native reader (csrc/reader.cc): tokenizer threads fill
        the buckets, this loop only forwards finished batches. """
        import threading
        from ctypes import byref, c_int, c_longlong, create_string_buffer
        import numpy as np
        from .cuda_bert import pybert
        config, handle, tok = self.config, self.handle, self.tokenlizer_line
        tok._native()
        bounds = np.ascontiguousarray(self.seq_length_split, dtype=np.int32)
        threads = int(getattr(config, "reader_threads", 0)) or max(1, min(16, (os.cpu_count() or 2) - 1))
        reader = pybert.reader_create(input_file.encode("utf-8"), tok._handle, config.max_seq_length, bounds,
                                      len(bounds), config.batch_size, threads,
                                      start_line + (1 if config.skip_first_line else 0), start_line)
        if not reader:
            raise RuntimeError("native reader: cannot open %r" % (input_file,))
        stop = threading.Event()

        def forward_flush_requests():      # the writer asks for the partly filled buckets
            while not stop.is_set():
                try:
                    handle.force_queue.get(timeout=0.2)
                    pybert.reader_flush(reader)
                except pyqueue.Empty:
                    pass
        flusher = threading.Thread(target=forward_flush_requests, daemon=True)
        flusher.start()
        try:
            rows, seq, first = c_int(0), c_int(0), c_longlong(0)
            while pybert.reader_next(reader, byref(rows), byref(seq), byref(first)) == 1:
                index = np.empty(rows.value, np.int64)
                offsets = np.empty(rows.value + 1, np.int64)
                tensor = [np.empty((rows.value, seq.value), np.int32) for _ in range(3)]
                got = pybert.reader_pop(reader, index, tensor[0], tensor[1], tensor[2], offsets)
                assert got == rows.value
                raw = create_string_buffer(int(offsets[-1]) + 1)
                pybert.reader_raw(reader, raw, int(offsets[-1]))
                handle.input_queue.put(Batch_Blob(index, raw.raw[:int(offsets[-1])], offsets, tensor))
            bad = c_longlong(-1)
            if pybert.reader_rejected(reader, byref(bad)) > 0:
                raise RuntimeError("native reader: line %d could not be tokenised or bucketed" % bad.value)
            total = pybert.reader_lines(reader)
        finally:
            stop.set()
            flusher.join()
            pybert.reader_destroy(reader)
        for _ in self.config.gpu:
            handle.input_queue.put(_DONE)
        self.logger.info("engine_preprocess (native reader, %d threads) done: %d lines", threads, total)

    def _engine_preprocess(self, input_file, start_line=0):
        config = self.config
        handle = self.handle
        from .tokenizer import Tokenlizer
        if getattr(config, "native_reader", True) and isinstance(self.tokenlizer_line, Tokenlizer):
            return self._engine_preprocess_native(input_file, start_line)
        with open(input_file, 'r', encoding='utf-8') as f:
            if self.config.skip_first_line:
                f.readline()
            for _ in range(start_line):      # a resumed run: these lines are in the output file already
                f.readline()
            index = start_line
            for line in f:
                handle.put(self._generate_tagged_line(self.tokenlizer_line(config.max_seq_length, line, index)))
                index += 1
                try:
                    handle.force_queue.get_nowait()
                    handle.force_enqueue()
                except pyqueue.Empty:
                    pass
            handle.force_enqueue()
        for _ in self.config.gpu:
            handle.input_queue.put(_DONE)
        self.logger.info("engine_preprocess done: %d lines", index)

    def _engine_postprocess(self, output_file, start_line=0, progress=None):
        """ progress: shared [lines written, bytes written], updated after every flush, so that the
        parent can cut the file back to a consistent state and resume if a replica dies. """
        handle = self.handle
        done = 0
        window = {}            # line number -> formatted text, for lines that arrived early
        next_line = start_line
        with open(output_file, 'a' if start_line else 'w', encoding='utf-8') as f:
            while done < len(self.config.gpu):
                packed_batch = handle.output_queue.get()
                if packed_batch == _DONE:
                    done += 1
                    continue
                for num_line, line_data, output in packed_batch.results():
                    if num_line in window or num_line < next_line:
                        raise RuntimeError("Line Index {} is written twice!".format(num_line))
                    window[num_line] = self.output_line(line_data, output)
                while next_line in window:
                    f.write(window.pop(next_line) + '\n')
                    next_line += 1
                if progress is not None:
                    f.flush()
                    with progress.get_lock():
                        progress[0], progress[1] = next_line, os.fstat(f.fileno()).st_size
                if len(window) > self.config.alert_size:
                    # too many lines wait for a slow bucket: make the reader flush its partial buckets
                    try:
                        handle.force_queue.put_nowait("force_enqueue Now")
                    except pyqueue.Full:
                        pass
            if window:
                raise RuntimeError("%d lines never received their predecessors" % len(window))
        self.logger.info("engine_postprocess done: %d lines", next_line)

    # ------------------------------------------------------------------ driver
    def run(self, input_file, output_file):
        """ Runs the pipeline.  If a replica's process dies, the stages are stopped, the output file
        is cut back to the last line the writer had flushed, and the pipeline starts again from the
        next input line on the remaining GPUs (``config.resume_without_dead_gpu``, default True;
        the reference waits forever for the dead replica's end marker, engine.py:312).  A reader or
        writer that dies, or the last replica dying, ends the run with RuntimeError. """
        assert(type(output_file) == str)
        assert(type(input_file) == str)
        self.config.input_file = input_file
        self.config.output_file = output_file
        assert(self.cuda_model is not None and self.finetune_layer is not None)
        assert(self.tokenlizer_line is not None and self.output_line is not None)
        assert(self.config.gpu != [])
        if self._wants_threads():
            self._run_threads(input_file, output_file)
            self.logger.info("ALL JOBS DONE")
            return
        start_line, offset = 0, 0     # lines and bytes of the output file that are known to be good
        while True:
            failed, progress = self._run_once(input_file, output_file, start_line, offset)
            if failed is None:
                break
            name, code = failed
            gpus = list(self.config.gpu)
            dead = [g for g in gpus if name == "gpu%s" % g]
            if not (dead and len(gpus) > 1 and getattr(self.config, "resume_without_dead_gpu", True)):
                raise RuntimeError("engine stage %s died with exit code %s; the run was stopped" % failed)
            # the writer publishes (lines, bytes) together after every flush; the pair starts at the
            # previous attempt's values, so a replica that dies before the writer's first batch
            # (e.g. at model load) leaves the file exactly as the previous attempt left it
            start_line, offset = max(start_line, int(progress[0])), max(offset, int(progress[1]))
            with open(output_file, 'a', encoding='utf-8') as f:
                f.truncate(offset if start_line else 0)
            self.config.gpu = [g for g in gpus if g not in dead]
            self.logger.warning("replica on gpu %s died with exit code %s: resuming at line %d on gpus %s",
                                dead[0], code, start_line, self.config.gpu)
        self.logger.info("ALL JOBS DONE")

    # ------------------------------------------------------------------ one process, one thread per replica
    def _wants_threads(self):
        """ Whether run() uses the in-process pipeline: config.replica_mode "thread" / "process", or
        "auto" (default): threads when the native reader can do the tokenising (the tokenizer function
        is a tokenizer.Tokenlizer and config.native_reader is on) and more than two replicas have to
        be fed, which is where one reader process and its pipes become the limit. """
        from .tokenizer import Tokenlizer
        mode = getattr(self.config, "replica_mode", "auto")
        native = getattr(self.config, "native_reader", True) and isinstance(self.tokenlizer_line, Tokenlizer)
        if mode == "thread":
            if not native:
                raise ValueError('replica_mode "thread" needs a tokenizer.Tokenlizer as tokenizer function '
                                 "(a Python tokenizer would hold the interpreter lock that the replicas need)")
            return True
        return mode == "auto" and native and len(self.config.gpu) > 2

    def _run_threads(self, input_file, output_file):
        """ The pipeline inside one process.  Threads: the native reader's tokenizer threads (no
        interpreter lock), a feeder that turns finished buckets into Batch_Blobs, one thread per
        replica, and the caller's thread as the writer.  A replica whose model fails to load or whose
        call raises is dropped and its batch goes to another replica; the run fails only when no
        replica is left.  (A replica that crashes the process -- not an exception -- takes the run with
        it: that isolation is what the process-per-replica mode is for.) """
        import threading
        from ctypes import byref, c_int, c_longlong, create_string_buffer
        import numpy as np
        from .cuda_bert import pybert
        self.generate_splits()
        config, tok, log = self.config, self.tokenlizer_line, self.logger
        gpus = list(config.gpu)
        tok._native()
        bounds = np.ascontiguousarray(self.seq_length_split, dtype=np.int32)
        threads = int(getattr(config, "reader_threads", 0)) or max(1, min(4 * len(gpus), (os.cpu_count() or 2) - 1))
        reader = pybert.reader_create(input_file.encode("utf-8"), tok._handle, config.max_seq_length, bounds,
                                      len(bounds), config.batch_size, threads, 1 if config.skip_first_line else 0, 0)
        if not reader:
            raise RuntimeError("native reader: cannot open %r" % (input_file,))
        batches = pyqueue.Queue(maxsize=max(4, 3 * len(gpus)))   # feeder -> replicas
        results = pyqueue.Queue()                                 # replicas -> writer
        stop = threading.Event()
        state = {"issued": 0, "fed": False}

        def put_until_stopped(q, item):
            while not stop.is_set():
                try:
                    q.put(item, timeout=0.2)
                    return True
                except pyqueue.Full:
                    pass
            return False

        def feeder():
            try:
                rows, seq, first = c_int(0), c_int(0), c_longlong(0)
                while not stop.is_set() and pybert.reader_next(reader, byref(rows), byref(seq), byref(first)) == 1:
                    index = np.empty(rows.value, np.int64)
                    offsets = np.empty(rows.value + 1, np.int64)
                    tensor = [np.empty((rows.value, seq.value), np.int32) for _ in range(3)]
                    got = pybert.reader_pop(reader, index, tensor[0], tensor[1], tensor[2], offsets)
                    assert got == rows.value
                    raw = create_string_buffer(int(offsets[-1]) + 1)
                    pybert.reader_raw(reader, raw, int(offsets[-1]))
                    state["issued"] += 1
                    if not put_until_stopped(batches, Batch_Blob(index, raw.raw[:int(offsets[-1])], offsets, tensor)):
                        return
                bad = c_longlong(-1)
                if pybert.reader_rejected(reader, byref(bad)) > 0:
                    raise RuntimeError("line %d could not be tokenised or bucketed" % bad.value)
                state["fed"] = True
                results.put(("fed", None, None, None))
            except BaseException as e:       # the writer must not wait for batches that will never come
                results.put(("feeder_failed", None, None, e))

        def replica(gpu):
            try:
                layer = self.finetune_layer(config.is_large)
                layer.init_finetune_layer(gpu)
                model = self.cuda_model(gpu, config)
            except BaseException as e:
                results.put(("replica_failed", gpu, None, e))
                return
            done, t0 = 0, time.time()
            while True:
                batch = batches.get()
                if batch is None:
                    break
                try:
                    batch.output = layer.run(model.encode(batch.tensor))
                except BaseException as e:
                    results.put(("replica_failed", gpu, batch, e))
                    return
                done += batch.tensor[0].shape[0]
                batch.drop_tensor()
                results.put(("done", gpu, batch, None))
            stats = ""
            handle = getattr(model, "model", None)
            if handle is not None and hasattr(getattr(model, "_pybert", None), "graph_replays"):
                # a caller whose batch shapes rarely repeat sees few replays: every pass then pays its launches
                stats = "; CUDA graphs: %d captured, %d passes replayed" % (model._pybert.graph_captures(handle),
                                                                           model._pybert.graph_replays(handle))
            close = getattr(model, "close", None)
            if close:
                close()
            log.info("replica thread on gpu %s done: %d lines in %.2f s%s", gpu, done, time.time() - t0, stats)

        workers = [threading.Thread(target=replica, args=(g,), daemon=True, name="replica-gpu%s" % g) for g in gpus]
        feed = threading.Thread(target=feeder, daemon=True, name="feeder")
        for t in workers + [feed]:
            t.start()
        alive, completed, next_line, window = len(gpus), 0, 0, {}
        failure = None
        t_first, lines_at_first = None, 0     # steady-state rate: from the first finished batch on
        try:
            with open(output_file, 'w', encoding='utf-8') as f:
                while not (state["fed"] and completed == state["issued"]):
                    kind, gpu, batch, exc = results.get()
                    if kind == "fed":
                        continue
                    if kind == "feeder_failed":
                        raise RuntimeError("engine reader failed: %r" % (exc,))
                    if kind == "replica_failed":
                        alive -= 1
                        log.warning("replica on gpu %s failed (%r): %d replicas left", gpu, exc, alive)
                        if gpu in self.config.gpu:
                            self.config.gpu = [g for g in self.config.gpu if g != gpu]
                        if alive == 0:
                            raise RuntimeError("engine: the last replica (gpu %s) failed: %r" % (gpu, exc))
                        if batch is not None:      # another replica takes the batch
                            batch.output = None
                            threading.Thread(target=put_until_stopped, args=(batches, batch), daemon=True).start()
                        continue
                    completed += 1
                    if t_first is None:
                        t_first, lines_at_first = time.time(), len(batch.index)
                    for num_line, line_data, output in batch.results():
                        if num_line in window or num_line < next_line:
                            raise RuntimeError("Line Index {} is written twice!".format(num_line))
                        window[num_line] = self.output_line(line_data, output)
                    while next_line in window:
                        f.write(window.pop(next_line) + '\n')
                        next_line += 1
                    if len(window) > config.alert_size:
                        pybert.reader_flush(reader)    # too many lines wait for a slow bucket
                if window:
                    raise RuntimeError("%d lines never received their predecessors" % len(window))
        except BaseException as e:
            failure = e
            raise
        finally:
            stop.set()
            for _ in workers:
                try:
                    batches.put_nowait(None)
                except pyqueue.Full:
                    try:
                        batches.get_nowait()
                        batches.put_nowait(None)
                    except (pyqueue.Empty, pyqueue.Full):
                        pass
            if failure is None:
                for t in workers:
                    t.join()
            feed.join(5)
            pybert.reader_destroy(reader)
        steady = time.time() - t_first if t_first else 0.0
        self.last_run = {"lines": next_line, "replicas_left": alive, "steady_seconds": steady,
                         "steady_lines_per_s": (next_line - lines_at_first) / steady if steady > 0 else 0.0}
        log.info("engine (threads): %d lines written; %.0f lines/s from the first finished batch on (%d replicas)",
                 next_line, self.last_run["steady_lines_per_s"], alive)

    def _run_once(self, input_file, output_file, start_line, offset=0):
        self._init()
        ctx = self._ctx
        progress = ctx.Array('q', [start_line, offset])
        procs = [("reader", ctx.Process(target=self._engine_preprocess, args=(input_file, start_line), daemon=True))]
        for num_gpu in self.config.gpu:
            procs.append(("gpu%s" % num_gpu, ctx.Process(target=self._engine_model, args=(num_gpu,), daemon=True)))
        procs.append(("writer", ctx.Process(target=self._engine_postprocess, args=(output_file, start_line, progress),
                                            daemon=True)))
        for _, p in procs:
            p.start()
        failed = None
        while failed is None and any(p.is_alive() for _, p in procs):
            for name, p in procs:
                if not p.is_alive() and p.exitcode not in (0, None):
                    failed = (name, p.exitcode)
                    break
            time.sleep(self.poll_seconds)
        for name, p in procs:
            if failed is None and p.exitcode not in (0, None):
                failed = (name, p.exitcode)
        if failed is not None:
            for _, p in procs:
                if p.is_alive():
                    p.terminate()
            for _, p in procs:
                p.join(5)
            return failed, progress
        for _, p in procs:
            p.join()
        return None, progress
