#!/usr/bin/env python
"""Throughput of the BERT-encoder hot path on B200 in sequences/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config 0|1|2|3|4] [--feed raw|engine]

--config picks one of the five workloads of the benchmark specification (cudabert_b200/synth.py:
CONFIGS); the default, 1, is the headline: BERT-large, batch 128, seq 200, valid lengths uniform in
[16, 200], pooler followed by the Linear(1024 -> 2) + Softmax head, 16-bit mode with bf16 weights.
  0  BERT-base  fp32  batch 8    seq 128  lengths U[32,128]
  2  BERT-base  bf16  batch 256  seq 128  lengths ~ N(60,25) clipped to [8,128]   (per GPU)
  3  BERT-large bf16  batch 32   seq 512  every position valid
  4  BERT-large fp8 weights  batch 1024  seq 64  lengths U[8,64]
--feed raw (default): one step = one fixed [batch, seq] array of synthetic lines, as stated above.
--feed engine: the same stream of lines first goes through the engine's length buckets and right-trim
(the library's native batcher, what Engine's reader stage runs), one step = one such batch.

Prints ONE JSON line:
  value      sequences/s with the batches already resident in HBM (device-side entry point),
             K steps timed with CUDA events on the replica's stream, max over ranks
  e2e        the same through the reference-facing call (Cuda_Classify: host arrays in, host
             probabilities out), copies inside the timed region
  roofline   achieved TFLOP/s of the dense-projection GEMM kernel (the kernel that holds ~97 % of the
             FLOPs), from CUDA events recorded around every launch on the launching stream
  cpu_baseline  the CPU oracle (a restatement of the reference's bundled PyTorch model) on a
             bounded sample of the same workload, on this box's host cores; when a build of the
             reference's own CUDA library is present (oracle/_ref), also that library's
             sequences/s on one batch of the workload on this GPU and the relative error of this
             library's pooler output against it (`reference_cuda_library_on_this_gpu`)

N > 1: one process per GPU (torchrun), independent replicas, weak scaling, no data-path
collective; ranks only meet in a host (gloo) barrier and a max-reduction of the timings.

--impl reference times the CPU oracle on all host cores on bounded samples of the workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from cudabert_b200 import synth  # noqa: E402

UNIT = "sequences/s"
L2_BYTES = 126e6


def describe(cfg):
    """(metric, workload description) of a configuration."""
    wl = synth.CONFIGS[cfg]
    d = synth.model_dims(wl["large"])
    size = "BERT-large" if wl["large"] else "BERT-base"
    prec = {"fp32": "fp32", "bf16": "bf16 weights, fp16 activations, fp32 accumulate",
            "fp8": "FP8-E4M3 weights (per-tensor scale), fp16 activations, fp32 accumulate"}[wl["precision"]]
    lens = {"full": "every position valid"}.get(wl["dist"], "valid lengths %s padded to %d" % (wl["dist"], wl["seq"]))
    metric = "%s seq%d sequences/sec" % (size, wl["seq"])
    work = ("C%d: %s (L%d H%d h%d F%d) %s, batch %d, seq %d, %s, pooler + Linear(%d->2) + Softmax"
            % (cfg, size, d["layers"], d["hidden"], d["heads"], d["ffn"], prec, wl["batch"], wl["seq"], lens, d["hidden"]))
    return metric, work


def flops_per_step(batch, seq, dims):
    """FLOPs of one padded batch: per token per layer 24 H^2 dense + 4 S H attention, plus the
    pooler (2 H^2 per sequence)."""
    H, L = dims["hidden"], dims["layers"]
    dense = batch * seq * L * 24 * H * H
    attn = batch * seq * L * 4 * seq * H
    return dense, attn, batch * 2 * H * H


def short_last_layer(precision):
    """Whether a pooler-only pass computes its last layer for the first token of each sequence only
    (16-bit modes, unless CUDABERT_LAST_LAYER=full)."""
    return precision != "fp32" and os.environ.get("CUDABERT_LAST_LAYER", "")[:1] != "f"


def executed_work(lens, dims, precision, padded_seq=None):
    """What one forward pass of a batch executes, given the rows each sequence has (`lens`: the live
    rows per sequence in the packed layout, or the padded length for every sequence otherwise):
    FLOPs of the dense-projection GEMMs, FLOPs of attention (4 * 64 per query-key pair and head),
    and the rows each of the 2 L LayerNorm launches works on."""
    H, L, F = dims["hidden"], dims["layers"], dims["ffn"]
    rows, seqs = int(lens.sum()), len(lens)
    keys = lens.astype(np.float64)
    per_row = 2 * (3 * H * H + H * H + 2 * H * F)
    pairs_full = float((keys * keys).sum())
    if short_last_layer(precision):
        gemm = (L - 1) * rows * per_row + rows * 2 * 3 * H * H + seqs * 2 * (H * H + 2 * H * F)
        attn = 4 * H * ((L - 1) * pairs_full + float(keys.sum()))      # last layer: one query per sequence
        ln_rows = [rows] * (2 * L - 2) + [seqs, seqs]
    else:
        gemm = L * rows * per_row
        attn = 4 * H * L * pairs_full
        ln_rows = [rows] * (2 * L)
    return gemm, attn, ln_rows


def layernorm_bytes_per_row(dims, precision):
    """Algorithmic bytes the residual LayerNorm moves per row.  16-bit modes: fp16 dense output and fp32
    residual in, fp16 GEMM operand and fp32 residual out (12 B per element).  fp32 mode: the GEMM
    epilogue has added the residual; fp32 in, fp32 out (8 B per element)."""
    return dims["hidden"] * (8 if precision == "fp32" else 12)


def live_tokens(mask):
    """Rows the packed layout computes for a batch: per line 1 + index of its last valid position
    (a line with no valid position counts as the full padded length)."""
    S = mask.shape[1]
    return np.where(mask.any(1), S - np.argmax(mask[:, ::-1] != 0, axis=1), S)


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(tensor=float(d.get("bf16_tflops_sustained", d.get("bf16_tflops"))), hbm=float(d["hbm_gbs"]),
                    burst=float(d.get("bf16_tflops", 0.0)) or None,
                    source="measured (MEASURED_PEAKS.json, sustained bf16)")
    return dict(tensor=1590.0, hbm=6650.0, burst=1590.0, source="fallback")


def measured_traffic(kernel, cfg):
    """DRAM bytes (read + write) per launch of `kernel` on configuration `cfg` from an ncu capture, as
    recorded in profiles/kernel_traffic.json ({kernel: {"c<cfg>": {"dram_bytes_per_launch": ...}}});
    None when no capture is on record."""
    p = os.path.join(ROOT, "profiles", "kernel_traffic.json")
    try:
        with open(p) as f:
            rec = json.load(f)[kernel]["c%d" % cfg]
        return float(rec["dram_bytes_per_launch"]), rec.get("source")
    except (OSError, KeyError, ValueError, TypeError):
        return None, None


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 50 ms while the timed and profiled regions run."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu):
        self.gpu = gpu
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [c for c, p in zip(sm, power) if p > 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "power_w_max": max(power), "samples": len(sm), "samples_under_load": len(busy),
                "period_ms": 50}


def engine_splits(seq):
    """Bucket boundaries of the engine for a maximum length `seq`: the reference's defaults (first
    inner boundary 50, last 180, step 2, for a maximum of 200; engine.py:225-232) scaled to `seq`."""
    lo, hi = max(2, 50 * seq // 200), max(4, 180 * seq // 200)
    inner = list(range(lo, hi + 1, 2))
    return [0] + [b for b in inner if 0 < b < seq] + [seq]


def make_batches(cfg, n_batches, rank, feed):
    """Host batches (ids, seg, mask) of the workload.  raw: n_batches arrays of the stated shape.
    engine: a stream of such lines pushed through the native batcher (length buckets, right-trim);
    n_batches of the full batches it emits, evenly spaced over the stream, are kept."""
    wl = synth.CONFIGS[cfg]
    B, S = wl["batch"], wl["seq"]
    if feed == "raw":
        return [synth.make_inputs(synth.input_seed(cfg) + 1000 * rank + i, B, S, wl["dist"]) for i in range(n_batches)]
    from ctypes import byref, c_int, c_longlong
    from cudabert_b200.cuda_bert import pybert
    bounds = np.ascontiguousarray(engine_splits(S), dtype=np.int32)
    batcher = pybert.batcher_create(bounds, len(bounds), B, S)
    if not batcher:
        raise RuntimeError("batcher_create failed")
    out = []
    line = 0
    # enough lines for every bucket to fill about three times, so that the batches kept below are the
    # engine's steady-state mix of lengths and not just its widest buckets
    n_lines = 3 * (len(bounds) - 1) * B
    try:
        for i in range((n_lines + B - 1) // B):
            ids, seg, mask = synth.make_inputs(synth.input_seed(cfg) + 1000 * rank + i, B, S, wl["dist"])
            for r in range(B):
                pybert.batcher_put(batcher, line, ids[r], seg[r], mask[r], S)
                line += 1
            while pybert.batcher_ready(batcher) > 0:
                rows, seq, first = c_int(0), c_int(0), c_longlong(0)
                pybert.batcher_next(batcher, byref(rows), byref(seq), byref(first))
                idx = np.empty(rows.value, np.int64)
                t = [np.empty((rows.value, seq.value), np.int32) for _ in range(3)]
                pybert.batcher_pop(batcher, idx, t[0], t[1], t[2])
                out.append(tuple(t))
    finally:
        pybert.batcher_destroy(batcher)
    if not out:
        raise RuntimeError("the batcher emitted no full batch")
    if len(out) > n_batches:     # evenly spaced over the stream
        out = [out[int(k * len(out) / n_batches)] for k in range(n_batches)]
    return out


def weights_dir(cfg, rank_local, barrier):
    """Seeded synthetic weights of the configuration's model in the reference's .npy layout, written
    once per box."""
    large = synth.CONFIGS[cfg]["large"]
    d = os.path.join(tempfile.gettempdir(), "cudabert_bench_%s_seed%d" % ("large" if large else "base", synth.weight_seed(cfg)))
    done = d + ".complete"   # beside the directory: the reference's loader parses every file inside it
    if rank_local == 0 and not os.path.exists(done):
        synth.write_weight_dir(d, synth.make_weights(large, synth.weight_seed(cfg)))
        open(done, "w").close()
    barrier()
    return d


def reference_cuda_library(wdir, large, batch):
    """The reference's own CUDA library (fp32, cuBLAS), when oracle/_ref holds a build of it, on one
    batch of the workload on this GPU, in a process of its own: its sequences/s (host arrays in, pooler
    output out, like `e2e`) and its pooler output.  Reported beside the CPU baseline; never on the
    product path."""
    lib = os.path.join(ROOT, "oracle", "_ref", "libcudaBERT_ref.so")
    if not os.path.exists(lib):
        return None
    tmp = tempfile.mkdtemp(prefix="cudabert_ref_")
    inp, out = os.path.join(tmp, "in.npz"), os.path.join(tmp, "out.npy")
    np.savez(inp, ids=batch[0], seg=batch[1], mask=batch[2])
    try:
        r = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "run_ref_cuda.py"), wdir, str(int(large)), inp,
                            out, "5"], capture_output=True, text=True, timeout=300)
        if r.returncode != 0:
            why = (r.stderr.strip().splitlines() or r.stdout.strip().splitlines() or [""])[-1][:200]
            return {"unavailable": "reference CUDA library exited with %d: %s" % (r.returncode, why)}
        info = json.loads(r.stdout.strip().splitlines()[-1])
        return {"value": info["sequences_per_s"], "unit": UNIT, "ms_per_batch": info["ms_per_batch"],
                "sample": "%d calls of Cuda_Bert on one batch of the workload (padded, fp32, cuBLAS), wall clock"
                          % info["calls"], "pooled": np.load(out)}
    except Exception as e:   # timeout, unreadable output
        return {"unavailable": "reference CUDA library: %s" % type(e).__name__}


# ------------------------------------------------------------------ CPU baseline / reference arm
def oracle_seq_per_s(cfg, n_seq, threads, repeats=1, weights=None):
    """Time the CPU oracle on n_seq sequences of the workload; returns (seq/s, seconds, weights)."""
    import torch
    from oracle import bert_oracle
    wl = synth.CONFIGS[cfg]
    torch.set_num_threads(threads)
    dims = synth.model_dims(wl["large"])
    if weights is None:
        weights = bert_oracle.Weights(synth.make_weights(wl["large"], synth.weight_seed(cfg)))
    ids, seg, mask = synth.make_inputs(synth.input_seed(cfg), n_seq, wl["seq"], wl["dist"])
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        _, pooled = bert_oracle.bert_forward(weights, ids, seg, mask, dims["heads"], dims["layers"])
        bert_oracle.classify(weights, torch.from_numpy(pooled))
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return n_seq / best, best, weights


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU implementation of the path (its bundled PyTorch
    model is not shipped to this box, so its restatement in oracle/ stands in: kind "port")."""
    if rank != 0:
        return
    cfg = args.config
    wl = synth.CONFIGS[cfg]
    metric, work = describe(cfg)
    threads = os.cpu_count() or 1
    # size the per-step sample so that warmup + steps stay within about two minutes
    rate, dt, w = oracle_seq_per_s(cfg, 2, threads)
    budget = 120.0 / max(args.steps + args.warmup, 1)
    n_seq = int(max(1, min(wl["batch"], rate * budget)))
    for _ in range(args.warmup):
        oracle_seq_per_s(cfg, n_seq, threads, weights=w)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle_seq_per_s(cfg, n_seq, threads, weights=w)
    total = time.perf_counter() - t0
    value = n_seq * args.steps / total
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": work, "sample_sequences_per_step": n_seq, "batch_of_the_workload": wl["batch"]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "%d sequences of the workload per step (seq %d, lengths %s), fp32, "
                                   "torch CPU ops, %d threads" % (n_seq, wl["seq"], wl["dist"], threads)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ our arm
def run_ours(args, rank, local_rank, world, barrier, allmax):
    import torch
    from cudabert_b200.cuda_bert import pybert
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the hot path has no CPU fallback")
    cfg = args.config
    wl = synth.CONFIGS[cfg]
    metric, work = describe(cfg)
    precision, large = wl["precision"], wl["large"]
    dev = local_rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    dims = synth.model_dims(large)
    B, S = wl["batch"], wl["seq"]
    wdir = weights_dir(cfg, local_rank, barrier)
    n_pool = 4 if args.feed == "raw" else 48
    host = make_batches(cfg, n_pool, rank, args.feed)
    n_pool = len(host)
    ref_cuda = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.layers:
        ref_cuda = reference_cuda_library(wdir, large, host[0])   # before this process takes device memory
    t_load = time.perf_counter()
    model = pybert.load_model(large, wdir, dev, B, S, precision=precision, num_layers=args.layers)
    load_seconds = time.perf_counter() - t_load   # .npy directory -> device-resident K-major operands
    if args.layers:
        dims = dict(dims, layers=min(args.layers, dims["layers"]))
    C = pybert.num_classes(model)
    stream = torch.cuda.ExternalStream(pybert.stream(model), device=dev)

    devb = [tuple(torch.from_numpy(a).to("cuda:%d" % dev) for a in hb) for hb in host]
    probs = [np.zeros((hb[0].shape[0], C), np.float32) for hb in host]
    rows_of = [hb[0].shape[0] for hb in host]

    def step_dev(i):
        ids, seg, mask = devb[i % n_pool]
        rc = pybert.classify_dev(model, ids.data_ptr(), seg.data_ptr(), mask.data_ptr(), ids.shape[0], ids.shape[1])
        if rc:
            raise RuntimeError("forward failed: " + pybert.last_error(model))

    def step_e2e(i):
        ids, seg, mask = host[i % n_pool]
        pybert.classify(model, probs[i % n_pool], ids, seg, ids.shape[0], ids.shape[1], C, mask)

    def timed(fn, steps, sync_after):
        barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(i)
        e1.record(stream)
        if sync_after:
            rc = pybert.sync(model)
            if rc:
                raise RuntimeError("sync failed: " + pybert.last_error(model))
        torch.cuda.synchronize(dev)
        barrier()
        return allmax(e0.elapsed_time(e1))

    # warm-up: W steps as asked, and at least three passes over every pooled batch, after which each of
    # them replays as a CUDA graph (a pass is captured the third time its arguments are seen)
    warm_steps = max(args.warmup, 3 * n_pool)
    for i in range(warm_steps):
        step_dev(i)
    pybert.sync(model)
    pybert.check(model)

    sampler = ClockSampler(dev)
    if rank == 0:
        sampler.start()
    # host cost of enqueueing one step into an empty stream (the timed loop below can block on a
    # full launch queue, so it cannot show this)
    torch.cuda.synchronize(dev)
    t_host = time.perf_counter()
    step_dev(0)
    host_enqueue_ms = (time.perf_counter() - t_host) * 1e3
    pybert.sync(model)
    ms_total = timed(step_dev, args.steps, True)
    launches = pybert.launch_count(model) * args.steps
    seqs_timed = sum(rows_of[i % n_pool] for i in range(args.steps))
    # end to end through the reference-facing call, host buffers in and out
    for i in range(max(min(args.warmup, 3), 3)):
        step_e2e(i)
    ms_e2e = timed(step_e2e, args.steps, False)
    pybert.check(model)

    value = world * seqs_timed / (ms_total / 1e3)
    e2e_value = world * seqs_timed / (ms_e2e / 1e3)

    # per-kernel device times: CUDA events around every launch on the launching stream, over steps
    # enqueued back to back right after the timed regions (one synchronisation at the end), so the
    # kernels run at the clocks the power cap allows in a long run, not at those of an idle GPU
    pybert.profile_reset(model)
    pybert.profile_enable(model, 1)
    prof_steps = min(args.steps, 40)
    for i in range(prof_steps):
        step_dev(i)
    pybert.sync(model)
    pybert.profile_enable(model, 0)
    prof = pybert.profile_get(model)
    pybert.check(model)
    clocks = sampler.stop() if rank == 0 else None

    if rank != 0:
        pybert.unload_model(model)
        return
    peaks = load_peaks()
    gemm_ms = sum(prof[k][0] for k in prof if k.startswith("gemm") and k != "gemm_pooler")
    gemm_n = sum(prof[k][1] for k in prof if k.startswith("gemm") and k != "gemm_pooler")
    packed = os.environ.get("CUDABERT_PACK", "1") != "0"
    lens = [live_tokens(hb[2]) if packed else np.full(hb[0].shape[0], hb[0].shape[1]) for hb in host]
    work_of = [executed_work(l, dims, precision) for l in lens]
    prof_idx = [i % n_pool for i in range(prof_steps)]
    gflops = sum(work_of[i][0] for i in prof_idx)
    attn_exec = sum(work_of[i][1] for i in prof_idx)
    ln_row_launches = sum(sum(work_of[i][2]) for i in prof_idx)    # rows summed over all LayerNorm launches
    live_rows = sum(int(lens[i].sum()) for i in prof_idx) / prof_steps
    achieved = gflops / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else 0.0
    dense, attn, pool = flops_per_step(B, S, dims)
    total_ms = sum(v[0] for v in prof.values())
    kernels = {k: {"ms_per_step": v[0] / prof_steps, "launches_per_step": v[1] / prof_steps,
                   "share": (v[0] / total_ms if total_ms else 0)} for k, v in prof.items()}
    attn_ms = prof["attention"][0]
    ln_ms = prof["layernorm"][0]
    ln_bytes = ln_row_launches * layernorm_bytes_per_row(dims, precision)

    if ref_cuda and ref_cuda.get("pooled") is not None:
        # the reference's own fp32 pooler output for batch 0 against this library's output, full size
        from oracle import bert_oracle
        b0 = host[0]
        ours = np.zeros((b0[0].shape[0], dims["hidden"]), np.float32)
        pybert.bert(model, ours, b0[0], b0[1], b0[0].shape[0], b0[0].shape[1], b0[2])
        pybert.check(model)
        ref = ref_cuda.pop("pooled")
        # max |a - b| / max |b| (the measure the parity tests bound by 2e-2 in the 16-bit mode) and the
        # relative Frobenius norm, over all pooler outputs of the batch
        ref_cuda["rel_err_of_this_library_%s" % precision] = float(bert_oracle.rel_err(ours, ref))
        ref_cuda["rel_fro_err_of_this_library_%s" % precision] = float(np.linalg.norm(ours - ref) / np.linalg.norm(ref))
        ref_cuda["max_abs_err_of_this_library_%s" % precision] = float(np.abs(ours - ref).max())
    elif ref_cuda:
        ref_cuda.pop("pooled", None)

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        n_seq = min(16 if large else 64, B)
        rate, dt, _ = oracle_seq_per_s(cfg, n_seq, threads)
        cpu = {"value": rate, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": "%d sequences of the workload (seq %d, lengths %s) in one batch, fp32, "
                         "torch CPU ops, %.1f s" % (n_seq, S, wl["dist"], dt)}
        if ref_cuda:
            cpu["reference_cuda_library_on_this_gpu"] = ref_cuda

    lowp = precision != "fp32"
    f32_cuda = not lowp and os.environ.get("CUDABERT_FP32_GEMM", "")[:1] == "c"
    gemm_kernel = "gemm_f32_kernel" if f32_cuda else "gemm_tcgen05_pair_kernel"
    traffic, traffic_source = (None, None) if args.layers else measured_traffic(gemm_kernel, cfg)
    act_bytes = live_rows * (dims["hidden"] * (4 + 4 + 2 + 2 + 2 + 2 + 6) + dims["ffn"] * 2) if lowp else \
        live_rows * 4 * (dims["hidden"] * 7 + dims["ffn"])
    mean_rows = seqs_timed / args.steps
    line = {
        "metric": metric, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "host_enqueue_ms_per_step": host_enqueue_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": {"fp32": "f32", "bf16": "bf16", "fp8": "fp8"}[precision], "data": "synthetic",
        "config": {"workload": work, "feed": args.feed, "batch_per_gpu": B, "seq_len": S,
                   "global_batch": B * world, "sample_sequences_per_step": mean_rows,
                   "operands": ("fp32 on CUDA cores" if f32_cuda else
                                "fp32 weights and activations, each split into three bf16 planes; the tensor cores "
                                "(tcgen05 kind::f16) sum the six leading cross terms with fp32 accumulation"
                                if not lowp else
                                "dense weights rounded to %s and held in fp16; activations fp16; both tensor-core "
                                "operands fp16 (tcgen05 kind::f16), fp32 accumulation, fp32 residual stream"
                                % ("bf16" if precision == "bf16" else "FP8-E4M3 with a per-tensor scale")),
                   "parallelism": "replicas x%d (batch sharding, no collective)" % world,
                   "untimed_warmup_steps_run": warm_steps,
                   "l2": "activations written and re-read per step (%.0f MB) %s the 126 MB L2; %d batches alternate"
                         % (act_bytes / 1e6, "exceed" if act_bytes > L2_BYTES else "DO NOT exceed", n_pool),
                   "tflops_per_step_padded": (dense + attn + pool) / 1e12,
                   "layout": ("packed: padding tokens are not computed (%.0f live of %.0f token slots per step)"
                              % (live_rows, sum(h[0].size for h in host) / n_pool)) if packed else "padded",
                   "last_layer": ("attention-output, FFN and LayerNorm for the first token of each sequence "
                                  "only (all the pooler reads; same bits out as the full layer)"
                                  if short_last_layer(precision) else "every token"),
                   "tflops_per_step_executed_gemm": gflops / prof_steps / 1e12},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": int(sum(3 * h[0].size * 4 for h in host) / n_pool),
                "d2h_bytes_per_step": int(mean_rows * C * 4 + 4)},
        "gpu_launches": int(launches),
        "roofline": {"bound": "tensor",
                     "kernel": (gemm_kernel + " (QKV, attention-output, FFN1, FFN2)" if lowp or f32_cuda else
                                "gemm_tcgen05_pair_kernel (QKV, FFN1), gemm_tcgen05_kernel (attention-output, FFN2)"),
                     "achieved": achieved, "peak": peaks["tensor"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["tensor"] if peaks["tensor"] else None, "peak_source": peaks["source"],
                     # the same against the measured burst figure and the nominal dense bf16 peak of the part
                     "frac_of_measured_burst": achieved / peaks["burst"] if peaks.get("burst") else None,
                     "frac_of_nominal_2250": achieved / 2250.0,
                     "launches": gemm_n / prof_steps, "avg_launch_ms": gemm_ms / gemm_n if gemm_n else None,
                     "traffic": traffic, "traffic_unit": "DRAM bytes per launch (ncu, mean over the four GEMMs of a layer)",
                     "traffic_source": traffic_source},
        "kernels": kernels,
        "attention_kernel": pybert.attention_kernel_name(S) if lowp else "attention_f32_kernel",
        "attention_tflops": (attn_exec / (attn_ms / 1e3) / 1e12) if attn_ms else None,
        "layernorm_gbs": (ln_bytes / (ln_ms / 1e3) / 1e9) if ln_ms else None,
        "layernorm_frac_of_hbm_peak": (ln_bytes / (ln_ms / 1e3) / 1e9 / peaks["hbm"]) if ln_ms else None,
        "weight_load_seconds": round(load_seconds, 3),
        "graph_replays": int(pybert.graph_replays(model)),
        "cpu_baseline": cpu,
    }
    if f32_cuda:
        line["roofline"]["note"] = ("CUDABERT_FP32_GEMM=cuda: the GEMMs run on the CUDA cores (FFMA); the tensor-core "
                                    "peak is the denominator only because the contract asks for one")
    elif not lowp:
        line["roofline"]["note"] = ("achieved counts the 2 M N K fp32 FLOPs of the model; the tensor cores execute "
                                    "six bf16 products for each, so their own rate is 6 x this figure")
    if args.layers:
        line["profiling_only"] = "first %d encoder layers only: not a benchmark result" % dims["layers"]
    print(json.dumps(line), flush=True)
    pybert.unload_model(model)


def rank_plumbing(world, rank):
    """(barrier, allmax) for `world` ranks launched by torchrun: the ranks are independent replicas
    and meet only here, on the host (gloo): a barrier around the timed regions and a max-reduction
    of the per-rank device times.  One rank: no process group at all."""
    if world <= 1:
        return (lambda: None), (lambda x: float(x))
    import torch
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def barrier():
        dist.barrier()

    def allmax(x):
        t = torch.tensor([float(x)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return barrier, allmax


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=1, choices=sorted(synth.CONFIGS))
    ap.add_argument("--feed", default="raw", choices=["raw", "engine"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=0,
                    help="profiling only: run the first N encoder layers (the printed line is then not a "
                         "benchmark result and says so)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1 and "RANK" not in os.environ:
        # launched by hand without torchrun: start one process per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(args.gpus),
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 1000), os.path.abspath(__file__)]
        sys.exit(subprocess.call(cmd + sys.argv[1:]))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    barrier, allmax = rank_plumbing(world, rank)

    run_ours(args, rank, local_rank, world, barrier, allmax)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
