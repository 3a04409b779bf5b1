#!/usr/bin/env python
"""Throughput of the BERT-encoder hot path on B200: sequences/s on the BERT-large, seq 200,
batch 128 workload (the configuration the reference's README number is quoted on), with the
pooler followed by the Linear(1024 -> 2) + Softmax head.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one batch of 128 synthetic lines (valid lengths uniform in [16, 200], padded to
200) through the whole path.  Prints ONE JSON line:

  value      sequences/s with the batch already resident in HBM (device-side entry point),
             K steps timed with CUDA events on the replica's stream, max over ranks
  e2e        the same through the reference-facing call (Cuda_Classify: host arrays in,
             host probabilities out), copies inside the timed region
  roofline   achieved TFLOP/s of the tcgen05 GEMM kernel (the kernel that holds ~97 % of the
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

CFG = 1
WL = synth.CONFIGS[CFG]
METRIC = "BERT-large seq200 sequences/sec"
UNIT = "sequences/s"
WORKLOAD = ("C1: BERT-large (L24 H1024 h16 F4096) bf16 weights fp32 accumulate, batch 128, seq 200, "
            "valid lengths U[16,200] padded to 200, pooler + Linear(1024->2) + Softmax")


def flops_per_step(batch, seq, dims):
    """Executed FLOPs of one padded batch: per token per layer 24 H^2 dense + 4 S H attention,
    plus the pooler (2 H^2 per sequence)."""
    H, L = dims["hidden"], dims["layers"]
    dense = batch * seq * L * 24 * H * H
    attn = batch * seq * L * 4 * seq * H
    return dense, attn, batch * 2 * H * H


def gemm_flops(tokens, dims, sequences=None):
    """FLOPs the tensor-core GEMMs execute for `tokens` rows (QKV, attention-output, FFN1, FFN2 of
    every layer).  With the packed layout only the valid tokens of a batch are rows.  `sequences`:
    the pass returns the pooler output only, so the last layer computes its attention-output and FFN
    GEMMs for the first token of every sequence only (its QKV GEMM still takes every token)."""
    H, L, F = dims["hidden"], dims["layers"], dims["ffn"]
    full = 2 * tokens * (3 * H * H + H * H + 2 * H * F)
    if sequences is None or os.environ.get("CUDABERT_LAST_LAYER", "")[:1] == "f":
        return L * full
    return (L - 1) * full + 2 * tokens * 3 * H * H + 2 * sequences * (H * H + 2 * H * F)


def live_tokens(mask):
    """Rows the packed layout computes for a batch: per line 1 + index of its last valid position
    (a line with no valid position counts as the full padded length)."""
    S = mask.shape[1]
    last = np.where(mask.any(1), S - np.argmax(mask[:, ::-1] != 0, axis=1), S)
    return last


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(tensor=float(d.get("bf16_tflops_sustained", d.get("bf16_tflops"))), hbm=float(d["hbm_gbs"]),
                    burst=float(d.get("bf16_tflops", 0.0)) or None,
                    source="measured (MEASURED_PEAKS.json, sustained bf16)")
    return dict(tensor=1590.0, hbm=6650.0, burst=1590.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
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
                                          "--format=csv,noheader,nounits", "-lms", "200"],
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
                "power_w_max": max(power), "samples": len(sm)}


def make_batches(n_batches, rank):
    out = []
    for i in range(n_batches):
        out.append(synth.make_inputs(synth.input_seed(CFG) + 1000 * rank + i, WL["batch"], WL["seq"], WL["dist"]))
    return out


def weights_dir(rank_local, barrier):
    """Seeded synthetic BERT-large weights in the reference's .npy layout, written once per box."""
    d = os.path.join(tempfile.gettempdir(), "cudabert_bench_large_seed%d" % synth.weight_seed(CFG))
    done = d + ".complete"   # beside the directory: the reference's loader parses every file inside it
    if rank_local == 0 and not os.path.exists(done):
        synth.write_weight_dir(d, synth.make_weights(True, synth.weight_seed(CFG)))
        open(done, "w").close()
    barrier()
    return d


def reference_cuda_library(wdir, batch):
    """The reference's own CUDA library (fp32, cuBLAS), when oracle/_ref holds a build of it, on one
    batch of the workload on this GPU, in a process of its own: its sequences/s (host arrays in, pooler
    output out, like `e2e`) and its pooler output.  Reported beside the CPU baseline; never on the
    product path."""
    lib = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle", "_ref", "libcudaBERT_ref.so")
    if not os.path.exists(lib):
        return None
    tmp = tempfile.mkdtemp(prefix="cudabert_ref_")
    inp, out = os.path.join(tmp, "in.npz"), os.path.join(tmp, "out.npy")
    np.savez(inp, ids=batch[0], seg=batch[1], mask=batch[2])
    try:
        r = subprocess.run([sys.executable, os.path.join(os.path.dirname(lib), "..", "run_ref_cuda.py"), wdir, "1", inp,
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
def oracle_seq_per_s(n_seq, threads, repeats=1, weights=None):
    """Time the CPU oracle on n_seq sequences of the workload; returns (seq/s, seconds)."""
    import torch
    from oracle import bert_oracle
    torch.set_num_threads(threads)
    dims = synth.model_dims(True)
    if weights is None:
        weights = bert_oracle.Weights(synth.make_weights(True, synth.weight_seed(CFG)))
    ids, seg, mask = synth.make_inputs(synth.input_seed(CFG), n_seq, WL["seq"], WL["dist"])
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
    threads = os.cpu_count() or 1
    # size the per-step sample so that warmup + steps stay within about two minutes
    rate, dt, w = oracle_seq_per_s(2, threads)
    budget = 120.0 / max(args.steps + args.warmup, 1)
    n_seq = int(max(1, min(WL["batch"], rate * budget)))
    for _ in range(args.warmup):
        oracle_seq_per_s(n_seq, threads, weights=w)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle_seq_per_s(n_seq, threads, weights=w)
    total = time.perf_counter() - t0
    value = n_seq * args.steps / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample_sequences_per_step": n_seq},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "%d sequences of the workload per step (seq 200, lengths U[16,200]), fp32, "
                                   "torch CPU ops, %d threads" % (n_seq, threads)},
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
    dev = local_rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    dims = synth.model_dims(True)
    B, S = WL["batch"], WL["seq"]
    wdir = weights_dir(local_rank, barrier)
    n_pool = 4
    host = make_batches(n_pool, rank)
    ref_cuda = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.layers:
        ref_cuda = reference_cuda_library(wdir, host[0])   # before this process takes device memory
    t_load = time.perf_counter()
    model = pybert.load_model(True, wdir, dev, B, S, precision="bf16", num_layers=args.layers)
    load_seconds = time.perf_counter() - t_load   # .npy directory -> device-resident bf16 K-major weights
    if args.layers:
        dims = dict(dims, layers=min(args.layers, dims["layers"]))
    C = pybert.num_classes(model)
    stream = torch.cuda.ExternalStream(pybert.stream(model), device=dev)

    devb = [tuple(torch.from_numpy(a).to("cuda:%d" % dev) for a in hb) for hb in host]
    probs = np.zeros((B, C), np.float32)

    def step_dev(i):
        ids, seg, mask = devb[i % n_pool]
        rc = pybert.classify_dev(model, ids.data_ptr(), seg.data_ptr(), mask.data_ptr(), B, S)
        if rc:
            raise RuntimeError("forward failed: " + pybert.last_error(model))

    def step_e2e(i):
        ids, seg, mask = host[i % n_pool]
        pybert.classify(model, probs, ids, seg, B, S, C, mask)

    def timed(fn, steps, sync_after):
        barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        t_host = time.perf_counter()
        for i in range(steps):
            fn(i)
        timed.host_ms = (time.perf_counter() - t_host) * 1e3 / steps
        e1.record(stream)
        if sync_after:
            rc = pybert.sync(model)
            if rc:
                raise RuntimeError("sync failed: " + pybert.last_error(model))
        torch.cuda.synchronize(dev)
        barrier()
        return allmax(e0.elapsed_time(e1))

    for i in range(args.warmup):
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
    # end to end through the reference-facing call, host buffers in and out
    for i in range(min(args.warmup, 3)):
        step_e2e(i)
    ms_e2e = timed(step_e2e, args.steps, False)
    clocks = sampler.stop() if rank == 0 else None
    pybert.check(model)

    value = world * args.steps * B / (ms_total / 1e3)
    e2e_value = world * args.steps * B / (ms_e2e / 1e3)

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

    if rank != 0:
        pybert.unload_model(model)
        return
    peaks = load_peaks()
    gemm_ms = sum(prof[k][0] for k in prof if k.startswith("gemm"))
    gemm_n = sum(prof[k][1] for k in prof if k.startswith("gemm"))
    packed = os.environ.get("CUDABERT_PACK", "1") != "0"
    lens = [live_tokens(hb[2]) if packed else np.full(B, S) for hb in host]
    prof_lens = [lens[i % n_pool] for i in range(prof_steps)]
    gflops = sum(gemm_flops(int(l.sum()), dims, sequences=B) for l in prof_lens)
    attn_exec = sum(dims["layers"] * 4 * dims["hidden"] * float((l.astype(np.float64) ** 2).sum()) for l in prof_lens)
    ln_rows = sum(int(l.sum()) for l in prof_lens) / prof_steps
    achieved = gflops / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else 0.0
    dense, attn, pool = flops_per_step(B, S, dims)
    total_ms = sum(v[0] for v in prof.values())
    kernels = {k: {"ms_per_step": v[0] / prof_steps, "launches_per_step": v[1] / prof_steps,
                   "share": (v[0] / total_ms if total_ms else 0)} for k, v in prof.items()}
    attn_ms = prof["attention"][0]
    ln_ms, ln_n = prof["layernorm"]
    # LayerNorm: read fp16 dense output + fp32 residual, write the bf16 GEMM copy + the fp32 residual copy
    ln_bytes = ln_rows * dims["hidden"] * 12

    if ref_cuda and ref_cuda.get("pooled") is not None:
        # the reference's own fp32 pooler output for batch 0 against this library's bf16 mode, full size
        from oracle import bert_oracle
        ours = np.zeros((B, dims["hidden"]), np.float32)
        pybert.bert(model, ours, host[0][0], host[0][1], B, S, host[0][2])
        pybert.check(model)
        ref = ref_cuda.pop("pooled")
        # max |a - b| / max |b| (the measure the parity tests bound by 2e-2 on their cases) and the
        # relative Frobenius norm, over all 128 x 1024 pooler outputs of the batch
        ref_cuda["rel_err_of_this_library_bf16"] = float(bert_oracle.rel_err(ours, ref))
        ref_cuda["rel_fro_err_of_this_library_bf16"] = float(np.linalg.norm(ours - ref) / np.linalg.norm(ref))
    elif ref_cuda:
        ref_cuda.pop("pooled", None)

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        n_seq = 16
        rate, dt, _ = oracle_seq_per_s(n_seq, threads)
        cpu = {"value": rate, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": "%d sequences of the workload (seq 200, lengths U[16,200]) in one batch, fp32, "
                         "torch CPU ops, %.1f s" % (n_seq, dt)}
        if ref_cuda:
            cpu["reference_cuda_library_on_this_gpu"] = ref_cuda

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "host_enqueue_ms_per_step": host_enqueue_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch_per_gpu": B, "seq_len": S, "global_batch": B * world,
                   "parallelism": "replicas x%d (batch sharding, no collective)" % world,
                   "l2": "working set per step (577 MB of activations, 604 MB of weights) is larger than L2",
                   "tflops_per_step_padded": (dense + attn + pool) / 1e12,
                   "layout": ("packed: padding tokens are not computed (%.0f live of %d token slots per step)"
                              % (ln_rows, B * S)) if packed else "padded",
                   "last_layer": ("every token" if os.environ.get("CUDABERT_LAST_LAYER", "")[:1] == "f" else
                                  "attention-output, FFN and LayerNorm for the first token of each sequence "
                                  "only (all the pooler reads; same bits out as the full layer)"),
                   "tflops_per_step_executed_gemm": gflops / prof_steps / 1e12},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": 3 * B * S * 4, "d2h_bytes_per_step": B * C * 4 + 4},
        "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_pair_kernel (QKV, attention-output, FFN1, FFN2)",
                     "achieved": achieved, "peak": peaks["tensor"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["tensor"] if peaks["tensor"] else None, "peak_source": peaks["source"],
                     # the same against the measured burst figure and the nominal dense bf16 peak of the part
                     "frac_of_measured_burst": achieved / peaks["burst"] if peaks.get("burst") else None,
                     "frac_of_nominal_2250": achieved / 2250.0,
                     "launches": gemm_n / prof_steps, "avg_launch_ms": gemm_ms / gemm_n if gemm_n else None,
                     # mean DRAM bytes (read + write) per GEMM launch from the ncu capture summarised in
                     # profiles/gemm_tcgen05_c1_2layers.md (QKV 70, attention-output 32, FFN1 99, FFN2 139 MB)
                     "traffic": 85.0e6 if not args.layers else None, "traffic_unit": "bytes per launch (ncu, mean of the four GEMMs of a layer)"},
        "kernels": kernels,
        "attention_tflops": (attn_exec / (attn_ms / 1e3) / 1e12) if attn_ms else None,
        "layernorm_gbs": (ln_bytes * ln_n / (ln_ms / 1e3) / 1e9) if ln_ms else None,
        "weight_load_seconds": round(load_seconds, 3),
        "cpu_baseline": cpu,
    }
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
