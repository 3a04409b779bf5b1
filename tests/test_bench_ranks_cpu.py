"""bench.py's multi-rank plumbing on CPU: two gloo ranks (the N > 1 mode is independent replicas, so
the ranks share only a host barrier and a max-reduction of their timings), the reference arm's
"rank 0 alone prints" rule, and the one-writer rule of the shared weight directory."""
import json
import os
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import json, os, sys, time
sys.path.insert(0, %(root)r)
import bench
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
barrier, allmax = bench.rank_plumbing(world, rank)
out = {"rank": rank, "max": allmax(10.0 + rank), "max_again": allmax(5.0 - rank)}
# one writer, everybody else waits for it behind the barrier
marker = os.path.join(%(tmp)r, "made_by")
if rank == 0:
    time.sleep(0.5)
    open(marker, "w").write("0")
barrier()
out["marker_seen"] = os.path.exists(marker)
barrier()
json.dump(out, open(os.path.join(%(tmp)r, "rank%%d.json" %% rank), "w"))
import torch.distributed as dist
dist.destroy_process_group()
"""


def test_two_gloo_ranks_barrier_and_max():
    with tempfile.TemporaryDirectory() as tmp:
        script = os.path.join(tmp, "worker.py")
        open(script, "w").write(WORKER % {"root": ROOT, "tmp": tmp})
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                            "--master-addr", "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300), script],
                           capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        res = [json.load(open(os.path.join(tmp, "rank%d.json" % k))) for k in range(2)]
    for k, o in enumerate(res):
        assert o["rank"] == k and o["max"] == 11.0 and o["max_again"] == 5.0 and o["marker_seen"]


def test_single_rank_needs_no_process_group():
    sys.path.insert(0, ROOT)
    import bench
    barrier, allmax = bench.rank_plumbing(1, 0)
    barrier()
    assert allmax(3.5) == 3.5


def test_reference_arm_other_ranks_print_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""
