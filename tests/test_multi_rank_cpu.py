"""world_size-2 checks of the multi-rank plumbing on CPU (gloo): shard ranges partition the
units, timings reduce with MAX, and bench.py's reference arm prints exactly one line under torchrun."""
import json
import os
import subprocess
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from mustafar_b200.sharding import max_over_ranks, shard_range
    b, e = shard_range(13, world, rank)
    got = [None] * world
    dist.all_gather_object(got, (b, e))
    slow = max_over_ranks(1.0 + rank, dist)
    if rank == 0:
        out.put((got, slow))
    dist.barrier()
    dist.destroy_process_group()


def test_shards_partition_and_timings_take_the_max():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29641, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    ranges, slow = out.get()
    assert ranges == [(0, 7), (7, 13)]
    assert slow == 2.0


def test_shard_range_edges():
    from mustafar_b200.sharding import shard_range
    assert [shard_range(8, 8, r) for r in range(8)] == [(r, r + 1) for r in range(8)]
    assert shard_range(3, 4, 3) == (3, 3)               # more ranks than units: empty shard
    covered = sorted(i for r in range(5) for i in range(*shard_range(512, 5, r)))
    assert covered == list(range(512))


def test_reference_arm_prints_one_line_under_torchrun():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29642", os.path.join(ROOT, "bench.py"), "--gpus", "2", "--impl", "reference",
           "--steps", "2", "--warmup", "1", "--kv-len", "512"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["cpu_baseline"]["kind"] == "port"
    assert d["e2e"]["h2d_bytes_per_step"] == 0
