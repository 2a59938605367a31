"""Times the fused peer reduction (all-reduce + residual add + RMSNorm in one launch) against NCCL all-reduce followed
by the add + RMSNorm kernel, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m mustafar_b200.peer_bench

Shape of the tensor-parallel decode step: rows = 32 sequences, hidden = 4096, 64 reductions per step (two per layer).
The fused arm replays one CUDA graph holding the 64 launches of a step; the NCCL arm launches its 64 all-reduces
eagerly (they are not captured) with the add + RMSNorm kernels in between.  CUDA events on the launching stream, the
maximum over ranks.  Per call every rank must receive (N - 1) * rows * hidden * 2 bytes over NVLink; the line printed
by rank 0 relates the measured time to that at 770 GB/s per direction (the peer-copy bandwidth measured on this pool).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import ops, step_ops
from .peer import PeerGroup
from .sharding import max_over_ranks

LINK_GBS = 770.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--calls", type=int, default=64, help="reductions per step (even)")
    ap.add_argument("--steps", type=int, default=50)
    a = ap.parse_args()
    import torch.distributed as dist
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # NCCL carries only barriers, scalar reductions and (in the NCCL arm) 256 KiB all-reduces here: in-switch
    # reduction buys nothing, and without multicast objects a rank that dies cannot disturb its peers' GPUs
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=dev)
    group = PeerGroup(dist, rank, world, dev, a.rows, a.hidden, a.calls)
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    part = (torch.randn(a.rows, a.hidden, generator=g, device=dev) * 0.01).half()
    group.slot(0).copy_(part)
    group.slot(1).copy_(part)
    w = torch.ones(a.hidden, dtype=torch.float16, device=dev)
    x = torch.zeros(a.rows, a.hidden, dtype=torch.float16, device=dev)
    out = torch.empty_like(x)

    def fused_step():
        for c in range(a.calls):
            group.reduce_add_rmsnorm(x, c, w, 1e-5, out=out)
        group.end_step()

    def nccl_step():
        for c in range(a.calls):
            y = part.clone()
            dist.all_reduce(y)
            step_ops.add_rmsnorm(x, y, w, 1e-5, out=out)

    def timed(fn, graph):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        run = fn
        if graph:
            cg = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                cg.capture_begin()
                fn()
                cg.capture_end()
            torch.cuda.current_stream().wait_stream(side)
            run = cg.replay
            run()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            run()
            x.zero_()
        e1.record()
        torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1), dist, dev) * 1e3 / (a.steps * a.calls)     # us per call

    fused_us = timed(fused_step, True)
    ops.check_device_status(dev)
    nccl_us = timed(nccl_step, False)
    link_bytes = (world - 1) * a.rows * a.hidden * 2
    if rank == 0:
        print(json.dumps({
            "kernel": "peer_reduce_rmsnorm_kernel", "n_gpus": world, "rows": a.rows, "hidden": a.hidden,
            "us_per_call_fused": round(fused_us, 2), "us_per_call_nccl_plus_add_rmsnorm": round(nccl_us, 2),
            "nvlink_bytes_in_per_rank_per_call": link_bytes,
            "link_bound_us_at_770GBps": round(link_bytes / (LINK_GBS * 1e3), 2),
            "achieved_over_link_bound": round(link_bytes / (LINK_GBS * 1e3) / fused_us, 3)}))
    group.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
