"""Worker of test_gpu_tensor_parallel.py::test_peer_wait_runs_out_when_a_rank_stays_silent (two ranks, one per GPU).

Rank 1 skips one reduction on purpose (it launches nothing: the failure is made on the host, no kernel faults or
hangs); rank 0's kernel waits its bound, sets the time-out bit and leaves its inputs untouched.  The next reduction,
which both ranks issue, succeeds on the same buffers: the context and the group stay usable."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mustafar_b200 import _lib, ops  # noqa: E402
from mustafar_b200.peer import PeerGroup  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rows, hidden = 4, 512
    group = PeerGroup(dist, rank, world, dev, rows, hidden, calls_per_step=4, wait_ms=300.0)
    w = torch.ones(hidden, dtype=torch.float16, device=dev)
    x = torch.full((rows, hidden), 1.0, dtype=torch.float16, device=dev)
    group.slot(0).fill_(0.25 * (rank + 1))
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:                      # rank 1 stays silent for call 0
        out = group.reduce_add_rmsnorm(x, 0, w, 1e-5)
        torch.cuda.synchronize()
        timed_out = False
        try:
            ops.check_device_status(dev)
        except _lib.MustafarError as e:
            timed_out = "time" in str(e).lower() or "wait" in str(e).lower()
        assert timed_out, "the silent peer was not noticed"
        assert float((x - 1.0).abs().max()) == 0.0       # nothing was added
    dist.barrier()
    # call 1: everybody takes part
    group.slot(1).fill_(0.5 * (rank + 1))
    torch.cuda.synchronize()
    dist.barrier()
    out = group.reduce_add_rmsnorm(x, 1, w, 1e-5)
    torch.cuda.synchronize()
    ops.check_device_status(dev)
    want = 1.0 + 0.5 * sum(r + 1 for r in range(world))
    assert float((x.float() - want).abs().max()) < 1e-2, float(x[0, 0])
    assert float((out.float() - 1.0).abs().max()) < 1e-2     # a constant row normalises to 1
    if rank == 0:
        print("PEER_TIMEOUT_OK", flush=True)
    group.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
