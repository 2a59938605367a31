"""Host-side bookkeeping of the peer reduction (no GPU): epochs grow by one from call to call across step boundaries,
consecutive calls never share a partial buffer, and the handle exchange PeerGroup relies on (all_gather_object of 64-byte
handles, every rank seeing every rank's in rank order) works over gloo with two ranks."""
import os
import subprocess
import sys

import pytest

from mustafar_b200 import peer


def test_epochs_are_consecutive_and_slots_alternate():
    calls = 64                               # two reductions per layer, 32 layers
    seq = [(s, c) for s in range(3) for c in range(calls)]
    epochs = [peer.epoch_of(s, calls, c) for s, c in seq]
    assert epochs == list(range(1, len(seq) + 1))
    slots = [peer.slot_of(c) for _, c in seq]
    assert all(a != b for a, b in zip(slots, slots[1:]))


def test_odd_call_count_is_refused_before_anything_is_allocated():
    with pytest.raises(RuntimeError, match="even"):
        peer.PeerGroup(None, 0, 2, "cpu", 4, 64, calls_per_step=3)
    with pytest.raises(RuntimeError, match="at most"):
        peer.PeerGroup(None, 0, 9, "cpu", 4, 64, calls_per_step=2)


WORKER = r"""
import os, sys
import torch.distributed as dist
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
mine = bytes([rank + 1]) * 64
got = [None] * world
dist.all_gather_object(got, mine)
assert got == [bytes([r + 1]) * 64 for r in range(world)], got
dist.barrier()
if rank == 0:
    print("HANDLES_OK", flush=True)
dist.destroy_process_group()
"""


def test_handle_exchange_over_gloo(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29664", str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env=dict(os.environ))
    assert r.returncode == 0, (r.stdout[-800:], r.stderr[-1500:])
    assert "HANDLES_OK" in r.stdout
