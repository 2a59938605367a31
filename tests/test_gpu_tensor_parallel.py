"""Head tensor parallelism of the model glue (partial sums after o_proj / down_proj meet in NCCL all-reduces, or in
the peer-buffer reduction fused with the RMSNorm): needs two GPUs; skipped on a single-GPU box.  The ranks are child
processes started by torch.distributed.run; NVLS is switched off for NCCL and the fused kernel uses plain peer loads."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("fused", ["0", "1"])
@pytest.mark.parametrize("graph", ["0", "1"])
def test_tp2_matches_single_gpu(graph, fused):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TP_WORKER_GRAPH=graph, TP_WORKER_FUSED=fused)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29661", os.path.join(HERE, "tp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    assert "TP_WORST_REL_L2" in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("graph", ["0", "1"])
def test_tp2_vocabulary_parallel_lm_head(graph):
    """Every rank keeps half of the lm_head; the gathered logits match the single-GPU model and the token the peer
    arg-max exchange picks is a maximum of them, the same on both ranks."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TP_WORKER_GRAPH=graph, TP_WORKER_FUSED="1", TP_WORKER_LMHEAD="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29662", os.path.join(HERE, "tp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    assert "TP_WORST_REL_L2" in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_peer_wait_runs_out_when_a_rank_stays_silent():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29663", os.path.join(HERE, "peer_timeout_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    assert "PEER_TIMEOUT_OK" in r.stdout
