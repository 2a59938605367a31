"""End-to-end decode benchmark of the Llama-3-8B-shaped model with the sparse KV cache.

    python -m mustafar_b200.e2e_llama [--batch 32] [--prompt 4096] [--new 256] [--parallel tp|dp]
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m mustafar_b200.e2e_llama --parallel tp

Random-init fp16 weights (seeded), uniformly random prompt ids, greedy decoding.  `tp` = 8-way
(or world-size-way) head tensor parallelism: the partial sums after o_proj and down_proj meet in a peer-buffer
reduction fused with the residual add + RMSNorm (`--tp-reduce fused`, the default) or in NCCL all-reduces (`nccl`);
`dp` = every rank runs the whole model on its own `--batch` sequences (no collective).
Prints one JSON line on rank 0: prefill time, time per output token and decode tokens/s of the
whole job, measured with CUDA events, maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .llama_shape import LlamaShape, SparseLlama
from .sharding import max_over_ranks


def _check_peer_reduction(peer, dist, dev) -> None:
    """One fused reduction on known data against NCCL's sum of the same partials, before the buffers are trusted with
    the timed run; raises ON EVERY RANK when any rank sees a disagreement or a wait that ran out (every rank walks
    through the same collectives whatever happens locally).  Leaves the group's step counter one step on."""
    from . import ops
    g = torch.Generator(device=dev).manual_seed(4242 + peer.rank)
    part = (torch.randn(peer.rows, peer.hidden, generator=g, device=dev) * 0.1).half()
    x = torch.ones(peer.rows, peer.hidden, dtype=torch.float16, device=dev)
    w = torch.ones(peer.hidden, dtype=torch.float16, device=dev)
    problem = None
    try:
        peer.slot(0).copy_(part)
        peer.reduce_add_rmsnorm(x, 0, w, 1e-5)
        peer.end_step()
    except Exception as e:
        problem = e
    total = part.float()
    dist.all_reduce(total)
    torch.cuda.synchronize()
    if problem is None:
        try:
            ops.check_device_status(dev)
            err = float((x.float() - (1.0 + total)).abs().max())
            if not err < 2e-2:      # fp16 rounding of 1 + sum of `world` partials of size ~0.1
                raise RuntimeError(f"peer reduction disagrees with NCCL (max abs error {err})")
        except Exception as e:
            problem = e
    bad = torch.tensor([0.0 if problem is None else 1.0], device=dev)
    dist.all_reduce(bad, op=dist.ReduceOp.MAX)
    if float(bad) != 0.0:
        raise RuntimeError(f"peer reduction self-check failed ({problem or 'on another rank'})")


def run_e2e(dev, rank: int, world: int, dist, batch: int = 32, prompt: int = 4096, new: int = 256,
            parallel: str = "dp", sparsity: float = 0.7, layers: int = 32, graph: bool = True, dense: bool = False,
            bits: int = 16, prune_mode: str = "block", tp_reduce: str = "fused", lm_head: str = "parallel", warm_up: bool = True) -> dict:
    """One generation (prefill + ``new`` greedy steps) on this rank's GPU; returns the result record (the same on
    every rank: times are the maximum over ranks).  ``dist``: an initialised torch.distributed module or None.
    ``tp_reduce``: "fused" = peer-buffer reduction fused with the RMSNorm, whole step one CUDA graph; "nccl" = NCCL
    all-reduces between graphs (also what "fused" falls back to when the peer mapping cannot be set up).
    ``lm_head``: "parallel" = with the fused reduction every rank keeps its slice of the vocabulary and the next token
    comes out of the peer arg-max exchange; "replicated" = every rank computes all logits."""
    tp = world if parallel == "tp" else 1
    shape = LlamaShape(n_layers=layers)
    kw = dict(sparsity=sparsity, seed=1234, tp_rank=rank if tp > 1 else 0, tp_world=tp, dist=dist, sparse=not dense,
              cache_bits=bits, prune_mode=prune_mode)
    reduce_used = "none"
    if tp > 1:
        reduce_used = "nccl"
        ok = torch.zeros(1, device=dev)
        model = None
        if tp_reduce == "fused" and not dense:
            try:
                model = SparseLlama(shape, batch, prompt + new, dev, tp_fused=True,
                                    lm_head_parallel=(lm_head == "parallel"), **kw)
                _check_peer_reduction(model.peer, dist, dev)
                ok += 1
            except Exception as e:      # e.g. CUDA IPC not permitted between the ranks' containers
                if rank == 0:
                    print(f"peer-buffer reduction unavailable ({type(e).__name__}: {e}); using NCCL", flush=True)
                model = None
            dist.all_reduce(ok)          # all ranks or none
            if int(ok.item()) == world:
                reduce_used = "fused peer buffers"
            else:
                model = None
        if model is None:
            torch.cuda.empty_cache()
            model = SparseLlama(shape, batch, prompt + new, dev, **kw)
    else:
        model = SparseLlama(shape, batch, prompt + new, dev, **kw)
    if warm_up:      # what a serving process does at start-up: the step graph is captured before the timed generation
        model.warm_up(graph)
    g = torch.Generator(device=dev).manual_seed(99 if tp > 1 else 99 + rank)
    toks = torch.randint(0, shape.vocab, (batch, prompt), generator=g, device=dev)

    def sync():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    sync()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    e[0].record()
    nxt = model.prefill_next(toks)
    e[1].record()
    marks = []
    for _ in range(new - 1):
        nxt = model.decode_next(nxt, graph=graph)
        marks.append(torch.cuda.Event(enable_timing=True))
        marks[-1].record()
    e[2].record()
    torch.cuda.synchronize()
    # device-reported errors (a wait that ran out, corrupt metadata): every rank learns of them, so that all raise together
    from . import ops
    flagged = ops._dev_status(dev).to(torch.float32).clone()
    if dist is not None:
        dist.all_reduce(flagged, op=dist.ReduceOp.MAX)
    if float(flagged) != 0.0:
        ops.check_device_status(dev)
        raise RuntimeError("another rank reported a device error during the generation")
    # per-step device time: the median leaves out the steps that append a block or capture the graph
    raw_gaps = [x.elapsed_time(y) for x, y in zip(marks[:-1], marks[1:])]
    slowest_at = (max(range(len(raw_gaps)), key=raw_gaps.__getitem__) + 1) if raw_gaps else -1   # 0-based decode step
    gaps = sorted(raw_gaps)
    steady_ms = max_over_ranks(gaps[len(gaps) // 2], dist, dev) if gaps else 0.0
    slowest_ms = max_over_ranks(gaps[-1], dist, dev) if gaps else 0.0
    prefill_ms = max_over_ranks(e[0].elapsed_time(e[1]), dist, dev)
    decode_ms = max_over_ranks(e[1].elapsed_time(e[2]), dist, dev)
    compress_ms = max_over_ranks(model.prefill_compress_ms, dist, dev)
    seqs = batch * (1 if tp > 1 else world)
    lm_head_used = "vocabulary-parallel" if getattr(model, "vocab_parallel", False) else "replicated"
    # bytes the compressed part of the cache takes per (token, kv head), K + V, measured on the first layer of this rank
    cache_bytes = None
    if not dense and model.compressed:
        L0 = model.layers[0]
        per = 0.0
        for st in (L0.ks, L0.vs):
            tiles = 2 * model.compressed
            if bits == 16:
                per += 8 * tiles + 4 * (tiles + 1) + 2.0 * float(st.packed_lengths().float().mean())
            else:
                per += (8 + 4 + 2 + 2) * tiles + 4.0 * float(st.head_tail.float().mean())
        cache_bytes = per / model.compressed
    if getattr(model, "peer", None) is not None:
        model.peer.close()
    del model
    torch.cuda.empty_cache()
    return {
        "metric": "llama3_8b_shape_decode_throughput", "unit": "tok/s", "n_gpus": world,
        "value": seqs * (new - 1) / (decode_ms * 1e-3), "tpot_ms": decode_ms / (new - 1), "tpot_median_ms": steady_ms,
        "slowest_step_ms": slowest_ms, "slowest_step_index": slowest_at, "ttft_ms": prefill_ms, "ttft_compression_ms": compress_ms,
        "compressed_cache_bytes_per_token_per_kv_head": cache_bytes, "dense_fp16_bytes_per_token_per_kv_head": 512,
        "config": {"workload": f"Llama-3-8B shape, {layers} layers, prompt {prompt}, {new} new tokens, "
                               f"batch {batch} per {'job' if tp > 1 else 'GPU'}, sparsity {sparsity}, window 128, "
                               f"pruning per {prune_mode}",
                   "parallelism": f"tp{tp}" if tp > 1 else f"dp{world}", "partial_sum_reduction": reduce_used,
                   "lm_head": lm_head_used,
                   "warm_up": "one short generation first (step graph captured there)" if warm_up else "none",
                   "cache": "dense-pruned torch" if dense else ("sparse fp16" if bits == 16 else f"sparse {bits}-bit"),
                   "cuda_graph": (False if (not graph or dense) else
                                  ("one graph per stretch between collectives" if reduce_used == "nccl" else True))},
        "data": "synthetic (random-init weights, random prompt ids)", "dtype": "f16"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=4096)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--parallel", default="dp", choices=["tp", "dp"])
    ap.add_argument("--sparsity", type=float, default=0.7)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--no-graph", action="store_true", help="launch every decode step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--dense", action="store_true", help="dense pruned cache + torch attention (comparison arm)")
    ap.add_argument("--bits", type=int, default=16, choices=[16, 4, 2],
                    help="16: pruned values kept as fp16; 4 / 2: quantised per tile")
    ap.add_argument("--tp-reduce", default="fused", choices=["fused", "nccl"],
                    help="tensor parallel only: partial sums through the fused peer-buffer kernel or through NCCL")
    ap.add_argument("--lm-head", default="parallel", choices=["parallel", "replicated"],
                    help="tensor parallel with the fused reduction only: split the lm_head over the vocabulary")
    ap.add_argument("--no-warm-up", action="store_true",
                    help="time the first generation of the process (pays library start-up and the graph capture)")
    ap.add_argument("--prune-mode", default="block", choices=["block", "step"],
                    help="block: prune with the compression, 256 tokens at a time; step: prune the token that leaves "
                         "the residual window at every decode step")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        # NCCL carries only barriers, scalar reductions and (in the NCCL arm) 256 KiB all-reduces here: in-switch
        # reduction buys nothing, and without multicast objects a rank that dies cannot disturb its peers' GPUs
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    res = run_e2e(dev, rank, world, dist, a.batch, a.prompt, a.new, a.parallel, a.sparsity, a.layers, not a.no_graph,
                  a.dense, a.bits, a.prune_mode, a.tp_reduce, a.lm_head, not a.no_warm_up)
    if rank == 0:
        print(json.dumps(res))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
