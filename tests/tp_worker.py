"""Worker of test_gpu_tensor_parallel.py (launched by torch.distributed.run, one rank per GPU):
the head-tensor-parallel model must reproduce the single-GPU logits."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mustafar_b200.llama_shape import SparseLlama, tiny_shape  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    shape, B, prompt = tiny_shape(), 2, 256 + 128 + 100
    if os.environ.get("TP_WORKER_LMHEAD", "0") == "1":
        shape.vocab = 1024          # a slice per rank that is a multiple of 8 logits
    toks = torch.randint(0, shape.vocab, (B, prompt), device="cuda", generator=torch.Generator(device="cuda").manual_seed(7))
    fused = os.environ.get("TP_WORKER_FUSED", "0") == "1"   # peer-buffer reduction fused with the RMSNorm instead of NCCL
    split_vocab = os.environ.get("TP_WORKER_LMHEAD", "0") == "1"   # vocabulary-parallel lm_head + peer arg-max exchange
    tp = SparseLlama(shape, B, 1024, "cuda", seed=11, tp_rank=rank, tp_world=world, dist=dist, tp_fused=fused,
                     lm_head_parallel=split_vocab)
    assert (tp.peer is not None) == fused and tp.vocab_parallel == (split_vocab and fused)

    def full_logits(local):
        """all ranks' slices side by side (NCCL, outside any graph): what a replicated lm_head would have produced"""
        if not tp.vocab_parallel:
            return local
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local.contiguous())
        return torch.cat(parts, dim=-1)

    def check_token(tok, logits):
        """the exchanged arg-max is a maximum of the gathered logits, and every rank holds the same ids"""
        if not tp.vocab_parallel:
            return
        picked = logits.gather(1, tok.view(-1, 1)).squeeze(1)
        assert torch.equal(picked, logits.max(dim=-1).values), (tok, logits.argmax(-1))
        same = tok.clone()
        dist.broadcast(same, 0)
        assert torch.equal(same, tok)

    if tp.vocab_parallel:
        tok0 = tp.prefill_next(toks)
        lt = full_logits(tp._logits_last)
        check_token(tok0, lt)
    else:
        lt = tp.prefill(toks)
    ref = SparseLlama(shape, B, 1024, "cuda", seed=11) if rank == 0 else None
    lr = ref.prefill(toks) if rank == 0 else None
    worst = 0.0
    use_graph = os.environ.get("TP_WORKER_GRAPH", "0") == "1"
    for i in range(12):
        nxt = lt.argmax(-1)
        dist.broadcast(nxt, 0)
        # graph: one CUDA graph per stretch between two collectives, the all-reduces launched eagerly in between
        if tp.vocab_parallel:
            tok = tp.decode_next(nxt, graph=use_graph)
            lt = full_logits(tp._step_out)
            check_token(tok, lt)
        else:
            lt = tp.decode_step(nxt, graph=use_graph)
        if rank == 0:
            lr = ref.decode_step(nxt)
            err = float(torch.linalg.norm(lt.float() - lr.float()) / torch.linalg.norm(lr.float()))
            worst = max(worst, err)
    from mustafar_b200 import ops
    ops.check_device_status()
    if rank == 0:
        print("TP_WORST_REL_L2", worst, flush=True)
        assert worst < 5e-3, worst
    if tp.peer is not None:
        tp.peer.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
