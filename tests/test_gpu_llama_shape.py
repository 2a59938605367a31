"""The patched model glue (sparse cache + fused decode attention) against the same model with a
dense cache of pruned tokens and plain torch attention (what the reference's torch accuracy path
computes, models/llama_mustafar_Kt_Mag_Vt_Mag.py:873-974), teacher-forced over a run that crosses
a 256-token block append."""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def test_sparse_model_matches_dense_pruned_model():
    from mustafar_b200.llama_shape import SparseLlama, tiny_shape
    shape, B, prompt, steps = tiny_shape(), 2, 256 + 128 + 200, 64
    kw = dict(batch=B, max_tokens=1024, device="cuda", sparsity=0.7, residual=128, seed=3)
    sparse = SparseLlama(shape, sparse=True, **kw)
    dense = SparseLlama(shape, sparse=False, **kw)
    g = torch.Generator(device="cuda").manual_seed(1)
    toks = torch.randint(0, shape.vocab, (B, prompt), generator=g, device="cuda")
    ls, ld = sparse.prefill(toks), dense.prefill(toks)
    assert sparse.compressed == 256 and sparse.wlen == prompt - 256
    assert oracle.rel_l2(ls.float().cpu(), ld.float().cpu()) < 5e-3
    appended = False
    for i in range(steps):
        nxt = ld.argmax(-1)                       # both models are fed the dense model's choice
        ls, ld = sparse.decode_step(nxt), dense.decode_step(nxt)
        assert oracle.rel_l2(ls.float().cpu(), ld.float().cpu()) < 5e-3, i
        appended |= sparse.compressed == 512
    assert appended and sparse.wlen == dense.wlen and sparse.tokens == prompt + steps
    for L in sparse.layers:
        L.ks.check(); L.vs.check()


def test_graph_replay_matches_eager_steps():
    """Replaying the captured step (device-resident position / window length) gives the eager logits,
    across a block append that forces a re-capture."""
    from mustafar_b200.llama_shape import SparseLlama, tiny_shape
    shape, B, prompt = tiny_shape(), 2, 256 + 128 + 240
    kw = dict(batch=B, max_tokens=1024, device="cuda", seed=5)
    a, b = SparseLlama(shape, **kw), SparseLlama(shape, **kw)
    toks = torch.randint(0, shape.vocab, (B, prompt), device="cuda", generator=torch.Generator(device="cuda").manual_seed(4))
    la, lb = a.prefill(toks), b.prefill(toks)
    for i in range(40):
        nxt = la.argmax(-1)
        la, lb = a.decode_step(nxt), b.decode_step(nxt, graph=True).clone()
        assert oracle.rel_l2(lb.float().cpu(), la.float().cpu()) < 1e-3, i
    assert a.compressed == b.compressed == 512 and a.wlen == b.wlen


def test_generate_runs_and_is_deterministic():
    from mustafar_b200.llama_shape import SparseLlama, tiny_shape
    shape = tiny_shape()
    toks = torch.randint(0, shape.vocab, (1, 300), device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    a = SparseLlama(shape, 1, 512, "cuda", seed=9).generate(toks, 8)
    b = SparseLlama(shape, 1, 512, "cuda", seed=9).generate(toks, 8)
    assert a.shape == (1, 8) and torch.equal(a, b)
