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


@pytest.mark.parametrize("graph", [False, True])
def test_per_step_pruning_matches_dense_model_pruned_per_step(graph):
    """prune_mode="step": the token leaving the 128 most recent ones is pruned in the window at every step (what the
    reference's torch path does, models/llama_mustafar_Kt_Mag_Vt_Mag.py:917-926); the dense comparison model prunes
    the same token at the same step.  Crosses a 256-token append, eager and as a replayed CUDA graph."""
    from mustafar_b200.llama_shape import SparseLlama, tiny_shape
    shape, B, prompt, steps = tiny_shape(), 2, 256 + 128 + 220, 50
    kw = dict(batch=B, max_tokens=1024, device="cuda", sparsity=0.7, residual=128, seed=3, prune_mode="step")
    sparse = SparseLlama(shape, sparse=True, **kw)
    dense = SparseLlama(shape, sparse=False, **kw)
    block = SparseLlama(shape, sparse=True, **{**kw, "prune_mode": "block"})
    toks = torch.randint(0, shape.vocab, (B, prompt), generator=torch.Generator(device="cuda").manual_seed(1), device="cuda")
    ls, ld, lb = sparse.prefill(toks), dense.prefill(toks), block.prefill(toks)
    assert oracle.rel_l2(ls.float().cpu(), ld.float().cpu()) < 5e-3
    differs = 0.0
    for i in range(steps):
        nxt = ld.argmax(-1)
        ls, ld, lb = sparse.decode_step(nxt, graph=graph).clone(), dense.decode_step(nxt), block.decode_step(nxt)
        assert oracle.rel_l2(ls.float().cpu(), ld.float().cpu()) < 5e-3, i
        differs = max(differs, oracle.rel_l2(ls.float().cpu(), lb.float().cpu()))
    assert sparse.compressed == 512 and sparse.wlen == dense.wlen
    assert differs > 1e-3          # pruning the window tokens early is a different computation from block mode
    from mustafar_b200 import ops
    ops.check_device_status()
    # behind the 128 most recent tokens (and the one the next step will prune first) every window row is pruned:
    # at most 40 + ties nonzeros of 128
    w = sparse.wlen
    nnz = (sparse.layers[0].kwin[:, :w - 129] != 0).sum(-1)
    assert int(nnz.max()) <= 44 and int((sparse.layers[0].kwin[:, w - 129:w] != 0).sum(-1).min()) > 100


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


@pytest.mark.parametrize("bits", [2, 4])
def test_quantised_cache_model_matches_dense_model_with_dequantised_cache(bits):
    """The quantised cache end to end: after the prefill the dense comparison model gets its compressed tokens
    replaced by what the oracle's quantise -> dequantise gives for them; the decode steps of both models then agree."""
    from mustafar_b200.llama_shape import SparseLlama, tiny_shape
    shape, B, prompt = tiny_shape(), 2, 256 + 128 + 40
    toks = torch.randint(0, shape.vocab, (B, prompt), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    qm = SparseLlama(shape, B, 1024, "cuda", seed=3, cache_bits=bits)
    dm = SparseLlama(shape, B, 1024, "cuda", seed=3, sparse=False)
    lq, ld = qm.prefill(toks), dm.prefill(toks)
    assert qm.compressed == 256 == dm.compressed
    for L in dm.layers:
        k = L.ks[:, :256].cpu()
        v = L.vs[:, :256].cpu()
        kf = oracle.quant_format.quant_compress_key_ref(k, bits, 64)
        vf = oracle.quant_format.quant_compress_value_ref(v, bits, 64)
        L.ks[:, :256] = torch.as_tensor(oracle.quant_format.dequant_key_ref(kf, 256, 128, bits, 64)).cuda()
        L.vs[:, :256] = torch.as_tensor(oracle.quant_format.dequant_value_ref(vf, 256, 128, bits, 64)).cuda()
    nxt = ld.argmax(-1)
    for i in range(6):
        lq, ld = qm.decode_step(nxt, graph=True).clone(), dm.decode_step(nxt)   # first step eager, then replayed graphs
        assert oracle.rel_l2(lq.float().cpu(), ld.float().cpu()) < 5e-3, i
        nxt = ld.argmax(-1)


@pytest.mark.parametrize("bits", [16, 2])
def test_second_generation_after_reset_replays_the_graph_and_matches_a_fresh_model(bits):
    """warm_up() runs a throw-away generation (capturing the step graph) and resets; the generation after it must give
    what a fresh model gives, across a block append, without capturing again."""
    from mustafar_b200.llama_shape import SparseLlama, tiny_shape
    shape, B, prompt = tiny_shape(), 2, 256 + 128 + 250
    toks = torch.randint(0, shape.vocab, (B, prompt), device="cuda", generator=torch.Generator(device="cuda").manual_seed(6))
    fresh = SparseLlama(shape, B, 1024, "cuda", seed=4, cache_bits=bits)
    want = fresh.generate(toks, 12, graph=False)
    m = SparseLlama(shape, B, 1024, "cuda", seed=4, cache_bits=bits)
    m.warm_up(graph=True)
    assert m.tokens == 0 and m._graph is not None
    captured = m._graph
    got = m.generate(toks, 12, graph=True)
    assert m._graph is captured
    assert torch.equal(got, want)
    assert m.compressed == 512
    from mustafar_b200 import ops
    ops.check_device_status()
