"""Seeded random configurations of the whole path against the CPU oracle: prune + compress bit-exact (including
inputs with many equal magnitudes, where the tie rule decides), then the fused decode attention within 2e-3.
The fixed grids of the other test files pick the shapes the reference uses; this one walks in between them:
odd head counts, every group size, ragged windows, empty caches, several appends per cache."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _cases(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        out.append(dict(
            Bh=int(rng.integers(1, 7)), G=int(rng.choice([1, 2, 4, 8])), blocks=int(rng.integers(0, 17)),
            W=int(rng.choice([0, 1, 63, 64, 65, 128, 200])), sparsity=float(rng.choice([0.0, 0.5, 0.7, 0.9])),
            ties=bool(rng.integers(0, 2)), appends=int(rng.integers(1, 4)), seed=1000 + i))
    return out


@pytest.mark.parametrize("c", _cases(24, 7), ids=lambda c: "Bh{Bh}-G{G}-b{blocks}-W{W}-s{sparsity}-t{ties:d}-a{appends}".format(**c))
def test_random_configuration(c):
    from mustafar_b200 import compression as comp, ops
    Bh, G, L, W, s = c["Bh"], c["G"], 64 * c["blocks"], c["W"], c["sparsity"]
    if L == 0 and W == 0:
        W = 5
    k, v = oracle.make_kv(Bh, max(L + W, 64), seed=c["seed"])
    if c["ties"]:                      # few distinct magnitudes: thresholds land on ties all the time
        k, v = (k * 2).round() / 2, (v * 2).round() / 2
    kc, vc = k[:, :L].contiguous(), v[:, :L].contiguous()
    kw, vw = k[:, L:L + W].contiguous(), v[:, L:L + W].contiguous()
    ks = comp.SparseStore(Bh, max(L, 64), comp.KEY, "cuda")
    vs = comp.SparseStore(Bh, max(L, 64), comp.VALUE, "cuda")
    # the cache is built in `appends` pieces (multiples of 64 tokens): must equal compressing it in one go
    cuts = sorted(set([0, L] + [64 * int(x) for x in np.linspace(0, L // 64, c["appends"] + 1)[1:-1]]))
    for a, b in zip(cuts[:-1], cuts[1:]):
        if b > a:
            ks.append(kc[:, a:b].cuda(), comp.keep_rank(s))
            vs.append(vc[:, a:b].cuda(), comp.keep_rank(s))
    ks.check(); vs.check()
    kp = oracle.prune_ref(kc, s) if L else kc
    vp = oracle.prune_ref(vc, s) if L else vc
    if L:
        for store, ref in ((ks, oracle.compress_key_ref(kp)), (vs, oracle.compress_value_ref(vp))):
            wb, wa, wp = ref
            T = 2 * L
            assert np.array_equal(store.bitmaps[:, :T].cpu().numpy(), wb[:, :T])
            assert np.array_equal(store.accum[:, :T + 1].cpu().numpy(), wa[:, :T + 1])
            for h in range(Bh):
                assert np.array_equal(store.nz[h, :len(wp[h])].cpu().numpy().view(np.uint16), wp[h].view(np.uint16))
    q = oracle.make_query(Bh * G, seed=c["seed"] + 1)
    out = ops.decode_attention(q.cuda(), ks, vs, kw.cuda() if W else None, vw.cuda() if W else None, G)
    want = oracle.decode_attention_ref(q, kp, vp, kw, vw, G)
    ops.check_device_status()
    assert oracle.rel_l2(out.float().cpu(), want) < TOL


def _quant_cases(n, seed):
    rng = np.random.default_rng(seed)
    return [dict(Bh=int(rng.integers(1, 5)), G=int(rng.choice([1, 2, 4, 8])), blocks=int(rng.integers(1, 9)),
                 W=int(rng.choice([0, 1, 64, 130])), sparsity=float(rng.choice([0.5, 0.7, 0.9])),
                 bits=int(rng.choice([2, 2, 4])), group=int(rng.choice([64, 64, 32])), seed=2000 + i) for i in range(n)]


@pytest.mark.parametrize("c", _quant_cases(14, 9),
                         ids=lambda c: "Bh{Bh}-G{G}-b{blocks}-W{W}-s{sparsity}-{bits}bit-g{group}".format(**c))
def test_random_quantised_configuration(c):
    """Quantised cache: the compressor's arrays bit-exact against the oracle (2-bit per tile is the pinned format; 4-bit
    and groups of 32 are checked against the oracle's restatement only), then the fused decode within 2e-3 of dense
    attention over the oracle-dequantised tensors."""
    from mustafar_b200 import compression as comp, compression_quant as cq, ops, ops_quant
    Bh, G, L, W, s, bits, group = c["Bh"], c["G"], 64 * c["blocks"], c["W"], c["sparsity"], c["bits"], c["group"]
    k, v = oracle.make_kv(Bh, L + max(W, 1), seed=c["seed"])
    kc, vc = k[:, :L].contiguous(), v[:, :L].contiguous()
    kw, vw = k[:, L:L + W].contiguous(), v[:, L:L + W].contiguous()
    kp, vp = oracle.prune_ref(kc, s), oracle.prune_ref(vc, s)
    kq = cq.compress_quant(kc.cuda(), comp.KEY, comp.keep_rank(s), bits, group)
    vq = cq.compress_quant(vc.cuda(), comp.VALUE, comp.keep_rank(s), bits, group)
    wk = oracle.quant_compress_key_ref(kp, bits=bits, group=group)
    wv = oracle.quant_compress_value_ref(vp, bits=bits, group=group)
    for got, want in ((kq, wk), (vq, wv)):
        for key in ("bitmaps", "tile_offsets", "counts", "units", "packed"):
            assert np.array_equal(got[key].cpu().numpy(), want[key]), key
        for key in ("scales", "zeros"):
            assert np.array_equal(np.ascontiguousarray(got[key].cpu().numpy()).view(np.uint16),
                                  np.ascontiguousarray(want[key]).view(np.uint16)), key
    kd = oracle.dequant_key_ref(wk, L, bits=bits, group=group)
    vd = oracle.dequant_value_ref(wv, L, bits=bits, group=group)
    q = oracle.make_query(Bh * G, seed=c["seed"] + 1)
    out = ops_quant.decode_attention_quant(q.cuda(), kq, vq, L, kw.cuda() if W else None, vw.cuda() if W else None, G, bits)
    ops.check_device_status()
    assert oracle.rel_l2(out.float().cpu(), oracle.decode_attention_ref(q, kd, vd, kw, vw, G)) < TOL
