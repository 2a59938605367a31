"""GPU parity of the decode kernels against the CPU oracle.

Tolerance: 2e-3 relative L2 (fp16 storage, fp32 accumulation), the bound the
north-star states for attention outputs."""
import math

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3


@pytest.fixture(scope="module")
def m():
    import os
    os.environ["MUSTAFAR_B200_CHECK"] = "1"
    from mustafar_b200 import compression, ops

    class M:
        pass
    M.c, M.o = compression, ops
    return M


def build_cache(m, Bh, L, sparsity, seed):
    k, v = oracle.make_kv(Bh, max(L, 64), seed=seed)
    k, v = k[:, :L], v[:, :L]
    kp = oracle.prune_ref(k, sparsity) if L else k
    vp = oracle.prune_ref(v, sparsity) if L else v
    ks = m.c.SparseStore(Bh, max(L, 64), m.c.KEY, "cuda")
    vs = m.c.SparseStore(Bh, max(L, 64), m.c.VALUE, "cuda")
    if L:
        ks.append(k.cuda().contiguous(), m.c.keep_rank(sparsity))
        vs.append(v.cuda().contiguous(), m.c.keep_rank(sparsity))
    return kp, vp, ks, vs


def reference_layout(store):
    """The tensors the reference model hands to its ops: compact bitmaps / accum, packed
    values of all heads concatenated, NZ_Offset in uint4 units
    (models/llama_mustafar_kernel.py:395, :546-548)."""
    T = store.tiles
    lens = store.packed_lengths().tolist()
    bmp = store.bitmaps[:, :T].contiguous()
    idx = store.accum[:, :T + 1].contiguous()
    nz = torch.cat([store.nz[h, :lens[h]] for h in range(store.n_heads)])
    off = torch.zeros(store.n_heads, dtype=torch.int32, device="cuda")
    for i in range(1, store.n_heads):
        off[i] = off[i - 1] + idx[i - 1][-1] // 4
    return bmp, nz, idx, off


@pytest.mark.parametrize("G,Bh,L", [(1, 3, 256), (4, 2, 512), (4, 3, 2048), (2, 2, 256), (8, 1, 256), (8, 3, 512), (1, 32, 4096)])
def test_key_formulation(m, G, Bh, L):
    kp, _, ks, _ = build_cache(m, Bh, L, 0.7, 11 + G)
    q = oracle.make_query(Bh * G, seed=5 + L)
    want = oracle.key_formulation_ref(kp, q, G)
    bmp, nz, idx, off = reference_layout(ks)
    padded = torch.nn.functional.pad(q.cuda().view(Bh * G, 1, 128), (0, 0, 0, 7))
    out = m.o.mustafar_key_formulation(bmp, nz, idx, off, padded, L, 128, Bh * G, G)
    assert out.shape == (Bh * G, 8, L) and out.dtype == torch.float16
    assert oracle.rel_l2(out[:, 0].cpu(), want) < TOL
    assert float(out[:, 1:].abs().max()) == 0.0


@pytest.mark.parametrize("G,Bh,L", [(1, 3, 256), (4, 2, 512), (4, 3, 2048), (2, 2, 320), (8, 1, 256), (8, 3, 512), (1, 32, 4096)])
def test_value_formulation(m, G, Bh, L):
    _, vp, _, vs = build_cache(m, Bh, L, 0.7, 21 + G)
    g = torch.Generator().manual_seed(3 + L)
    p = torch.softmax(torch.randn(Bh * G, L, generator=g) * 3, dim=-1).half()
    want = oracle.value_formulation_ref(vp, p, G)
    bmp, nz, idx, off = reference_layout(vs)
    padded = torch.nn.functional.pad(p.cuda().view(Bh * G, 1, L), (0, 0, 0, 7)).contiguous()
    ws = torch.zeros(1, dtype=torch.float16, device="cuda")
    out = m.o.mustafar_value_formulation(bmp, nz, idx, off, padded, ws, 128, L, Bh * G, G)
    assert out.shape == (Bh * G, 8, 128)
    assert oracle.rel_l2(out[:, 0].cpu(), want) < TOL


@pytest.mark.parametrize("G,Bh,L,W,s", [
    (1, 32, 4096, 0, 0.7),        # MHA, whole cache compressed, no window
    (4, 8, 4096, 128, 0.7),       # Llama-3-8B GQA shape, one sequence
    (4, 4, 1024, 129, 0.5),
    (4, 2, 256, 384, 0.7),        # window at its largest (residual + 256)
    (2, 3, 192, 77, 0.7),
    (8, 1, 512, 5, 0.7),
    (8, 3, 1024, 130, 0.7),       # 8 query heads per kv head: run as two groups of 4
    (4, 2, 0, 200, 0.7),          # nothing compressed yet
    (1, 2, 64, 0, 0.0),           # unpruned: every tile full, worst-case stage
])
def test_fused_decode_attention(m, G, Bh, L, W, s):
    if s > 0:
        kp, vp, ks, vs = build_cache(m, Bh, L, s, 31 + L + W)
    else:
        k, v = oracle.make_kv(Bh, L, seed=77)
        kp, vp = k, v
        ks = m.c.SparseStore(Bh, L, m.c.KEY, "cuda"); ks.append(k.cuda(), 0)
        vs = m.c.SparseStore(Bh, L, m.c.VALUE, "cuda"); vs.append(v.cuda(), 0)
    kw, vw = oracle.make_kv(Bh, max(W, 1), seed=99 + W)
    kw, vw = kw[:, :W], vw[:, :W]
    q = oracle.make_query(Bh * G, seed=8 + L)
    want = oracle.decode_attention_ref(q, kp, vp, kw, vw, G)
    out = m.o.decode_attention(q.cuda(), ks, vs, kw.cuda() if W else None, vw.cuda() if W else None, G)
    assert oracle.rel_l2(out.float().cpu(), want) < TOL
    if L and W:
        # the reference's own order of fp16 roundings agrees to the same tolerance
        model = oracle.decode_attention_model_order_ref(q, kp, vp, kw, vw, G)
        assert oracle.rel_l2(out.float().cpu(), model.float()) < 2 * TOL


def test_decode_split_invariance(m):
    kp, vp, ks, vs = build_cache(m, 2, 2048 + 64, 0.7, 5)     # 33 blocks: a ragged last split
    kw, vw = oracle.make_kv(2, 128, seed=6)
    q = oracle.make_query(8, seed=7).cuda()
    outs = [m.o.decode_attention(q, ks, vs, kw.cuda(), vw.cuda(), 4, nsplit=n).float()
            for n in (1, 3, 32)]
    want = oracle.decode_attention_ref(q.cpu(), kp, vp, kw, vw, 4)
    assert oracle.rel_l2(outs[0].cpu(), want) < TOL
    for o in outs[1:]:
        assert oracle.rel_l2(o.cpu(), outs[0].cpu()) < 1e-3


def test_small_stage_is_reported_not_silent(m):
    """A stage hint below the real block size must raise, never return garbage silently."""
    kp, vp, ks, vs = build_cache(m, 1, 128, 0.5, 3)
    q = oracle.make_query(1, seed=1).cuda()
    with pytest.raises(RuntimeError):
        m.o.decode_attention(q, ks, vs, None, None, 1, stage_halves=64)


@pytest.mark.parametrize("kind", ["misaligned", "beyond_extent", "negative"])
def test_corrupt_offsets_are_reported_not_followed(m, kind):
    """Offsets that the caller spliced wrongly (the reference-shaped ops take ``idx`` / ``NZ_Offset`` from torch
    code) must set the status bit; the kernels skip the copy instead of issuing a misaligned or out-of-range one."""
    kp, vp, ks, vs = build_cache(m, 2, 256, 0.7, 3)
    q = oracle.make_query(2, seed=1).cuda()
    bmp, nz, idx, off = reference_layout(ks)
    idx = idx.clone()
    if kind == "misaligned":
        idx[1, 128] += 1            # block start no longer a multiple of 16 bytes
    elif kind == "beyond_extent":
        idx[1, 128:] += 1 << 20     # (aligned) ranges far past the end of NZ
    else:
        idx[0, 256] = -8
    padded = torch.nn.functional.pad(q.view(2, 1, 128), (0, 0, 0, 7))
    m.o.check_device_status()
    with pytest.raises(RuntimeError):
        m.o.mustafar_key_formulation(bmp, nz, idx, off, padded, 256, 128, 2, 1)
    # the arena path: the same corruption inside a store
    ks.accum[1, 128] += 1 if kind == "misaligned" else (1 << 28 if kind == "beyond_extent" else -(1 << 20))
    with pytest.raises(RuntimeError):
        m.o.decode_attention(q, ks, vs, None, None, 1)


def test_op_argument_errors(m):
    kp, vp, ks, vs = build_cache(m, 1, 64, 0.7, 3)
    bmp, nz, idx, off = reference_layout(ks)
    q = torch.zeros(1, 8, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        m.o.mustafar_key_formulation(bmp, nz, idx, off, q.float(), 64, 128, 1, 1)
    with pytest.raises(RuntimeError):
        m.o.mustafar_key_formulation(bmp.int(), nz, idx, off, q, 64, 128, 1, 1)
    with pytest.raises(RuntimeError):
        m.o.mustafar_key_formulation(bmp.cpu(), nz, idx, off, q, 64, 128, 1, 1)


@pytest.mark.parametrize("L", [0, 64, 512, 1024])
def test_device_resident_length_matches_host_length(L):
    """mfar_decode_attention_fp16_dyn: the launch is sized for the stores' capacity (1024 tokens), the number of
    compressed tokens is read on the device; the result equals the host-length call for the same cache state."""
    from mustafar_b200 import compression as comp, ops
    Bh, G, cap_tokens, W = 4, 4, 1024, 96
    k, v = oracle.make_kv(Bh, cap_tokens, seed=321)
    kw, vw = oracle.make_kv(Bh, W, seed=322)
    q = oracle.make_query(Bh * G, seed=9).cuda()
    rank = comp.keep_rank(0.7)
    ks, vs = comp.SparseStore(Bh, cap_tokens, comp.KEY, "cuda"), comp.SparseStore(Bh, cap_tokens, comp.VALUE, "cuda")
    if L:
        ks.append(k[:, :L].cuda(), rank)
        vs.append(v[:, :L].cuda(), rank)
    want = ops.decode_attention(q, ks, vs, kw.cuda(), vw.cuda(), G)
    n_dev = torch.tensor([L], dtype=torch.int32, device="cuda")
    got = ops.decode_attention(q, ks, vs, kw.cuda(), vw.cuda(), G, n_tokens=n_dev, stage_halves=64 * rank_keep(0.7) + 896)
    ops.check_device_status()
    assert oracle.rel_l2(got.float().cpu(), want.float().cpu()) < 1e-3
    # appending one more block and bumping the device counter is all a replayed launch needs
    if L + 64 <= cap_tokens:
        ks.append(k[:, L:L + 64].cuda(), rank)
        vs.append(v[:, L:L + 64].cuda(), rank)
        n_dev += 64
        want2 = ops.decode_attention(q, ks, vs, kw.cuda(), vw.cuda(), G)
        got2 = ops.decode_attention(q, ks, vs, kw.cuda(), vw.cuda(), G, n_tokens=n_dev, stage_halves=64 * rank_keep(0.7) + 896)
        assert oracle.rel_l2(got2.float().cpu(), want2.float().cpu()) < 1e-3


def rank_keep(sparsity):
    """values kept per token (of 128) at this sparsity: 128 - keep_rank + 1"""
    from mustafar_b200 import compression as comp
    return 128 - comp.keep_rank(sparsity) + 1
