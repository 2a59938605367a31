"""GPU parity of the quantised path: compression bit-exact against the golden fixtures
(reference Triton kernels) and the oracle; ops against dequantise-then-dense (2e-3 rel L2)."""
import os

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3
G_DIR = os.path.join(os.path.dirname(__file__), "golden")


def bits16(a):
    return np.ascontiguousarray(a).view(np.uint16)


@pytest.fixture(scope="module")
def m():
    os.environ["MUSTAFAR_B200_CHECK"] = "1"
    from mustafar_b200 import compression, compression_quant, ops_quant

    class M:
        pass
    M.c, M.cq, M.oq = compression, compression_quant, ops_quant
    return M


@pytest.mark.parametrize("kind", ["key", "value"])
def test_convert_quant_matches_golden(m, kind):
    f = np.load(os.path.join(G_DIR, "quant_cases.npz"))
    names = sorted({k.split("/")[0] for k in f.files})
    for name in names:
        x = torch.from_numpy(f[f"{name}/x"]).cuda()
        if kind == "key":
            bmp, off, packed, counts, units, scales, zeros = m.cq.convert_key_batched_quant(x, return_metadata=True)
            assert len(m.cq.convert_key_batched_quant(x)) == 5
        else:
            bmp, off, packed, counts, units, scales, zeros = m.cq.convert_value_batched_quant(x)
        got = dict(bitmaps=bmp, tile_offsets=off, packed=packed, counts=counts, units=units)
        for key, t in got.items():
            assert np.array_equal(t.cpu().numpy(), f[f"{name}/{kind}/{key}"]), (name, key)
        assert np.array_equal(bits16(scales.cpu().numpy()), bits16(f[f"{name}/{kind}/scales"])), name
        assert np.array_equal(bits16(zeros.cpu().numpy()), bits16(f[f"{name}/{kind}/zeros"])), name
        assert packed.dtype == torch.int32 and scales.dtype == torch.float16


@pytest.mark.parametrize("bits,group", [(2, 64), (4, 64), (2, 32), (4, 32)])
@pytest.mark.parametrize("kind", ["key", "value"])
def test_fused_prune_quant_vs_oracle(m, kind, bits, group):
    k, v = oracle.make_kv(3, 320, seed=oracle.synth.BASE_SEED + 7)
    x = k if kind == "key" else v
    want_in = oracle.prune_ref(x, 0.5)
    fn = oracle.quant_compress_key_ref if kind == "key" else oracle.quant_compress_value_ref
    want = fn(want_in, bits=bits, group=group)
    got = m.cq.compress_quant(x.cuda(), m.c.KEY if kind == "key" else m.c.VALUE, m.c.keep_rank(0.5), bits, group)
    for key in ("bitmaps", "tile_offsets", "counts", "units", "packed"):
        assert np.array_equal(got[key].cpu().numpy(), want[key]), key
    for key in ("scales", "zeros"):
        assert np.array_equal(bits16(got[key].cpu().numpy()), bits16(want[key])), key


def build(m, Bh, L, s, bits, group, seed):
    k, v = oracle.make_kv(Bh, L, seed=seed)
    kp, vp = oracle.prune_ref(k, s), oracle.prune_ref(v, s)
    kq = m.cq.compress_quant(k.cuda(), m.c.KEY, m.c.keep_rank(s), bits, group)
    vq = m.cq.compress_quant(v.cuda(), m.c.VALUE, m.c.keep_rank(s), bits, group)
    kd = oracle.dequant_key_ref(oracle.quant_compress_key_ref(kp, bits, group), L, bits=bits, group=group)
    vd = oracle.dequant_value_ref(oracle.quant_compress_value_ref(vp, bits, group), L, bits=bits, group=group)
    return kq, vq, kd, vd


@pytest.mark.parametrize("G,Bh,L,s,bits,group", [
    (1, 3, 256, 0.7, 2, 64), (4, 2, 512, 0.5, 2, 64), (4, 2, 1024, 0.7, 2, 64), (8, 1, 256, 0.7, 2, 64), (8, 3, 512, 0.7, 2, 64),
    (4, 2, 256, 0.7, 4, 64), (4, 2, 256, 0.5, 2, 32), (2, 2, 192, 0.5, 4, 32),
])
def test_quant_ops_vs_dequantise_then_dense(m, G, Bh, L, s, bits, group):
    kq, vq, kd, vd = build(m, Bh, L, s, bits, group, 40 + L)
    q = oracle.make_query(Bh * G, seed=9 + L)
    cap = 32 // bits
    # key op
    want = oracle.key_formulation_ref(kd, q, G)
    padded = torch.nn.functional.pad(q.cuda().view(Bh * G, 1, 128), (0, 0, 0, 7))
    args = (kq["bitmaps"], kq["packed"], kq["tile_offsets"])
    out = m.oq.mustafar_key_formulation_quant(*args, kq["scales"], kq["zeros"], padded, L, 128, Bh * G, G, bits, cap, 0)
    assert out.shape == (Bh * G, 8, L)
    assert oracle.rel_l2(out[:, 0].cpu(), want) < TOL
    out2 = m.oq.mustafar_key_formulation_quant_meta(*args, kq["counts"], kq["units"], kq["scales"], kq["zeros"], padded,
                                                    L, 128, Bh * G, G, bits, cap, 1)
    assert torch.equal(out, out2)
    # value ops
    gen = torch.Generator().manual_seed(L)
    p = torch.softmax(torch.randn(Bh * G, L, generator=gen) * 3, dim=-1).half()
    want_v = oracle.value_formulation_ref(vd, p, G)
    pp = torch.nn.functional.pad(p.cuda().view(Bh * G, 1, L), (0, 0, 0, 7)).contiguous()
    ws = torch.zeros(1, dtype=torch.float16, device="cuda")
    vargs = (vq["bitmaps"], vq["packed"], vq["tile_offsets"], vq["counts"], vq["units"], vq["scales"], vq["zeros"])
    o1 = m.oq.mustafar_value_formulation_quant(*vargs, pp, ws, 128, L, Bh * G, G, bits, cap, 0, 4, 2)
    assert o1.shape == (Bh * G, 8, 128)
    assert oracle.rel_l2(o1[:, 0].cpu(), want_v) < TOL
    o2 = m.oq.mustafar_value_formulation_quant_decode_n1(*vargs, p.cuda(), ws, 128, L, Bh * G, G, bits, cap, 0, 4)
    assert o2.shape == (Bh * G, 128)
    assert oracle.rel_l2(o2.cpu(), want_v) < TOL
    assert m.oq.mustafar_quant_sparse_forward is m.oq.mustafar_key_formulation_quant


@pytest.mark.parametrize("G,Bh,L,W,s,bits,group", [
    (4, 8, 2048, 128, 0.7, 2, 64), (4, 2, 512, 200, 0.5, 2, 64), (1, 4, 256, 0, 0.7, 2, 64),
    (4, 2, 256, 128, 0.7, 4, 64), (4, 2, 256, 128, 0.5, 2, 32), (4, 2, 0, 130, 0.7, 2, 64),
    (8, 3, 512, 130, 0.7, 2, 64), (8, 2, 256, 0, 0.7, 4, 64),      # 8 query heads per kv head: two groups of 4
])
def test_fused_quant_attention(m, G, Bh, L, W, s, bits, group):
    if L:
        kq, vq, kd, vd = build(m, Bh, L, s, bits, group, 60 + L + W)
    else:
        kq = vq = dict(bitmaps=torch.zeros(Bh, 0, dtype=torch.int64, device="cuda"),
                       tile_offsets=torch.zeros(Bh, 0, dtype=torch.int32, device="cuda"),
                       scales=torch.zeros(Bh, 0, dtype=torch.float16, device="cuda"),
                       zeros=torch.zeros(Bh, 0, dtype=torch.float16, device="cuda"),
                       packed=torch.zeros(1, dtype=torch.int32, device="cuda"))
        kd = vd = torch.zeros(Bh, 0, 128, dtype=torch.float16)
    kw, vw = oracle.make_kv(Bh, max(W, 1), seed=70 + W)
    kw, vw = kw[:, :W], vw[:, :W]
    q = oracle.make_query(Bh * G, seed=3 + L)
    want = oracle.decode_attention_ref(q, kd, vd, kw, vw, G)
    out = m.oq.decode_attention_quant(q.cuda(), kq, vq, L, kw.cuda() if W else None, vw.cuda() if W else None, G, bits)
    assert oracle.rel_l2(out.float().cpu(), want) < TOL


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("bits,group", [(2, 64), (4, 64), (2, 32)])
def test_quant_store_appends_match_one_shot_compression(m, kind, bits, group):
    """Arena mode of mfar_compress_quant: three appends (256 + 64 + 192 tokens) leave, tile by tile, what one
    call over all 512 tokens leaves in the compact layout; decode over the arena equals decode over the compact one."""
    from mustafar_b200 import compression as comp
    from mustafar_b200 import compression_quant as cq
    Bh, L, G = 4, 512, 4
    k, v = oracle.make_kv(Bh, L, seed=91 + kind)
    x = (k if kind == 0 else v).cuda()
    rank = comp.keep_rank(0.7)
    ref = cq.compress_quant(x, kind, rank, bits, group)
    st = cq.QuantStore(Bh, 1024, kind, "cuda", bits, group)
    for a, b in ((0, 256), (256, 320), (320, 512)):
        st.append(x[:, a:b], rank)
    st.check()
    T = 2 * L
    d = st.as_dict()
    assert st.tokens == L
    assert torch.equal(d["bitmaps"][:, :T], ref["bitmaps"])
    assert torch.equal(d["counts"][:, :T], ref["counts"]) and torch.equal(d["units"][:, :T], ref["units"])
    assert torch.equal(d["scales"][:, :T], ref["scales"]) and torch.equal(d["zeros"][:, :T], ref["zeros"])
    # same code words tile by tile (the offsets differ: per-head arena vs one flat stream)
    offs_a, offs_r, units = d["tile_offsets"][:, :T].cpu(), ref["tile_offsets"].cpu(), ref["units"].cpu()
    flat_a, flat_r = d["packed"].cpu(), ref["packed"].cpu()
    for h in range(Bh):
        for t in range(0, T, 37):
            n = int(units[h, t])
            assert torch.equal(flat_a[offs_a[h, t]:offs_a[h, t] + n], flat_r[offs_r[h, t]:offs_r[h, t] + n])
    assert (st.head_tail.cpu() == units.sum(1).to(torch.int32)).all()
    if kind == 0:
        vs = cq.QuantStore(Bh, 1024, 1, "cuda", bits, group)
        vs.append(v.cuda(), rank)
        vref = cq.compress_quant(v.cuda(), 1, rank, bits, group)
        q = oracle.make_query(Bh * G, seed=5).cuda()
        a = m.oq.decode_attention_quant(q, d, vs.as_dict(), L, None, None, G, bits)
        b = m.oq.decode_attention_quant(q, ref, vref, L, None, None, G, bits)
        assert torch.equal(a, b)


def test_quant_store_reports_a_full_code_arena(m):
    from mustafar_b200 import compression_quant as cq
    from mustafar_b200._lib import MustafarError
    k, _ = oracle.make_kv(2, 128, seed=7)
    st = cq.QuantStore(2, 128, 0, "cuda", words_capacity=64)     # far too small
    st.append(k.cuda(), 0)
    with pytest.raises(MustafarError):
        st.check()


def test_dequant_rounding_difference_is_bounded(m):
    """The reference's kernels round every dequantised value to fp16 before the dot product
    (kernel_quant/csrc/SpMM_Kernel_Quant.cuh:235-240); this library keeps (code - zero) * scale in fp32.  The two
    conventions must stay within a small fraction of the 2e-3 tolerance of each other: the kernel's output is
    compared with dense attention on the fp16-rounded values (the oracle's mode 0) and on unrounded fp32 values."""
    Bh, G, L, bits = 2, 4, 1024, 2
    k, v = oracle.make_kv(Bh, L, seed=77)
    kp, vp = oracle.prune_ref(k, 0.7), oracle.prune_ref(v, 0.7)
    kq = m.cq.compress_quant(k.cuda(), m.c.KEY, m.c.keep_rank(0.7), bits, 64)
    vq = m.cq.compress_quant(v.cuda(), m.c.VALUE, m.c.keep_rank(0.7), bits, 64)
    fk, fv = oracle.quant_compress_key_ref(kp, bits, 64), oracle.quant_compress_value_ref(vp, bits, 64)
    kd16 = torch.from_numpy(oracle.dequant_key_ref(fk, L, bits=bits))
    vd16 = torch.from_numpy(oracle.dequant_value_ref(fv, L, bits=bits))

    def exact(fmt, to_dense):
        """(code - zero) * scale without the fp16 rounding, through the oracle's own unpacking"""
        import numpy as np
        from oracle import quant_format as qf
        tiles16 = qf._dequant_tiles(fmt, bits, 64, 0)
        bitmaps = fmt["bitmaps"].view(np.uint64)
        bit = ((bitmaps[..., None] >> np.arange(63, -1, -1, dtype=np.uint64)) & np.uint64(1)).astype(bool)
        rank = np.cumsum(bit, axis=-1) - 1
        cap = 32 // bits
        word = fmt["tile_offsets"][..., None].astype(np.int64) + np.where(bit, rank // cap, 0)
        packed = fmt["packed"].view(np.uint32)
        q = (packed[np.minimum(word, packed.size - 1)] >> ((np.where(bit, rank, 0) % cap) * bits).astype(np.uint32)) & np.uint32(3)
        s = fmt["scales"].astype(np.float32)[..., None]
        z = fmt["zeros"].astype(np.float32)[..., None]
        t = np.where(bit, (q.astype(np.float32) - z) * s, 0.0).astype(np.float32)
        assert np.array_equal(t.astype(np.float16), tiles16)
        return to_dense(t)

    Bh_, T = fk["bitmaps"].shape
    kd32 = torch.from_numpy(np.ascontiguousarray(exact(fk, lambda t: t.reshape(Bh, L // 64, 128, 64).transpose(0, 1, 3, 2))).reshape(Bh, L, 128))
    vd32 = torch.from_numpy(np.ascontiguousarray(exact(fv, lambda t: t.reshape(Bh, L // 64, 2, 64, 64).transpose(0, 1, 3, 2, 4))).reshape(Bh, L, 128))
    q = oracle.make_query(Bh * G, seed=3)
    empty = torch.zeros(Bh, 0, 128, dtype=torch.float16)

    def dense_attention(kd, vd):
        kk, vv = kd.float().repeat_interleave(G, 0), vd.float().repeat_interleave(G, 0)
        s = torch.bmm(kk, q.float().unsqueeze(-1)).squeeze(-1) / 128 ** 0.5
        return torch.bmm(torch.softmax(s, -1).unsqueeze(1), vv).squeeze(1)

    want16, want32 = dense_attention(kd16, vd16), dense_attention(kd32, vd32)
    out = m.oq.decode_attention_quant(q.cuda(), kq, vq, L, None, None, G, bits).float().cpu()
    between = oracle.rel_l2(want32, want16)
    assert between < 5e-4, between                       # the two conventions themselves
    assert oracle.rel_l2(out, want32) < 1e-3             # what the kernel computes
    assert oracle.rel_l2(out, want16) < TOL              # what the reference's convention gives
