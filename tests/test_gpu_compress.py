"""GPU parity of prune + compression against the CPU oracle and the golden fixtures
(bit-exact: bitmaps, offsets, packed values).  Everything goes through the C ABI."""
import os

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

G = os.path.join(os.path.dirname(__file__), "golden")


def bits16(a):
    return np.ascontiguousarray(a).view(np.uint16)


@pytest.fixture(scope="module")
def mod():
    from mustafar_b200 import compression
    return compression


def _golden():
    f = np.load(os.path.join(G, "fp16_cases.npz"))
    return f, sorted({k.split("/")[0] for k in f.files})


@pytest.mark.parametrize("kind", ["key", "value"])
def test_convert_matches_golden(mod, kind):
    f, names = _golden()
    fn = mod.convert_key_batched if kind == "key" else mod.convert_value_batched
    for name in names:
        x = torch.from_numpy(f[f"{name}/x"]).cuda()
        bitmaps, accum, packed = fn(x)
        assert np.array_equal(bitmaps.cpu().numpy(), f[f"{name}/{kind}/bitmaps"]), name
        assert np.array_equal(accum.cpu().numpy(), f[f"{name}/{kind}/accum"]), name
        flat = torch.cat(packed).cpu().numpy() if packed else np.zeros(0, np.float16)
        assert np.array_equal(bits16(flat), bits16(f[f"{name}/{kind}/packed_flat"])), name
        assert len(packed) == x.shape[0]
        assert bitmaps.dtype == torch.int64 and accum.dtype == torch.int32 and packed[0].dtype == torch.float16


def test_prune_matches_golden(mod):
    f = np.load(os.path.join(G, "prune_cases.npz"))
    raw = torch.from_numpy(f["raw"]).cuda()
    for s in (10, 50, 70, 90, 99):
        got = mod.prune(raw, s / 100.0).cpu().numpy()
        assert np.array_equal(bits16(got), bits16(f[f"s{s}"])), s


@pytest.mark.parametrize("sparsity", [0.5, 0.7])
@pytest.mark.parametrize("kind", ["key", "value"])
def test_fused_prune_compress_vs_oracle(mod, kind, sparsity):
    k, v = oracle.make_kv(5, 512, seed=oracle.synth.BASE_SEED + 3)
    x = k if kind == "key" else v
    x[0, :7] = 0
    x[1, 5] = 1.0                      # all-equal row: everything kept
    x[2, 9, ::3] = x[2, 9, 1]          # ties
    want = oracle.prune_ref(x, sparsity)
    fn = oracle.compress_key_ref if kind == "key" else oracle.compress_value_ref
    wb, wa, wp = fn(want)
    store = mod.SparseStore(5, 512, mod.KEY if kind == "key" else mod.VALUE, "cuda")
    store.append(x.cuda(), mod.keep_rank(sparsity))
    store.check()
    assert np.array_equal(store.bitmaps.cpu().numpy(), wb)
    assert np.array_equal(store.accum.cpu().numpy(), wa)
    for h in range(5):
        n = len(wp[h])
        assert np.array_equal(bits16(store.nz[h, :n].cpu().numpy()), bits16(wp[h]))
    assert store.stage_hint() >= 2 * int(np.diff(wa[:, ::128], axis=1).max())


@pytest.mark.parametrize("kind", ["key", "value"])
def test_block_append_equals_one_shot(mod, kind):
    """Appending 256-token blocks (what the decode loop does every 256 steps,
    models/llama_mustafar_kernel.py:445-519) gives the same cache as compressing at once."""
    k, v = oracle.make_kv(4, 768, seed=oracle.synth.BASE_SEED + 4)
    x = (k if kind == "key" else v).cuda()
    kk = mod.KEY if kind == "key" else mod.VALUE
    rank = mod.keep_rank(0.7)
    a = mod.SparseStore(4, 768, kk, "cuda")
    a.append(x, rank)
    b = mod.SparseStore(4, 768, kk, "cuda")
    for t0 in range(0, 768, 256):
        b.append(x[:, t0:t0 + 256], rank)     # strided view: no copy
    a.check(); b.check()
    assert torch.equal(a.bitmaps, b.bitmaps) and torch.equal(a.accum, b.accum)
    n = int(a.packed_lengths().max())
    lens = a.packed_lengths().tolist()
    for h in range(4):
        assert torch.equal(a.nz[h, :lens[h]].view(torch.int16), b.nz[h, :lens[h]].view(torch.int16))
    assert n > 0


def test_capacity_overflow_is_reported(mod):
    k, _ = oracle.make_kv(2, 128)
    store = mod.SparseStore(2, 128, mod.KEY, "cuda", nz_capacity=1024)
    store.append(k.cuda(), 0)          # dense input cannot fit 1024 halves per head
    with pytest.raises(RuntimeError):
        store.check()


def test_argument_errors(mod):
    with pytest.raises(RuntimeError):
        mod.convert_key_batched(torch.zeros(1, 64, 128, dtype=torch.float16))          # CPU tensor
    with pytest.raises(RuntimeError):
        mod.convert_key_batched(torch.zeros(1, 65, 128, dtype=torch.float16, device="cuda"))
    with pytest.raises(RuntimeError):
        mod.convert_key_batched(torch.zeros(1, 64, 128, dtype=torch.float32, device="cuda"))


def _torch_prune(x, sparsity):
    # the reference's own formula on the GPU (models/llama_mustafar_kernel.py:215-228)
    D = x.shape[-1]
    k = max(1, int(sparsity * D))
    flat = x.reshape(-1, D)
    thr, _ = torch.kthvalue(flat.abs().float(), k, dim=-1, keepdim=True)
    return (flat * (flat.abs().float() >= thr)).view(x.shape)


@pytest.mark.parametrize("sparsity", [0.5, 0.7])
def test_full_size_properties(mod, sparsity):
    """Prefill shape [8 sequences x 8 kv heads, 8192 tokens, 128]: size-independent checks."""
    g = torch.Generator(device="cuda").manual_seed(1234)
    x = torch.randn(64, 8192, 128, generator=g, device="cuda", dtype=torch.float32)
    x[:, :, [3, 40, 77, 120]] *= 10
    x = x.half()
    want = _torch_prune(x, sparsity)
    got = mod.prune(x, sparsity)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    for kind, kk in (("key", mod.KEY), ("value", mod.VALUE)):
        store = mod.SparseStore(64, 8192, kk, "cuda")
        store.append(x, mod.keep_rank(sparsity))
        store.check()
        nz = want != 0
        if kind == "key":
            per_tile = nz.view(64, 128, 64, 128).sum(dim=2).reshape(64, -1)          # [h, blk, c]
        else:
            per_tile = nz.view(64, 128, 64, 2, 64).sum(dim=4).permute(0, 1, 3, 2).reshape(64, -1)
        # popcount of every bitmap, padded counts, prefix sums
        bm = store.bitmaps
        pop = torch.zeros_like(bm)
        for sh in range(64):
            pop += (bm >> sh) & 1
        assert torch.equal(pop, per_tile.to(torch.int64))
        counts = ((per_tile + 7) & ~7) >> 1
        acc = torch.zeros_like(store.accum)
        acc[:, 1:] = torch.cumsum(counts, dim=1).to(torch.int32)
        assert torch.equal(acc, store.accum)
        # checksum of the packed values == checksum of the kept values (order-free, exact in int64)
        lens = store.packed_lengths()
        idx = torch.arange(store.nz_capacity, device="cuda")[None, :] < lens[:, None]
        got_sum = (store.nz.view(torch.int16).to(torch.int64) & 0xffff)[idx].sum()
        want_sum = (torch.where(nz, want, torch.zeros_like(want)).view(torch.int16).to(torch.int64) & 0xffff).sum()
        assert int(got_sum) == int(want_sum)
        del store


def test_wire_format_round_trip_feeds_decode():
    """A cache that went through the wire format (device -> blob -> device) decodes to the same output."""
    import torch
    from mustafar_b200 import compression as comp, ops, wire
    g = torch.Generator(device="cuda").manual_seed(11)
    Bh, L, G = 4, 512, 4
    k = torch.randn(Bh, L, 128, generator=g, device="cuda").half()
    v = torch.randn(Bh, L, 128, generator=g, device="cuda").half()
    q = torch.randn(Bh * G, 128, generator=g, device="cuda").half()
    ks, vs = comp.SparseStore(Bh, L, comp.KEY, "cuda"), comp.SparseStore(Bh, L, comp.VALUE, "cuda")
    ks.append(k, comp.keep_rank(0.7))
    vs.append(v, comp.keep_rank(0.7))
    ks2 = wire.unpack_store(wire.pack_store(ks), "cuda", max_tokens=1024, nz_capacity=1024 * 64)
    vs2 = wire.unpack_store(wire.pack_store(vs), "cuda", max_tokens=1024, nz_capacity=1024 * 64)
    a = ops.decode_attention(q, ks, vs, None, None, G)
    b = ops.decode_attention(q, ks2, vs2, None, None, G)
    assert torch.equal(a, b)
    # and the restored arena takes further appends
    ks2.append(k[:, :64], comp.keep_rank(0.7))
    assert ks2.tokens == L + 64
    ks2.check()


@pytest.mark.parametrize("kind", ["key", "value"])
def test_projection_layout_is_compressed_in_place(kind):
    """A [batch, token, kv head, 128] slice of a fused q|k|v projection output, viewed as [batch, kv head, token, 128]
    (what the prefill hands over for V), is read through its strides: same cache as for the flattened copy."""
    from mustafar_b200 import compression as comp
    B, T, hq, hkv = 3, 320, 8, 2
    g = torch.Generator(device="cuda").manual_seed(12)
    qkv = torch.randn(B, T, (hq + 2 * hkv) * 128, generator=g, device="cuda").half()
    v = qkv[..., (hq + hkv) * 128:].view(B, T, hkv, 128).transpose(1, 2)          # strided view, nothing contiguous
    assert not v.is_contiguous()
    k = comp.KEY if kind == "key" else comp.VALUE
    a, b = comp.SparseStore(B * hkv, 512, k, "cuda"), comp.SparseStore(B * hkv, 512, k, "cuda")
    rank = comp.keep_rank(0.7)
    a.append(v[:, :, :256], rank)
    a.append(v[:, :, 256:], rank)
    b.append(v.reshape(B * hkv, T, 128).contiguous(), rank)
    a.check(); b.check()
    assert torch.equal(a.bitmaps[:, :a.tiles], b.bitmaps[:, :b.tiles]) and torch.equal(a.accum[:, :a.tiles + 1], b.accum[:, :b.tiles + 1])
    for h, n in enumerate(a.packed_lengths().tolist()):
        assert torch.equal(a.nz[h, :n].view(torch.int16), b.nz[h, :n].view(torch.int16))
