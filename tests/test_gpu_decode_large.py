"""Parity of the decode kernels at the sizes the benchmark runs (up to 64 sequences x 32768 tokens).

The caches are built on the GPU exactly as ``bench.py`` builds them; the check is sampled so that the CPU
side stays at seconds: a few kv heads' slices of the compressed cache are copied to the host, expanded by the
oracle (``decompress_*_ref`` / ``dequant_*_ref``), and the oracle's fp32 attention over
[expanded ; window] is compared with the kernel's output for those heads' query heads.
Tolerance: 2e-3 relative L2 (fp16 storage, fp32 accumulation)."""
import os
import sys

import numpy as np
import pytest
import torch

import oracle

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402  (the benchmark's own cache builder and sampled check)

pytestmark = pytest.mark.gpu
TOL = 2e-3
G = 4


@pytest.mark.parametrize("batch,kv_len", [(1, 4096), (8, 32768), (64, 16384), (64, 32768)])
def test_fused_attention_at_benchmark_sizes(batch, kv_len):
    """Llama-3-8B head shape, 128-token window, 70 % sparsity: 16-32 splits of up to 32 blocks, grids of several
    thousand CTAs, packed offsets close to 2^30 halves per arena."""
    from mustafar_b200 import ops
    dev = torch.device("cuda")
    ks, vs, kw, vw = bench.build_cache(batch, kv_len, 128, 0.7, dev, 20260302 + 9973 * 2)
    gen = torch.Generator(device=dev).manual_seed(7)
    q = torch.randn(batch * 32, 128, generator=gen, device=dev).half()
    out = ops.decode_attention(q, ks, vs, kw, vw, G, stage_halves=max(ks.stage_hint(), vs.stage_hint()))
    ops.check_device_status(dev)
    res = bench.parity_check(q, out, ks, vs, kw, vw, 4, TOL)
    assert res["ok"], res
    del ks, vs
    torch.cuda.empty_cache()


def test_device_resident_length_at_full_capacity():
    """mfar_decode_attention_fp16_dyn with max_tokens = 32768: the launch is sized for the capacity, the length
    (here 24576 + a ragged 192) is read on the device; the result equals the host-length call."""
    from mustafar_b200 import compression as comp, ops
    dev = torch.device("cuda")
    batch, cap_tokens, L = 4, 32768, 24576 + 192
    Bh = batch * 8
    gen = torch.Generator(device=dev).manual_seed(11)
    rank = comp.keep_rank(0.7)
    ks = comp.SparseStore(Bh, cap_tokens, comp.KEY, dev, nz_capacity=cap_tokens * 64)
    vs = comp.SparseStore(Bh, cap_tokens, comp.VALUE, dev, nz_capacity=cap_tokens * 64)
    for t0 in range(0, L, 4096):
        n = min(4096, L - t0)
        ks.append(torch.randn(Bh, n, 128, generator=gen, device=dev).half(), rank)
        vs.append(torch.randn(Bh, n, 128, generator=gen, device=dev).half(), rank)
    kw = torch.randn(Bh, 384, 128, generator=gen, device=dev).half()
    vw = torch.randn(Bh, 384, 128, generator=gen, device=dev).half()
    q = torch.randn(Bh * G, 128, generator=gen, device=dev).half()
    want = ops.decode_attention(q, ks, vs, kw[:, :200], vw[:, :200], G)
    n_dev = torch.tensor([L], dtype=torch.int32, device=dev)
    w_dev = torch.tensor([200], dtype=torch.int32, device=dev)
    kept = 128 - rank + 1
    got = ops.decode_attention(q, ks, vs, kw, vw, G, n_tokens=n_dev, window_len=w_dev, stage_halves=64 * kept + 896)
    ops.check_device_status(dev)
    assert oracle.rel_l2(got.float().cpu(), want.float().cpu()) < 1e-3
    res = bench.parity_check(q, got, ks, vs, kw[:, :200], vw[:, :200], 3, TOL)
    assert res["ok"], res


def _quant_head_dense(store, h, kind, bits):
    """Oracle expansion of head h of a QuantStore (offsets rebased to the head's own code words)."""
    T = 2 * store.tokens
    fmt = dict(
        bitmaps=store.bitmaps[h:h + 1, :T].cpu().numpy(),
        tile_offsets=(store.tile_offsets[h:h + 1, :T] - h * store.words_capacity).cpu().numpy(),
        packed=store.packed[h].cpu().numpy(),
        scales=store.scales[h:h + 1, :T].cpu().numpy(),
        zeros=store.zeros[h:h + 1, :T].cpu().numpy(),
    )
    fn = oracle.dequant_key_ref if kind == "key" else oracle.dequant_value_ref
    return torch.from_numpy(fn(fmt, store.tokens, bits=bits, group=64))


@pytest.mark.parametrize("batch,kv_len,sparsity", [(32, 16384, 0.5), (32, 16384, 0.7), (64, 32768, 0.7)])
def test_quantised_attention_at_benchmark_sizes(batch, kv_len, sparsity):
    """2-bit codes per tile (the reference's quantised format) at the sizes the kernel table times."""
    from mustafar_b200 import compression as comp, compression_quant as cq, ops, ops_quant
    dev = torch.device("cuda")
    Bh = batch * 8
    gen = torch.Generator(device=dev).manual_seed(5)
    rank = comp.keep_rank(sparsity)
    ks = cq.QuantStore(Bh, kv_len, comp.KEY, dev, 2, 64)
    vs = cq.QuantStore(Bh, kv_len, comp.VALUE, dev, 2, 64)
    chunk = max(256, min(kv_len, (1 << 28) // (Bh * 128) // 256 * 256))
    for t0 in range(0, kv_len, chunk):
        n = min(chunk, kv_len - t0)
        ks.append(torch.randn(Bh, n, 128, generator=gen, device=dev).half(), rank)
        vs.append(torch.randn(Bh, n, 128, generator=gen, device=dev).half(), rank)
    ks.check(); vs.check()
    kw = torch.randn(Bh, 128, 128, generator=gen, device=dev).half()
    vw = torch.randn(Bh, 128, 128, generator=gen, device=dev).half()
    q = torch.randn(Bh * G, 128, generator=gen, device=dev).half()
    out = ops_quant.decode_attention_quant(q, ks.as_dict(), vs.as_dict(), kv_len, kw, vw, G, 2)
    ops.check_device_status(dev)
    worst = 0.0
    for h in (0, Bh // 2 + 1, Bh - 1):
        kd, vd = _quant_head_dense(ks, h, "key", 2), _quant_head_dense(vs, h, "value", 2)
        want = oracle.decode_attention_ref(q[h * G:(h + 1) * G].cpu(), kd, vd, kw[h:h + 1].cpu(), vw[h:h + 1].cpu(), G)
        worst = max(worst, oracle.rel_l2(out[h * G:(h + 1) * G].float().cpu(), want))
    assert worst < TOL, worst
    del ks, vs
    torch.cuda.empty_cache()
