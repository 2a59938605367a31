"""Per-kernel timings of the hot path on one GPU (CUDA events, warm-up, inputs larger than L2).

    python -m mustafar_b200.kernel_bench [--what compress,decode,ops,quant] [--quick]

Prints one JSON line per measurement: the workload, microseconds per call, the algorithmic bytes
the call has to move and the resulting GB/s.  Inputs are seeded synthetic tensors (K, V ~ N(0,1),
four K outlier channels x10), shapes follow the Llama-3-8B head layout (32 q heads, 8 kv heads,
head_dim 128).  bench.py stays the headline benchmark; this is the table behind it.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import _lib
from . import compression as comp
from . import compression_quant as cq
from . import ops, ops_quant

HQ, HKV, D = 32, 8, 128
G = HQ // HKV


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters       # microseconds


def timed_graph(fn, iters=10, warmup=3):
    """Same as timed(), but the calls are captured in a CUDA graph first, which removes the host's
    launch cost (Python + ctypes, ~20 us per call) from the figure: what a graph-replayed decode step pays."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def emit(name, us, nbytes, **kw):
    print(json.dumps({"kernel": name, "us": round(us, 2), "algorithmic_bytes": int(nbytes),
                      "GBps": round(nbytes / us / 1e3, 1), **kw}), flush=True)


def synth(Bh, L, seed, outliers):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(Bh, L, D, generator=g, device="cuda")
    if outliers:
        x[:, :, [3, 40, 77, 120]] *= 10
    return x.half()


def store_bytes(st):
    return 8 * st.n_heads * st.tiles + 4 * st.n_heads * (st.tiles + 1) + 2 * int(st.packed_lengths().sum())


def bench_compress(quick):
    Bh, L = (16, 4096) if quick else (64, 8192)              # prefill shape [8 sequences x 8 kv heads, 8192 tokens, 128]
    for s in (0.5, 0.7):
        for kind, name in ((comp.KEY, "K"), (comp.VALUE, "V")):
            x = synth(Bh, L, 11, kind == comp.KEY)
            st = comp.SparseStore(Bh, L, kind, "cuda")

            def run():
                st.tokens = 0
                st.append(x, comp.keep_rank(s))
            us = timed(run)
            st.check()
            emit(f"prune+compress {name} fp16", us, x.numel() * 2 + store_bytes(st), heads=Bh, tokens=L, sparsity=s)
            pruned = comp.prune(x, s)
            fn = comp.convert_key_batched if kind == comp.KEY else comp.convert_value_batched
            us = timed(lambda: fn(pruned), iters=3, warmup=1)
            emit(f"convert_{'key' if kind == comp.KEY else 'value'}_batched API (pruned input, reference return types)",
                 us, x.numel() * 2 + store_bytes(st), heads=Bh, tokens=L, sparsity=s)
            us = timed(lambda: cq.compress_quant(x, kind, comp.keep_rank(s), 2, 64), iters=3, warmup=1)
            emit(f"prune+compress {name} 2-bit (API incl. allocation and one sync)", us, x.numel() * 2, heads=Bh,
                 tokens=L, sparsity=s)
            del st, x, pruned
    # the decode-time append: one 256-token block behind an 8192-token cache
    x = synth(Bh, L + 256, 12, True)
    st = comp.SparseStore(Bh, L + 256, comp.KEY, "cuda")
    st.append(x[:, :L], comp.keep_rank(0.7))

    def app():
        st.tokens = L
        st.append(x[:, L:], comp.keep_rank(0.7))
    emit("append 256-token block (K, prune fused)", timed(app), Bh * 256 * D * 2 * 1.47, heads=Bh, cache_tokens=L)
    xc = x[:, :L].contiguous()
    y = torch.empty_like(xc)
    us = timed(lambda: comp.prune(xc, 0.7, out=y))
    emit("prune only", us, 2 * Bh * L * D * 2, heads=Bh, tokens=L)


def bench_compress_fp16(quick, iters=3, warmup=1):
    """Only the fused prune+compress kernel (K and V, 70 %) and the prune-only kernel: few launches,
    the case to put under a profiler."""
    Bh, L = (16, 4096) if quick else (64, 8192)
    for kind, name in ((comp.KEY, "K"), (comp.VALUE, "V")):
        x = synth(Bh, L, 11, kind == comp.KEY)
        st = comp.SparseStore(Bh, L, kind, "cuda")

        def run():
            st.tokens = 0
            st.append(x, comp.keep_rank(0.7))
        us = timed(run, iters=iters, warmup=warmup)
        emit(f"prune+compress {name} fp16", us, x.numel() * 2 + store_bytes(st), heads=Bh, tokens=L, sparsity=0.7)
        if kind == comp.KEY:
            y = torch.empty_like(x)
            us = timed(lambda: comp.prune(x, 0.7, out=y), iters=iters, warmup=warmup)
            emit("prune only", us, 2 * x.numel() * 2, heads=Bh, tokens=L)
        # the quantised kernel alone: outputs preallocated once, no host sync inside the timed calls
        T, worst = 2 * L, Bh * 2 * L * 4
        bufs = [torch.empty((Bh, T), dtype=dt, device="cuda") for dt in (torch.int64, torch.int32, torch.int32, torch.int32,
                                                                          torch.float16, torch.float16)]
        packed = torch.empty(worst, dtype=torch.int32, device="cuda")
        info = torch.zeros(Bh + 1, dtype=torch.int32, device="cuda")
        need = _lib.lib().mfar_compress_scratch_bytes(Bh, L)
        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")

        def runq():
            _lib.check(_lib.lib().mfar_compress_quant(
                x.data_ptr(), x.stride(0), x.stride(1), 0, 0, Bh, L, kind, comp.keep_rank(0.7), 2, 64,
                bufs[0].data_ptr(), T, bufs[1].data_ptr(), bufs[2].data_ptr(), bufs[3].data_ptr(), bufs[4].data_ptr(),
                bufs[5].data_ptr(), T, 0, packed.data_ptr(), 0, worst, info.data_ptr(), scratch.data_ptr(), need,
                info.data_ptr() + 4 * Bh, torch.cuda.current_stream().cuda_stream), "mfar_compress_quant")
        us = timed(runq, iters=iters, warmup=warmup)
        emit(f"prune+compress {name} 2-bit (kernel only)", us, x.numel() * 2, heads=Bh, tokens=L, sparsity=0.7)
        del st, x


def make_cache(B, L, s, seed=5):
    Bh = B * HKV
    cap = int(L * D * (1.0 - s + 0.25)) // 8 * 8
    ks = comp.SparseStore(Bh, L, comp.KEY, "cuda", nz_capacity=cap)
    vs = comp.SparseStore(Bh, L, comp.VALUE, "cuda", nz_capacity=cap)
    chunk = max(256, min(L, (1 << 27) // (Bh * D) // 256 * 256))
    for t0 in range(0, L, chunk):
        n = min(chunk, L - t0)
        ks.append(synth(Bh, n, seed + t0, True), comp.keep_rank(s))
        vs.append(synth(Bh, n, seed + t0 + 1, False), comp.keep_rank(s))
    return ks, vs


def bench_decode(quick):
    grid = [(1, 4096), (8, 4096)] if quick else [(b, l) for l in (4096, 16384, 32768) for b in (1, 8, 32, 64)]
    for B, L in grid:
        ks, vs = make_cache(B, L, 0.7)
        Bh = B * HKV
        kw, vw = synth(Bh, 128, 1, True), synth(Bh, 128, 2, False)
        q = synth(B * HQ, 1, 3, False).view(B * HQ, D)
        out = torch.empty_like(q)
        hint = max(ks.stage_hint(), vs.stage_hint())
        nbytes = store_bytes(ks) + store_bytes(vs) + 2 * 2 * Bh * 128 * D + 4 * B * HQ * D
        _, ws_bytes = ops.plan(Bh, L, 128, G)
        ws = ops.new_workspace(q.device, ws_bytes)
        us = timed(lambda: ops.decode_attention(q, ks, vs, kw, vw, G, out=out, stage_halves=hint, workspace=ws))
        emit("fused decode attention", us, nbytes, batch=B, kv_len=L, window=128, sparsity=0.7)
        us = timed_graph(lambda: ops.decode_attention(q, ks, vs, kw, vw, G, out=out, stage_halves=hint, workspace=ws))
        emit("fused decode attention (CUDA-graph replay)", us, nbytes, batch=B, kv_len=L, window=128, sparsity=0.7)
        ops.check_device_status()
        del ks, vs


def bench_decode_groups(quick):
    """Same cache, 1 / 2 / 4 / 8 query heads per kv head: the compressed bytes are read once per kv head whatever the
    group size, the FMAs grow with it."""
    B, L = (2, 4096) if quick else (32, 16384)
    ks, vs = make_cache(B, L, 0.7)
    Bh = B * HKV
    kw, vw = synth(Bh, 128, 1, True), synth(Bh, 128, 2, False)
    hint = max(ks.stage_hint(), vs.stage_hint())
    for group in (1, 2, 4, 8):
        q = synth(Bh * group, 1, 3, False).view(Bh * group, D)
        out = torch.empty_like(q)
        nbytes = store_bytes(ks) + store_bytes(vs) + 2 * 2 * Bh * 128 * D + 4 * Bh * group * D
        _, ws_bytes = ops.plan(Bh, L, 128, group)
        ws = ops.new_workspace(q.device, ws_bytes)
        us = timed_graph(lambda: ops.decode_attention(q, ks, vs, kw, vw, group, out=out, stage_halves=hint, workspace=ws))
        emit("fused decode attention (CUDA-graph replay)", us, nbytes, batch=B, kv_len=L, window=128, sparsity=0.7,
             q_heads_per_kv_head=group)
    ops.check_device_status()


def bench_ops(quick):
    B, L = (2, 4096) if quick else (8, 16384)
    ks, vs = make_cache(B, L, 0.7)
    Bh, Bq = B * HKV, B * HQ
    T = ks.tiles

    def ref_layout(st):
        lens = st.packed_lengths().tolist()
        nz = torch.cat([st.nz[h, :lens[h]] for h in range(st.n_heads)])
        idx = st.accum[:, :T + 1].contiguous()
        off = torch.zeros(st.n_heads, dtype=torch.int32, device="cuda")
        off[1:] = torch.cumsum(idx[:-1, -1] // 4, dim=0).to(torch.int32)
        return st.bitmaps[:, :T].contiguous(), nz, idx, off
    kb, knz, kidx, koff = ref_layout(ks)
    vb, vnz, vidx, voff = ref_layout(vs)
    q8 = torch.nn.functional.pad(synth(Bq, 1, 3, False), (0, 0, 0, 7)).contiguous()
    p8 = torch.nn.functional.pad(torch.softmax(torch.randn(Bq, 1, L, device="cuda"), -1).half(), (0, 0, 0, 7)).contiguous()
    ws = torch.zeros(1, dtype=torch.float16, device="cuda")
    us = timed(lambda: ops.mustafar_key_formulation(kb, knz, kidx, koff, q8, L, D, Bq, G))
    emit("mustafar_key_formulation (reference signature, incl. output memset)", us, store_bytes(ks) + 2 * Bq * L,
         batch=B, kv_len=L)
    us = timed(lambda: ops.mustafar_value_formulation(vb, vnz, vidx, voff, p8, ws, D, L, Bq, G))
    emit("mustafar_value_formulation (reference signature)", us, store_bytes(vs) + 2 * Bq * L, batch=B, kv_len=L)
    ops.check_device_status()


def bench_quant(quick, batch=None, kv_len=None, bit_list=(2, 4), sparsities=(0.5, 0.7), groups=(64, 32)):
    """Decode over the quantised cache.  group 64 = one scale / zero-point per tile (what the reference implements);
    group 32 = one per 32 nonzeros of a tile (the variant its write-up describes; oracle restatement only)."""
    B, L = (2, 4096) if quick else (32, 16384)
    B, L = batch or B, kv_len or L
    Bh = B * HKV
    for s in sparsities:
        for bits, group in [(b, g) for g in groups for b in bit_list]:
            kq = cq.compress_quant(synth(Bh, L, 21, True), comp.KEY, comp.keep_rank(s), bits, group)
            vq = cq.compress_quant(synth(Bh, L, 22, False), comp.VALUE, comp.keep_rank(s), bits, group)
            kw, vw = synth(Bh, 128, 1, True), synth(Bh, 128, 2, False)
            q = synth(B * HQ, 1, 3, False).view(B * HQ, D)
            nbytes = sum((8 + 4) * d["bitmaps"].numel() + 2 * (d["scales"].numel() + d["zeros"].numel()) +
                         4 * d["packed"].numel() for d in (kq, vq))
            nbytes += 2 * 2 * Bh * 128 * D + 4 * B * HQ * D
            us = timed(lambda: ops_quant.decode_attention_quant(q, kq, vq, L, kw, vw, G, bits))
            emit(f"fused decode attention {bits}-bit" + ("" if group == 64 else ", groups of 32 nonzeros"), us, nbytes,
                 batch=B, kv_len=L, window=128, sparsity=s)
            del kq, vq
    ops.check_device_status()


def bench_step(quick):
    """The launches around the attention call in one decode step of one layer (Llama-3-8B shape): RoPE + window append
    with and without the per-step pruning of the token that leaves the 128 most recent ones, residual add + RMSNorm,
    SiLU * up.  Replayed CUDA graphs (these kernels take a few microseconds)."""
    from . import step_ops
    B, cap, hidden, ffn = (4 if quick else 32), 384, 4096, 14336
    qkv = torch.randn(B, (HQ + 2 * HKV) * D, device="cuda").half()
    inv = step_ops.rope_inv_freq(500000.0, "cuda")
    q_out = torch.empty(B * HQ, D, dtype=torch.float16, device="cuda")
    kwin, vwin = synth(B * HKV, cap, 32, True), synth(B * HKV, cap, 33, False)
    io = 2 * qkv.numel() * 2
    for name, kw, extra in (("RoPE + window append", {}, 0),
                            ("RoPE + window append + prune of the token leaving the window (1 token/step)",
                             dict(prune_rank=comp.keep_rank(0.7), prune_back=128), 2 * 2 * B * HKV * D * 2)):
        us = timed_graph(lambda: step_ops.rope_append(qkv, inv, 5000, 300, HQ, HKV, q_out, kwin, vwin, **kw))
        emit(name, us, io + extra, batch=B, q_heads=HQ, kv_heads=HKV)
    x = torch.randn(B, hidden, device="cuda").half()
    d = torch.randn(B, hidden, device="cuda").half()
    w = torch.ones(hidden, device="cuda").half()
    o = torch.empty_like(x)
    us = timed_graph(lambda: step_ops.add_rmsnorm(x, d, w, 1e-5, out=o))
    emit("residual add + RMSNorm", us, 4 * x.numel() * 2 + hidden * 2, batch=B, hidden=hidden)
    gu = torch.randn(B, 2 * ffn, device="cuda").half()
    so = torch.empty(B, ffn, dtype=torch.float16, device="cuda")
    us = timed_graph(lambda: step_ops.silu_mul(gu, out=so))
    emit("SiLU(gate) * up", us, 3 * B * ffn * 2, batch=B, width=ffn)
    ops.check_device_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="compress,decode,decode_groups,ops,quant,step")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--quant-case", default="", help="batch,kv_len,bits,sparsity: run the quantised decode on this one case "
                                                     "(a small one to put under a profiler)")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    table = {"compress": bench_compress, "compress_fp16": bench_compress_fp16, "decode_groups": bench_decode_groups, "decode": bench_decode, "ops": bench_ops, "quant": bench_quant, "step": bench_step}
    if a.quant_case:
        b, l, bits, sp = a.quant_case.split(",")
        bench_quant(False, int(b), int(l), (int(bits),), (float(sp),), (64,))
        return
    for w in a.what.split(","):
        table[w](a.quick)


if __name__ == "__main__":
    main()
