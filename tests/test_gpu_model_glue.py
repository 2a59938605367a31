"""Drives the drop-in modules the way the reference attention layer does during decode
(models/llama_mustafar_kernel.py:377-521 and models/llama_mustafar_quant_kernel.py:426-662):
prefill compression, per-step key op / softmax / value op with 8-row padded operands, and the
256-token block append that splices new tiles into the cache.  The result of every step is
compared with dense attention over the pruned (or dequantised) tensors from the CPU oracle."""
import math
import os

import pytest
import torch
import torch.nn.functional as F

import oracle

pytestmark = pytest.mark.gpu
D = 128


@pytest.fixture(scope="module")
def mods():
    os.environ["MUSTAFAR_B200_CHECK"] = "1"
    from mustafar_b200 import compat, compression as native
    compat.install()
    import mustafar_package
    import mustafar_package_quant
    import kernel.compression as compression
    import kernel_quant.compression_quant as compression_quant
    yield mustafar_package, mustafar_package_quant, compression, compression_quant, native
    compat.uninstall()


def repeat_kv(x, n):
    b, h, t, d = x.shape
    return x if n == 1 else x[:, :, None].expand(b, h, n, t, d).reshape(b, h * n, t, d)


def prune(native, x, s):
    return native.prune(x.contiguous(), s)          # the GPU stand-in for dh_prune_key / dh_prune_value


def nz_offsets(idxs):
    off = torch.zeros(idxs.shape[0], dtype=torch.int32, device=idxs.device)
    for i in range(1, idxs.shape[0]):
        off[i] = off[i - 1] + idxs[i - 1][-1] // 4
    return off


def test_fp16_decode_loop_with_block_append(mods):
    pkg, _, compression, _, native = mods
    B, Hkv, G, s, residual = 2, 2, 4, 0.7, 32
    Hq, Bh, Bq = Hkv * G, B * Hkv, B * Hkv * G
    prompt, steps = 256 + residual + 250, 12          # the window reaches residual + 256 inside the loop
    k_all, v_all = oracle.make_kv(Bh, prompt + steps, seed=2024)
    k_all, v_all = k_all.view(B, Hkv, -1, D).cuda(), v_all.view(B, Hkv, -1, D).cuda()

    # ---- prefill (models/llama_mustafar_kernel.py:540-560)
    L = ((prompt - residual) // 256) * 256
    kc = prune(native, k_all[:, :, :L], s)
    vc = prune(native, v_all[:, :, :L], s)
    k_bmps, k_idxs, k_nzs = compression.convert_key_batched(kc.reshape(Bh, -1, D))
    v_bmps, v_idxs, v_nzs = compression.convert_value_batched(vc.reshape(Bh, -1, D))
    k_comp = [k_bmps, k_idxs, k_nzs, nz_offsets(k_idxs)]
    v_comp = [v_bmps, v_idxs, v_nzs, nz_offsets(v_idxs)]
    k_win, v_win = k_all[:, :, L:prompt].clone(), v_all[:, :, L:prompt].clone()
    pruned_k, pruned_v = kc.cpu(), vc.cpu()
    ws = torch.zeros(1, dtype=torch.float16, device="cuda")
    appended = 0

    for step in range(steps):
        pos = prompt + step
        q = oracle.make_query(Bq, seed=500 + step).view(B, Hq, 1, D).cuda()
        k_win = torch.cat([k_win, k_all[:, :, pos:pos + 1]], dim=2)
        v_win = torch.cat([v_win, v_all[:, :, pos:pos + 1]], dim=2)
        padded_q = F.pad(q.view(Bq, -1, D), (0, 0, 0, 7))
        att_c = pkg.mustafar_key_formulation(k_comp[0], torch.cat(k_comp[2]), k_comp[1], k_comp[3], padded_q, L, D, Bq, G)
        att_c = att_c[:, 0:1, :].view(B, Hq, 1, L)
        att_l = torch.matmul(q, repeat_kv(k_win, G).transpose(2, 3))
        w = torch.cat([att_c, att_l], dim=-1) / math.sqrt(D)
        w = F.softmax(w, dim=-1, dtype=torch.float32).to(q.dtype)
        padded_p = F.pad(w[:, :, :, :L].view(Bq, -1, L), (0, 0, 0, 7)).contiguous()
        out_c = pkg.mustafar_value_formulation(v_comp[0], torch.cat(v_comp[2]), v_comp[1], v_comp[3], padded_p, ws, D, L, Bq, G)
        out = out_c[:, 0:1, :].view(B, Hq, 1, D) + torch.matmul(w[:, :, :, L:], repeat_kv(v_win, G))

        want = oracle.decode_attention_ref(q.view(Bq, D).cpu(), pruned_k.reshape(Bh, -1, D), pruned_v.reshape(Bh, -1, D),
                                           k_win.reshape(Bh, -1, D).cpu(), v_win.reshape(Bh, -1, D).cpu(), G)
        assert oracle.rel_l2(out.view(Bq, D).float().cpu(), want) < 4e-3, step     # model order: several fp16 roundings

        # ---- block append (models/llama_mustafar_kernel.py:445-519)
        if (pos + 1 - residual - L) % 256 == 0:
            nk = prune(native, k_win[:, :, :256], s)
            nv = prune(native, v_win[:, :, :256], s)
            for comp, new, fn in ((k_comp, nk, compression.convert_key_batched), (v_comp, nv, compression.convert_value_batched)):
                n_bmps, n_idxs, n_nzs = fn(new.reshape(Bh, -1, D))
                last = torch.tensor([int(i[-1]) for i in n_idxs[:-1]], device="cuda")
                comp[3][1:] += torch.cumsum(last // 4, dim=0).to(torch.int32)
                base = comp[1].view(Bh, -1)[:, -1].unsqueeze(1)
                comp[1] = torch.cat([comp[1].view(Bh, -1)[:, :-1], n_idxs.view(Bh, -1) + base], dim=1).flatten()
                comp[0] = torch.cat([comp[0].view(Bh, 2 * L), n_bmps.view(Bh, 512)], dim=1).flatten()
                comp[2] = [torch.cat([comp[2][b], n_nzs[b]]) for b in range(Bh)]
            pruned_k = torch.cat([pruned_k, nk.cpu()], dim=2)
            pruned_v = torch.cat([pruned_v, nv.cpu()], dim=2)
            k_win, v_win = k_win[:, :, 256:].clone(), v_win[:, :, 256:].clone()
            L += 256
            appended += 1
    assert appended == 1 and L == 512


def test_quant_decode_loop_with_block_append(mods):
    _, pkgq, _, cq, native = mods
    B, Hkv, G, s, residual = 1, 2, 4, 0.5, 32
    Hq, Bh, Bq = Hkv * G, B * Hkv, B * Hkv * G
    prompt, steps = 256 + residual + 252, 8
    k_all, v_all = oracle.make_kv(Bh, prompt + steps, seed=77)
    k_all, v_all = k_all.view(B, Hkv, -1, D).cuda(), v_all.view(B, Hkv, -1, D).cuda()
    L = ((prompt - residual) // 256) * 256

    def comp_k(x):
        b, off, pk, cnt, un, sc, ze = cq.convert_key_batched_quant(x.reshape(Bh, -1, D), return_metadata=True)
        return [b, off, [pk], cnt, un, sc, ze]

    def comp_v(x):
        b, off, pk, cnt, un, sc, ze = cq.convert_value_batched_quant(x.reshape(Bh, -1, D))
        return [b, off, [pk], cnt, un, sc, ze]

    def append(c, n):                                   # models/llama_mustafar_quant_kernel.py:322-345
        n[1] = n[1] + c[2][0].numel()
        for i in (0, 1, 3, 4, 5, 6):
            c[i] = torch.cat([c[i], n[i]], dim=1)
        c[2] = [torch.cat([c[2][0], n[2][0]])]

    def dequant(x, kind):
        fn = oracle.quant_compress_key_ref if kind == "k" else oracle.quant_compress_value_ref
        de = oracle.dequant_key_ref if kind == "k" else oracle.dequant_value_ref
        xr = x.reshape(Bh, -1, D).cpu()
        return torch.from_numpy(de(fn(xr), xr.shape[1]))

    kc, vc = prune(native, k_all[:, :, :L], s), prune(native, v_all[:, :, :L], s)
    k_comp, v_comp = comp_k(kc), comp_v(vc)
    dk, dv = dequant(kc, "k"), dequant(vc, "v")
    k_win, v_win = k_all[:, :, L:prompt].clone(), v_all[:, :, L:prompt].clone()
    ws = torch.zeros(1, dtype=torch.float16, device="cuda")
    appended = 0
    for step in range(steps):
        pos = prompt + step
        q = oracle.make_query(Bq, seed=900 + step).view(B, Hq, 1, D).cuda()
        k_win = torch.cat([k_win, k_all[:, :, pos:pos + 1]], dim=2)
        v_win = torch.cat([v_win, v_all[:, :, pos:pos + 1]], dim=2)
        padded_q = F.pad(q.view(Bq, -1, D), (0, 0, 0, 7))
        att_c = pkgq.mustafar_key_formulation_quant_meta(k_comp[0], k_comp[2][0], k_comp[1], k_comp[3], k_comp[4],
                                                         k_comp[5], k_comp[6], padded_q, L, D, Bq, G, 2, 16, 0)
        att_c = att_c[:, 0:1, :].view(B, Hq, 1, L)
        att_l = torch.matmul(q, repeat_kv(k_win, G).transpose(2, 3))
        w = F.softmax(torch.cat([att_c, att_l], dim=-1) / math.sqrt(D), dim=-1, dtype=torch.float32).to(q.dtype)
        if step % 2 == 0:
            padded_p = F.pad(w[:, :, :, :L].view(Bq, -1, L), (0, 0, 0, 7)).contiguous()
            out_c = pkgq.mustafar_value_formulation_quant(v_comp[0], v_comp[2][0], v_comp[1], v_comp[3], v_comp[4],
                                                          v_comp[5], v_comp[6], padded_p, ws, D, L, Bq, G, 2, 16, 0, 4, 2)
            out_c = out_c[:, 0:1, :].view(B, Hq, 1, D)
        else:
            score = w[:, :, :, :L].reshape(Bq, L).contiguous()
            out_c = pkgq.mustafar_value_formulation_quant_decode_n1(v_comp[0], v_comp[2][0], v_comp[1], v_comp[3],
                                                                    v_comp[4], v_comp[5], v_comp[6], score, ws, D, L,
                                                                    Bq, G, 2, 16, 0, 4).view(B, Hq, 1, D)
        out = out_c + torch.matmul(w[:, :, :, L:], repeat_kv(v_win, G))
        want = oracle.decode_attention_ref(q.view(Bq, D).cpu(), dk, dv, k_win.reshape(Bh, -1, D).cpu(),
                                           v_win.reshape(Bh, -1, D).cpu(), G)
        assert oracle.rel_l2(out.view(Bq, D).float().cpu(), want) < 4e-3, step
        if (pos + 1 - residual - L) % 256 == 0:
            nk, nv = prune(native, k_win[:, :, :256], s), prune(native, v_win[:, :, :256], s)
            append(k_comp, comp_k(nk))
            append(v_comp, comp_v(nv))
            dk, dv = torch.cat([dk, dequant(nk, "k")], dim=1), torch.cat([dv, dequant(nv, "v")], dim=1)
            k_win, v_win = k_win[:, :, 256:].clone(), v_win[:, :, 256:].clone()
            L += 256
            appended += 1
    assert appended == 1
