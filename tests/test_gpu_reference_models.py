"""The reference's own model files, unmodified, on top of this library.

``models/llama_mustafar_kernel.py`` and ``models/llama_mustafar_quant_kernel.py`` are imported from a reference
checkout (never copied into this repository): the directory named by ``MUSTAFAR_REFERENCE``, else
``baseline/_ref`` (git-ignored; ``oracle.build_ref.stage_model_files`` puts the two files there), else the
test is skipped.  ``compat.install()`` provides ``mustafar_package`` / ``mustafar_package_quant`` /
``kernel.compression`` / ``kernel_quant.compression_quant``; ``hf_shim.install()`` lets the files import under
the installed ``transformers``.

Each file's ``LlamaForCausalLM_MUSTAFAR`` (2 random-init layers, 8 query / 2 kv heads, sparsity 0.7, residual
window 128, the settings of ``benchmark/mem_spd_test.py:71-81``) prefills 895 tokens (512 compressed, a 383-token
window) and decodes 6 tokens, which crosses one 256-token append (``models/llama_mustafar_kernel.py:445-519``).
The same model object then repeats the run with its extension replaced by an emulation built on the CPU oracle
(decompress / dequantise, dense fp32 products, one fp16 rounding); the logits of the two runs must agree."""
import importlib
import os
import sys
import types

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_root():
    for cand in (os.environ.get("MUSTAFAR_REFERENCE"), os.path.join(ROOT, "baseline", "_ref")):
        if cand and os.path.exists(os.path.join(cand, "models", "llama_mustafar_kernel.py")):
            return cand
    return None


def load_reference_module(name):
    ref = reference_root()
    if ref is None:
        pytest.skip("no reference checkout (set MUSTAFAR_REFERENCE or run oracle.build_ref.stage_model_files)")
    try:
        import flash_attn  # noqa: F401  (the reference's prefill calls flash_attn_func)
    except Exception:
        pytest.skip("flash_attn is not installed")
    from mustafar_b200 import compat, hf_shim
    compat.install()
    hf_shim.install()
    if ref not in sys.path:
        sys.path.insert(0, ref)
    return importlib.import_module(f"models.{name}")


def make_model(mod, **extra):
    from mustafar_b200 import hf_shim
    cfg = hf_shim.llama_config(hidden_size=1024, intermediate_size=2048, num_hidden_layers=2, num_attention_heads=8,
                               num_key_value_heads=2, vocab_size=2048, max_position_embeddings=4096,
                               k_sparsity=0.7, v_sparsity=0.7, residual_length=128)
    for k, v in extra.items():
        setattr(cfg, k, v)
    torch.manual_seed(1234)
    model = mod.LlamaForCausalLM_MUSTAFAR(cfg)
    return model.half().cuda().eval()


@torch.no_grad()
def run(model, ids, steps):
    """The reference's own driver loop (``benchmark/low_memory_generation.py:5-58``) with the next token forced, so
    that both runs see the same inputs: returns the logits of the prefill and of every decode step."""
    logits, past = [], None
    cur = ids
    for t in range(steps + 1):
        out = model.model(input_ids=cur, attention_mask=None, past_key_values=past, use_cache=True, return_dict=True)
        past = out.past_key_values
        logits.append(model.lm_head(out.last_hidden_state[:, -1:, :]).float())
        cur = ((ids[:, :1] * 31 + 7 * (t + 1)) % model.config.vocab_size)     # fixed, run-independent next tokens
    return torch.cat(logits, dim=1), past


# ----------------------------------------------------------------- oracle-backed stand-ins for the two extensions
def emulated_fp16_extension():
    def conv(fn):
        def convert(x):
            bmp, acc, packed = fn(x.detach().cpu())
            dev = x.device
            return (torch.from_numpy(bmp).to(dev), torch.from_numpy(acc).to(dev), [torch.from_numpy(p).to(dev) for p in packed])
        return convert

    def unpack(bmp, NZ, idx, off, Bh, L, fn):
        T = L * 128 // 64
        b, a = bmp.reshape(Bh, T).cpu().numpy(), idx.reshape(Bh, T + 1).cpu().numpy()
        nz, o = NZ.cpu().numpy(), off.cpu().numpy()
        packed = [nz[8 * int(o[h]): 8 * int(o[h]) + 2 * int(a[h, -1])] for h in range(Bh)]
        return fn(b, a, packed, L)

    def key(bmp, NZ, idx, off, B, M, K, Batch, G):
        dense = unpack(bmp, NZ, idx, off, Batch // G, M, oracle.decompress_key_ref)
        out = torch.zeros(Batch, 8, M, dtype=torch.float16, device=B.device)
        out[:, 0] = oracle.key_formulation_ref(dense, B[:, 0].cpu(), G).to(B.device)
        return out

    def value(bmp, NZ, idx, off, B, ws, M, K, Batch, G):
        dense = unpack(bmp, NZ, idx, off, Batch // G, K, oracle.decompress_value_ref)
        out = torch.zeros(Batch, 8, M, dtype=torch.float16, device=B.device)
        out[:, 0] = oracle.value_formulation_ref(dense, B[:, 0].cpu(), G).to(B.device)
        return out

    ext = types.SimpleNamespace(mustafar_key_formulation=key, mustafar_value_formulation=value)
    comp = types.SimpleNamespace(convert_key_batched=conv(oracle.compress_key_ref),
                                 convert_value_batched=conv(oracle.compress_value_ref))
    return ext, comp


def emulated_quant_extension():
    order = ("bitmaps", "tile_offsets", "packed", "counts", "units", "scales", "zeros")

    def conv(fn):
        def convert(x, return_metadata=True):
            fmt = fn(x.detach().cpu(), bits=2, group=64)
            t = [torch.from_numpy(np.ascontiguousarray(fmt[k])).to(x.device) for k in order]
            return tuple(t) if return_metadata else (t[0], t[1], t[2], t[5], t[6])
        return convert

    def dense(bmp, NZq, offs, scales, zeros, Bh, L, fn):
        T = L * 128 // 64
        fmt = dict(bitmaps=bmp.reshape(Bh, T).cpu().numpy(), tile_offsets=offs.reshape(Bh, T).cpu().numpy(),
                   packed=NZq.cpu().numpy(), scales=scales.reshape(Bh, T).cpu().numpy(),
                   zeros=zeros.reshape(Bh, T).cpu().numpy())
        return fn(fmt, L, bits=2, group=64)

    def key(bmp, NZq, offs, scales, zeros, B, M, K, Batch, G, bit, capacity, dequant_mode=0):
        d = dense(bmp, NZq, offs, scales, zeros, Batch // G, M, oracle.dequant_key_ref)
        out = torch.zeros(Batch, 8, M, dtype=torch.float16, device=B.device)
        out[:, 0] = oracle.key_formulation_ref(d, B[:, 0].cpu(), G).to(B.device)
        return out

    def key_meta(bmp, NZq, offs, counts, units, scales, zeros, B, M, K, Batch, G, bit, capacity, dequant_mode=0):
        return key(bmp, NZq, offs, scales, zeros, B, M, K, Batch, G, bit, capacity, dequant_mode)

    def value(bmp, NZq, offs, counts, units, scales, zeros, B, ws, M, K, Batch, G, bit, capacity, dequant_mode=0,
              split_k=1, value_tile_config=0):
        d = dense(bmp, NZq, offs, scales, zeros, Batch // G, K, oracle.dequant_value_ref)
        out = torch.zeros(Batch, 8, M, dtype=torch.float16, device=B.device)
        out[:, 0] = oracle.value_formulation_ref(d, B[:, 0].cpu(), G).to(B.device)
        return out

    def value_n1(bmp, NZq, offs, counts, units, scales, zeros, score, ws, M, K, Batch, G, bit, capacity, dequant_mode=0,
                 split_k=1):
        d = dense(bmp, NZq, offs, scales, zeros, Batch // G, K, oracle.dequant_value_ref)
        return oracle.value_formulation_ref(d, score.cpu(), G).to(score.device)

    ext = types.SimpleNamespace(mustafar_key_formulation_quant=key, mustafar_key_formulation_quant_meta=key_meta,
                                mustafar_value_formulation_quant=value,
                                mustafar_value_formulation_quant_decode_n1=value_n1)
    comp = types.SimpleNamespace(convert_key_batched_quant=conv(oracle.quant_compress_key_ref),
                                 convert_value_batched_quant=conv(oracle.quant_compress_value_ref))
    return ext, comp


def compare(a, b, what):
    err = oracle.rel_l2(a.cpu(), b.cpu())
    assert err < 5e-3, (what, err)
    # greedy choices agree wherever the top-2 margin is larger than the numerical noise
    ta, tb = a.argmax(-1), b.argmax(-1)
    top2 = a.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 0.05
    assert torch.equal(ta[clear], tb[clear]), what


def test_fp16_reference_model_runs_unchanged_on_the_drop_in():
    mod = load_reference_module("llama_mustafar_kernel")
    model = make_model(mod)
    ids = torch.randint(0, 2048, (2, 895), generator=torch.Generator().manual_seed(5)).cuda()
    real_ext, real_comp = mod.mustafar_package, mod.compression
    assert real_ext.__doc__.startswith("mustafar_b200"), "the model must be bound to this library's drop-in"
    got, past = run(model, ids, 6)
    k_compressed, k_window, v_compressed, v_window, compressed_length, kv_len = past[0]
    assert compressed_length == 768 and kv_len == 895 + 6 and k_window.shape[2] == kv_len - 768
    assert k_compressed[0].numel() == 4 * 768 * 2            # bitmaps of 2 sequences x 2 kv heads
    ext, comp = emulated_fp16_extension()
    mod.mustafar_package, mod.compression = ext, comp
    try:
        want, _ = run(model, ids, 6)
    finally:
        mod.mustafar_package, mod.compression = real_ext, real_comp
    compare(got, want, "fp16 sparse model")
    assert model.model.layers[0].self_attn.latest_compression_stats["compressed_length"] == 512


@pytest.mark.parametrize("variant", [dict(), dict(quant_k_use_meta=True, quant_v_decode_n1=True)])
def test_quantised_reference_model_runs_unchanged_on_the_drop_in(variant):
    mod = load_reference_module("llama_mustafar_quant_kernel")
    model = make_model(mod, quant_bits=2, **variant)
    ids = torch.randint(0, 2048, (2, 895), generator=torch.Generator().manual_seed(6)).cuda()
    real_ext, real_comp = mod.mustafar_package_quant, mod.compression_quant
    assert real_ext.__doc__.startswith("mustafar_b200")
    got, past = run(model, ids, 6)
    assert past[0][4] == 768
    ext, comp = emulated_quant_extension()
    mod.mustafar_package_quant, mod.compression_quant = ext, comp
    try:
        want, _ = run(model, ids, 6)
    finally:
        mod.mustafar_package_quant, mod.compression_quant = real_ext, real_comp
    compare(got, want, f"2-bit model {variant}")
