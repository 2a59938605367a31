"""Decode ops over the quantised cache, with the signatures of the reference extension
``mustafar_package_quant`` (``kernel_quant/kernel_wrapper/pybind_quant.cpp:10-177``).

``dequant_mode``, ``split_k``, ``value_tile_config`` and the optional counts / units
metadata are accepted and do not change the result: values are always
``fp16((code - zero) * scale)`` in fp32 arithmetic (the reference's mode 0).  Unlike the
reference's ``decode_n1`` / tile-64 experiments (which index tiles in an order the
compressor does not emit) every entry returns the mathematically correct product.
"""
from __future__ import annotations

import math

import torch

from . import _lib
from .compression import D, _stream
from .ops import _debug_check, _dev_status, _take_workspace, _workspace, check_device_status, plan


def _check(bmp, NZ_quant, tile_offsets, scales, zeros, B):
    dev = B.device
    ts = (bmp, NZ_quant, tile_offsets, scales, zeros)
    if any(t.device != dev for t in ts):
        raise RuntimeError("All input tensors must be on the same device.")
    if not all(t.is_cuda for t in ts + (B,)):
        raise RuntimeError("all tensors must be on a CUDA device.")
    if B.dtype != torch.float16:
        raise RuntimeError("Tensor B must be of type float16.")
    if NZ_quant.dtype != torch.int32:
        raise RuntimeError("Tensor NZ_quant must be of type int32.")
    if bmp.dtype != torch.int64:
        raise RuntimeError("Tensor bmp must be of type int64.")
    if tile_offsets.dtype != torch.int32:
        raise RuntimeError("Tensor tile_offsets must be of type int32.")
    if scales.dtype != torch.float16 or zeros.dtype != torch.float16:
        raise RuntimeError("Tensors scales and zeros must be of type float16.")
    if not all(t.is_contiguous() for t in ts):
        raise RuntimeError("bmp, NZ_quant, tile_offsets, scales and zeros must be contiguous.")


def _qgroup(scales, n_kv, tiles):
    per_tile = scales.numel() // max(1, n_kv * tiles)
    if per_tile not in (1, 2) or per_tile * n_kv * tiles != scales.numel():
        raise RuntimeError("scales has an unexpected number of entries")
    return 64 if per_tile == 1 else 32


def mustafar_key_formulation_quant(bmp, NZ_quant, tile_offsets, scales, zeros, B, M_Global, K_Global, Batch_Size,
                                   num_key_value_groups, bit, capacity, dequant_mode=0):
    """S = dequant(K~) q; B [Batch_Size, 8, 128] (row 0 = the query) -> fp16 [Batch_Size, 8, M_Global]."""
    _check(bmp, NZ_quant, tile_offsets, scales, zeros, B)
    if K_Global != D or M_Global % 64 or Batch_Size % num_key_value_groups or bit * capacity != 32:
        raise RuntimeError("unsupported shape: head_dim 128, M_Global % 64 == 0, bit * capacity == 32")
    if not B.is_contiguous():
        raise RuntimeError("B must be contiguous.")
    n_kv = Batch_Size // num_key_value_groups
    tiles = M_Global * K_Global // 64
    out = torch.zeros((Batch_Size, 8, M_Global), dtype=torch.float16, device=B.device)
    st = _dev_status(B.device)
    rows = B.shape[1] if B.dim() == 3 else 1
    r = _lib.lib().mfar_key_scores_quant(
        B.data_ptr(), rows * K_Global, n_kv, num_key_value_groups, bmp.data_ptr(), tiles, tile_offsets.data_ptr(),
        scales.data_ptr(), zeros.data_ptr(), tiles, NZ_quant.data_ptr(), NZ_quant.numel(), M_Global, bit,
        _qgroup(scales, n_kv, tiles), out.data_ptr(), 8 * M_Global, st.data_ptr(), _stream())
    _lib.check(r, "mfar_key_scores_quant")
    if _debug_check():
        check_device_status(B.device)
    return out


def mustafar_key_formulation_quant_meta(bmp, NZ_quant, tile_offsets, tile_counts, tile_units, scales, zeros, B,
                                        M_Global, K_Global, Batch_Size, num_key_value_groups, bit, capacity,
                                        dequant_mode=0):
    """As ``mustafar_key_formulation_quant``; counts / units are redundant with the bitmaps and unused."""
    return mustafar_key_formulation_quant(bmp, NZ_quant, tile_offsets, scales, zeros, B, M_Global, K_Global,
                                          Batch_Size, num_key_value_groups, bit, capacity, dequant_mode)


def _value(bmp, NZ_quant, tile_offsets, scales, zeros, P, probs_stride, M_Global, K_Global, Batch_Size, groups, bit,
           capacity, out, out_stride, split_k):
    _check(bmp, NZ_quant, tile_offsets, scales, zeros, P)
    if M_Global != D or K_Global % 64 or Batch_Size % groups or bit * capacity != 32:
        raise RuntimeError("unsupported shape: head_dim 128, K_Global % 64 == 0, bit * capacity == 32")
    n_kv = Batch_Size // groups
    tiles = M_Global * K_Global // 64
    _, nbytes = plan(n_kv, K_Global, 0, groups)
    ws = _workspace(P.device, max(nbytes, 65536 + n_kv * max(1, K_Global // 64) * groups * 132 * 4))
    st = _dev_status(P.device)
    r = _lib.lib().mfar_value_output_quant(
        P.data_ptr(), probs_stride, n_kv, groups, bmp.data_ptr(), tiles, tile_offsets.data_ptr(), scales.data_ptr(),
        zeros.data_ptr(), tiles, NZ_quant.data_ptr(), NZ_quant.numel(), K_Global, bit, _qgroup(scales, n_kv, tiles),
        out.data_ptr(), out_stride, ws.data_ptr(), ws.numel(), 0, st.data_ptr(), _stream())
    _lib.check(r, "mfar_value_output_quant")
    if _debug_check():
        check_device_status(P.device)
    return out


def mustafar_value_formulation_quant(bmp, NZ_quant, tile_offsets, tile_counts, tile_units, scales, zeros, B,
                                     Reduction_Workspace, M_Global, K_Global, Batch_Size, num_key_value_groups, bit,
                                     capacity, dequant_mode=0, split_k=1, value_tile_config=0):
    """O = dequant(V~)^T p; B [Batch_Size, 8, L] (row 0 = probabilities) -> fp16 [Batch_Size, 8, 128]."""
    Bc = B if B.is_contiguous() else B.contiguous()
    out = torch.zeros((Batch_Size, 8, M_Global), dtype=torch.float16, device=B.device)
    rows = Bc.shape[1] if Bc.dim() == 3 else 1
    return _value(bmp, NZ_quant, tile_offsets, scales, zeros, Bc, rows * K_Global, M_Global, K_Global, Batch_Size,
                  num_key_value_groups, bit, capacity, out, 8 * M_Global, split_k)


def mustafar_value_formulation_quant_decode_n1(bmp, NZ_quant, tile_offsets, tile_counts, tile_units, scales, zeros,
                                               score, Reduction_Workspace, M_Global, K_Global, Batch_Size,
                                               num_key_value_groups, bit, capacity, dequant_mode=0, split_k=1):
    """Decode-only form: score [Batch_Size, L] -> fp16 [Batch_Size, 128]."""
    sc = score if score.is_contiguous() else score.contiguous()
    if sc.dim() != 2 or sc.shape[1] != K_Global:
        raise RuntimeError("score must be [Batch_Size, K_Global]")
    out = torch.empty((Batch_Size, M_Global), dtype=torch.float16, device=score.device)
    return _value(bmp, NZ_quant, tile_offsets, scales, zeros, sc, K_Global, M_Global, K_Global, Batch_Size,
                  num_key_value_groups, bit, capacity, out, M_Global, split_k)


# aliases kept by the reference for its model code (pybind_quant.cpp:95-177)
mustafar_quant_sparse_forward = mustafar_key_formulation_quant
mustafar_quant_sparse_forward_meta = mustafar_key_formulation_quant_meta
mustafar_quant_sparse_value_forward = mustafar_value_formulation_quant
mustafar_quant_sparse_value_forward_decode_n1 = mustafar_value_formulation_quant_decode_n1


def decode_attention_quant(q, kq: dict, vq: dict, n_tokens: int, k_window, v_window, group: int, bits: int = 2,
                           softmax_scale: float | None = None, nsplit: int = 0, out: torch.Tensor | None = None,
                           n_tokens_dev: torch.Tensor | None = None, window_len: torch.Tensor | None = None,
                           workspace: torch.Tensor | None = None):
    """Fused decode attention over two quantised tensors (dicts as returned by
    ``compression_quant.compress_quant`` or ``QuantStore.as_dict``) plus the dense fp16 window, one launch.
    Dequantised values are ``fp16((code - zero) * scale)`` as in the reference's kernels.
    ``n_tokens_dev`` / ``window_len``: optional CUDA int32 tensors [1] with the current compressed length (then
    ``n_tokens`` is its upper bound and sizes the launch) / window length (the window tensors give the capacity),
    so that a captured launch can be replayed while the cache grows; ``workspace`` as in ``ops.decode_attention``."""
    n_kv = kq["bitmaps"].shape[0]
    tiles = 2 * n_tokens
    if q.shape != (n_kv * group, D) or q.dtype != torch.float16 or not q.is_cuda:
        raise RuntimeError("q must be CUDA float16 [n_kv_heads*group, 128]")
    if q.stride(1) != 1 or q.stride(0) % 2 or q.data_ptr() % 4:
        q = q.contiguous()
    W, kw, vw, wh, wt = 0, None, None, 0, 0
    if k_window is not None and k_window.shape[1] > 0:
        if k_window.stride() != v_window.stride() or k_window.stride(2) != 1:
            k_window, v_window = k_window.contiguous(), v_window.contiguous()
        W, kw, vw = k_window.shape[1], k_window.data_ptr(), v_window.data_ptr()
        wh, wt = k_window.stride(0), k_window.stride(1)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty((n_kv * group, D), dtype=torch.float16, device=q.device)
    ws = _take_workspace(workspace, q.device, 65536 + n_kv * (max(1, n_tokens // 64) + 1) * group * 132 * 4)
    for t, name in ((n_tokens_dev, "n_tokens_dev"), (window_len, "window_len")):
        if t is not None and (not t.is_cuda or t.dtype != torch.int32 or t.numel() != 1):
            raise RuntimeError(f"{name} must be a CUDA int32 tensor with one element")
    st = _dev_status(q.device)
    # compact tensors hold exactly `tiles` tiles per head; an arena (QuantStore.as_dict) says how far apart heads are
    hs = int(kq.get("head_stride", tiles))
    if int(vq.get("head_stride", tiles)) != hs:
        raise RuntimeError("key and value tensors must share their head stride")
    qg = _qgroup(kq["scales"], n_kv, hs) if n_tokens else 64
    r = _lib.lib().mfar_decode_attention_quant(
        q.data_ptr(), q.stride(0), n_kv, group,
        kq["bitmaps"].data_ptr(), kq["tile_offsets"].data_ptr(), kq["scales"].data_ptr(), kq["zeros"].data_ptr(),
        kq["packed"].data_ptr(), kq["packed"].numel(),
        vq["bitmaps"].data_ptr(), vq["tile_offsets"].data_ptr(), vq["scales"].data_ptr(), vq["zeros"].data_ptr(),
        vq["packed"].data_ptr(), vq["packed"].numel(),
        hs, hs, n_tokens, None if n_tokens_dev is None else n_tokens_dev.data_ptr(), bits, qg, kw, vw, wh, wt, W,
        None if window_len is None else window_len.data_ptr(), float(softmax_scale), out.data_ptr(), out.stride(0),
        ws.data_ptr(), ws.numel(), nsplit, st.data_ptr(), _stream())
    _lib.check(r, "mfar_decode_attention_quant")
    if _debug_check():
        check_device_status(q.device)
    return out
