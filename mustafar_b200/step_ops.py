"""Fused kernels for the one-token decode step around the sparse attention (C ABI ``mfar_add_rmsnorm_f16``,
``mfar_rope_append_f16``, ``mfar_silu_mul_f16``).  The reference's model file does this work with torch ops
(RMSNorm ``models/llama_mustafar_kernel.py:744,760``, rotary embedding ``:373-374``, the window ``torch.cat`` of
``:391`` / ``:430``, the MLP activation behind ``:761``); here a layer's glue is four launches.  CUDA only."""
from __future__ import annotations

import torch

from . import _lib

D = 128


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, what: str):
    if not t.is_cuda or t.dtype != torch.float16 or not t.is_contiguous():
        raise RuntimeError(f"{what}: expects a contiguous CUDA float16 tensor")


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """``x += delta`` in place (skipped when delta is None), returns ``rmsnorm(x) * weight``; x [rows, hidden]."""
    _need(x, "add_rmsnorm x")
    _need(weight, "add_rmsnorm weight")
    if delta is not None:
        _need(delta, "add_rmsnorm delta")
        if delta.shape != x.shape:
            raise RuntimeError("add_rmsnorm: delta and x differ in shape")
    hidden = x.shape[-1]
    if weight.numel() != hidden:
        raise RuntimeError("add_rmsnorm: weight does not match the hidden size")
    if out is None:
        out = torch.empty_like(x)
    _lib.check(_lib.lib().mfar_add_rmsnorm_f16(x.data_ptr(), None if delta is None else delta.data_ptr(), weight.data_ptr(),
                                               out.data_ptr(), x.numel() // hidden, hidden, float(eps), _stream()),
               "mfar_add_rmsnorm_f16")
    return out


def rope_inv_freq(theta: float, device) -> torch.Tensor:
    """fp32 [64] inverse frequencies, computed the way the torch expression it replaces computes them."""
    half = D // 2
    return (1.0 / (theta ** (torch.arange(0, half, device=device, dtype=torch.float32) / half))).contiguous()


def rope_append(qkv: torch.Tensor, inv_freq: torch.Tensor, pos, slot, n_q_heads: int, n_kv_heads: int,
                q_out: torch.Tensor, k_window: torch.Tensor, v_window: torch.Tensor,
                prune_rank: int = 0, prune_back: int = 0) -> torch.Tensor:
    """qkv [B, (hq + 2*hkv) * 128] of one new token per sequence: RoPE on q and k at position ``pos``; q ->
    q_out [B*hq, 128]; k, v -> k_window / v_window [B*hkv, cap, 128] at token slot ``slot``.  pos and slot are
    Python ints or CUDA int32 tensors of one element (read on the device at run time).  A device-resident slot
    outside the window writes nothing and is reported by ``ops.check_device_status``.
    ``prune_rank`` > 0 (see ``compression.keep_rank``): per-step pruning, the window token at ``slot - prune_back - 1``
    of every K and V head is magnitude-pruned in place by the same launch."""
    _need(qkv, "rope_append qkv")
    _need(q_out, "rope_append q_out")
    B = qkv.shape[0]
    if qkv.numel() != B * (n_q_heads + 2 * n_kv_heads) * D or q_out.numel() != B * n_q_heads * D:
        raise RuntimeError("rope_append: shapes do not match the head counts")
    for win in (k_window, v_window):
        if not win.is_cuda or win.dtype != torch.float16 or win.dim() != 3 or win.shape[0] != B * n_kv_heads \
                or win.shape[2] != D or win.stride(2) != 1:
            raise RuntimeError("rope_append: window must be CUDA float16 [B*hkv, cap, 128] with unit channel stride")
    if k_window.stride() != v_window.stride():
        raise RuntimeError("rope_append: key and value windows must share their strides")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != D // 2 or not inv_freq.is_cuda:
        raise RuntimeError("rope_append: inv_freq must be CUDA float32 [64]")

    def dev_or_host(v, name):
        if isinstance(v, torch.Tensor):
            if not v.is_cuda or v.dtype != torch.int32 or v.numel() != 1:
                raise RuntimeError(f"rope_append: {name} tensor must be CUDA int32 with one element")
            return v.data_ptr(), 0
        if int(v) < 0:
            raise RuntimeError(f"rope_append: negative {name}")
        return None, int(v)
    from .ops import _dev_status
    pd, ph = dev_or_host(pos, "pos")
    sd, sh = dev_or_host(slot, "slot")
    if sd is None and sh >= k_window.shape[1]:
        raise RuntimeError("rope_append: slot beyond the window capacity")
    _lib.check(_lib.lib().mfar_rope_append_f16(qkv.data_ptr(), inv_freq.data_ptr(), pd, ph, sd, sh, B, n_q_heads, n_kv_heads,
                                               q_out.data_ptr(), k_window.data_ptr(), v_window.data_ptr(),
                                               k_window.stride(0), k_window.stride(1), k_window.shape[1],
                                               int(prune_rank), int(prune_back),
                                               _dev_status(qkv.device).data_ptr(), _stream()),
               "mfar_rope_append_f16")
    return q_out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """gate_up [rows, 2*width] -> silu(gate) * up, [rows, width]."""
    _need(gate_up, "silu_mul gate_up")
    width = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * width)
    if out is None:
        out = torch.empty(gate_up.shape[:-1] + (width,), dtype=torch.float16, device=gate_up.device)
    _lib.check(_lib.lib().mfar_silu_mul_f16(gate_up.data_ptr(), out.data_ptr(), rows, width, _stream()), "mfar_silu_mul_f16")
    return out
