"""Decode ops over the fp16 compressed cache.

``mustafar_key_formulation`` / ``mustafar_value_formulation`` keep the positional
signatures, checks and return shapes of the reference extension
``mustafar_package`` (``kernel/kernel_wrapper/mustafar_wrapper.cu:19-133``,
``:139-263``; ``pybind.cpp:9-10``).  ``decode_attention`` is the fused entry
(one call per layer per step) over two ``SparseStore`` arenas.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import torch

from . import _lib
from .compression import D, SparseStore, _stream

_workspaces: dict = {}
_status: dict = {}


def _debug_check() -> bool:
    """MUSTAFAR_B200_CHECK=1: synchronise after every op and raise on device-reported errors
    (never while the stream is being captured into a CUDA graph, where a sync is illegal)."""
    return os.environ.get("MUSTAFAR_B200_CHECK", "0") == "1" and not torch.cuda.is_current_stream_capturing()


def new_workspace(device, nbytes: int) -> torch.Tensor:
    """A decode workspace of at least ``nbytes`` (see ``plan``).  Zero-filled: its first bytes are the arrival
    counters of the fused attention kernel, which every call leaves at zero again."""
    return torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)


def _workspace(device, nbytes: int) -> torch.Tensor:
    """Default workspace: one per (device, stream), grown on demand.  A caller that captures CUDA graphs or runs
    decode calls on several streams hands its own buffer to ``decode_attention(workspace=...)`` instead: growing
    this one while a captured graph still holds the old pointer would leave the graph writing into freed memory,
    so growth during capture is refused."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("decode workspace would have to grow during CUDA graph capture: pass workspace= "
                               "(ops.new_workspace sized by ops.plan) to the captured calls")
        ws = new_workspace(device, nbytes)
        _workspaces[key] = ws
    return ws


def _dev_status(device) -> torch.Tensor:
    st = _status.get(device)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=device)
        _status[device] = st
    return st


def check_device_status(device=None) -> None:
    """Synchronises and raises if any decode kernel on ``device`` reported an error."""
    for dev, st in _status.items():
        if device is None or dev == torch.device(device):
            word = int(st.item())
            if word:
                st.zero_()
                for (d, _), ws in _workspaces.items():   # a kernel that gave up may have left counters behind
                    if d == dev:
                        ws.zero_()
            _lib.check_dev_status(word, "decode")


def _take_workspace(workspace, device, nbytes: int) -> torch.Tensor:
    if workspace is None:
        return _workspace(device, nbytes)
    if (not workspace.is_cuda or workspace.dtype != torch.uint8 or workspace.numel() < nbytes
            or workspace.data_ptr() % 16 or not workspace.is_contiguous()):
        raise RuntimeError(f"workspace must be a contiguous CUDA uint8 tensor of at least {nbytes} bytes, 16-byte aligned")
    return workspace


def plan(n_kv_heads: int, n_tokens: int, window: int, group: int, nsplit: int = 0):
    ns, nbytes = C.c_int(0), C.c_size_t(0)
    _lib.check(_lib.lib().mfar_decode_plan(n_kv_heads, n_tokens, window, nsplit, C.byref(ns), C.byref(nbytes), group),
               "mfar_decode_plan")
    return ns.value, nbytes.value


def _check_op_inputs(bmp, NZ, idx, NZ_Offset, B):
    dev = B.device
    if any(t.device != dev for t in (bmp, NZ, idx, NZ_Offset)):
        raise RuntimeError("All input tensors must be on the same device.")
    if B.dtype != torch.float16:
        raise RuntimeError("Tensor B must be of type float16.")
    if NZ.dtype != torch.float16:
        raise RuntimeError("Tensor NZ must be of type float16.")
    if bmp.dtype != torch.int64:
        raise RuntimeError("Tensor bmp must be of type int64.")
    if idx.dtype != torch.int32:
        raise RuntimeError("Tensor idx must be of type int.")
    if NZ_Offset.dtype != torch.int32:
        raise RuntimeError("Tensor NZ_Offset must be of type int.")
    if not all(t.is_cuda for t in (bmp, NZ, idx, NZ_Offset, B)):
        raise RuntimeError("bmp, NZ, idx, B and NZ_Offset tensors must be on CUDA device.")
    if not all(t.is_contiguous() for t in (bmp, NZ, idx, NZ_Offset)):
        raise RuntimeError("bmp, NZ, idx and NZ_Offset tensors must be contiguous.")


def mustafar_key_formulation(bmp, NZ, idx, NZ_Offset, B, M_Global, K_Global, Batch_Size, num_key_value_groups):
    """S = K~ q.  B is the query padded to 8 rows [Batch_Size, 8, K_Global]; returns fp16
    [Batch_Size, 8, M_Global] whose row 0 is the result and rows 1..7 are zero (the
    reference multiplies its 7 zero rows; ``models/llama_mustafar_kernel.py:394-396``)."""
    _check_op_inputs(bmp, NZ, idx, NZ_Offset, B)
    if K_Global != D:
        raise RuntimeError("head_dim must be 128")
    if M_Global % 64 or Batch_Size % num_key_value_groups:
        raise RuntimeError("M_Global must be a multiple of 64 and Batch_Size a multiple of the group size")
    if not B.is_contiguous():
        raise RuntimeError("B must be contiguous.")
    n_kv = Batch_Size // num_key_value_groups
    tiles = M_Global * K_Global // 64
    out = torch.zeros((Batch_Size, 8, M_Global), dtype=torch.float16, device=B.device)
    st = _dev_status(B.device)
    rows = B.shape[1] if B.dim() == 3 else 1
    r = _lib.lib().mfar_key_scores_fp16(
        B.data_ptr(), rows * K_Global, n_kv, num_key_value_groups,
        bmp.data_ptr(), tiles, idx.data_ptr(), tiles + 1, NZ.data_ptr(), NZ_Offset.data_ptr(), 0, NZ.numel(),
        M_Global, out.data_ptr(), 8 * M_Global, 0, st.data_ptr(), _stream())
    _lib.check(r, "mfar_key_scores_fp16")
    if _debug_check():
        check_device_status(B.device)
    return out


def mustafar_value_formulation(bmp, NZ, idx, NZ_Offset, B, Reduction_Workspace, M_Global, K_Global, Batch_Size,
                               num_key_value_groups):
    """O = V~^T p.  B is the probabilities padded to 8 rows [Batch_Size, 8, K_Global = L];
    returns fp16 [Batch_Size, 8, M_Global = 128], row 0 real.  ``Reduction_Workspace`` is
    accepted for signature compatibility and not used (split partials live in an
    internal fp32 workspace)."""
    _check_op_inputs(bmp, NZ, idx, NZ_Offset, B)
    if M_Global != D:
        raise RuntimeError("head_dim must be 128")
    if K_Global % 64 or Batch_Size % num_key_value_groups:
        raise RuntimeError("K_Global must be a multiple of 64 and Batch_Size a multiple of the group size")
    Bc = B if B.is_contiguous() else B.contiguous()
    n_kv = Batch_Size // num_key_value_groups
    tiles = M_Global * K_Global // 64
    out = torch.zeros((Batch_Size, 8, M_Global), dtype=torch.float16, device=B.device)
    _, nbytes = plan(n_kv, K_Global, 0, num_key_value_groups)
    ws = _workspace(B.device, nbytes)
    st = _dev_status(B.device)
    rows = Bc.shape[1] if Bc.dim() == 3 else 1
    r = _lib.lib().mfar_value_output_fp16(
        Bc.data_ptr(), rows * K_Global, n_kv, num_key_value_groups,
        bmp.data_ptr(), tiles, idx.data_ptr(), tiles + 1, NZ.data_ptr(), NZ_Offset.data_ptr(), 0, NZ.numel(),
        K_Global, out.data_ptr(), 8 * M_Global, ws.data_ptr(), ws.numel(), 0, 0, st.data_ptr(), _stream())
    _lib.check(r, "mfar_value_output_fp16")
    if _debug_check():
        check_device_status(B.device)
    return out


def decode_attention(q: torch.Tensor, k_store: SparseStore, v_store: SparseStore,
                     k_window: torch.Tensor | None, v_window: torch.Tensor | None,
                     group: int, softmax_scale: float | None = None, out: torch.Tensor | None = None,
                     nsplit: int = 0, stage_halves: int | None = None,
                     window_len: torch.Tensor | None = None, n_tokens: torch.Tensor | None = None,
                     workspace: torch.Tensor | None = None) -> torch.Tensor:
    """Fused decode attention of one query token per q-head.

    q [n_kv_heads*group, 128] fp16; k_store / v_store hold the compressed tokens;
    k_window / v_window [n_kv_heads, W, 128] fp16 are the dense recent tokens (or None).
    ``window_len``: optional CUDA int32 tensor [1] with the number of valid window tokens (the window
    tensors then give the capacity); a captured launch can so be replayed while the window grows.
    ``n_tokens``: optional CUDA int32 tensor [1] with the number of compressed tokens to attend to (a multiple
    of 64, at most ``k_store.max_tokens``): the launch is then sized for the stores' capacity and keeps working
    while blocks are appended.  ``stage_halves`` must then cover every block still to come
    (``64 * kept + 896`` does unless tokens have more than three ties at the pruning threshold).
    ``workspace``: optional uint8 CUDA tensor from ``new_workspace`` (at least ``plan(...)`` bytes) owned by the caller;
    required for calls captured into a CUDA graph next to other decode users, or issued on several streams.
    One kernel launch.  Returns fp16 [n_kv_heads*group, 128].
    """
    n_kv = k_store.n_heads
    if q.dim() != 2 or q.shape != (n_kv * group, D) or q.dtype != torch.float16 or not q.is_cuda:
        raise RuntimeError("q must be CUDA float16 [n_kv_heads*group, 128]")
    if q.stride(1) != 1 or q.stride(0) % 2 or q.data_ptr() % 4:
        q = q.contiguous()
    L = k_store.tokens
    if v_store.tokens != L or v_store.n_heads != n_kv:
        raise RuntimeError("K and V stores disagree")
    W = 0
    kw = vw = None
    wh = wt = 0
    if k_window is not None and k_window.shape[1] > 0:
        if k_window.shape != v_window.shape or k_window.shape[0] != n_kv or k_window.shape[2] != D:
            raise RuntimeError("window tensors must be [n_kv_heads, W, 128]")
        if k_window.stride() != v_window.stride() or k_window.stride(2) != 1:
            k_window, v_window = k_window.contiguous(), v_window.contiguous()
        W, kw, vw = k_window.shape[1], k_window.data_ptr(), v_window.data_ptr()
        wh, wt = k_window.stride(0), k_window.stride(1)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty((n_kv * group, D), dtype=torch.float16, device=q.device)
    if stage_halves is None and n_tokens is None:
        stage_halves = max(k_store.stage_hint(), v_store.stage_hint()) if L else 8
    wl = None if window_len is None else window_len.data_ptr()
    st = _dev_status(q.device)
    if n_tokens is not None:
        if not n_tokens.is_cuda or n_tokens.dtype != torch.int32 or n_tokens.numel() != 1:
            raise RuntimeError("n_tokens must be a CUDA int32 tensor with one element")
        if stage_halves is None:
            raise RuntimeError("n_tokens on the device needs an explicit stage_halves bound")
        Lmax = min(k_store.max_tokens, v_store.max_tokens)
        _, nbytes = plan(n_kv, Lmax, W, group, nsplit)
        ws = _take_workspace(workspace, q.device, nbytes)
        r = _lib.lib().mfar_decode_attention_fp16_dyn(
            q.data_ptr(), q.stride(0), n_kv, group,
            k_store.bitmaps.data_ptr(), k_store.tiles_cap, k_store.accum.data_ptr(), k_store.tiles_cap + 1,
            k_store.nz.data_ptr(), None, k_store.nz_capacity, k_store.nz.numel(),
            v_store.bitmaps.data_ptr(), v_store.tiles_cap, v_store.accum.data_ptr(), v_store.tiles_cap + 1,
            v_store.nz.data_ptr(), None, v_store.nz_capacity, v_store.nz.numel(),
            Lmax, n_tokens.data_ptr(), kw, vw, wh, wt, W, wl, float(softmax_scale), out.data_ptr(), out.stride(0),
            ws.data_ptr(), ws.numel(), nsplit, stage_halves, st.data_ptr(), _stream())
        _lib.check(r, "mfar_decode_attention_fp16_dyn")
        if _debug_check():
            check_device_status(q.device)
        return out
    _, nbytes = plan(n_kv, L, W, group, nsplit)
    ws = _take_workspace(workspace, q.device, nbytes)
    r = _lib.lib().mfar_decode_attention_fp16(
        q.data_ptr(), q.stride(0), n_kv, group,
        k_store.bitmaps.data_ptr(), k_store.tiles_cap, k_store.accum.data_ptr(), k_store.tiles_cap + 1,
        k_store.nz.data_ptr(), None, k_store.nz_capacity, k_store.nz.numel(),
        v_store.bitmaps.data_ptr(), v_store.tiles_cap, v_store.accum.data_ptr(), v_store.tiles_cap + 1,
        v_store.nz.data_ptr(), None, v_store.nz_capacity, v_store.nz.numel(),
        L, kw, vw, wh, wt, W, wl, float(softmax_scale), out.data_ptr(), out.stride(0), ws.data_ptr(), ws.numel(),
        nsplit, stage_halves, st.data_ptr(), _stream())
    _lib.check(r, "mfar_decode_attention_fp16")
    if _debug_check():
        check_device_status(q.device)
    return out
