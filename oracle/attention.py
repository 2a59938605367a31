"""Decode attention over the pruned cache, CPU restatement (test infrastructure).

* ``key_formulation_ref`` / ``value_formulation_ref`` give what the two reference
  ops return in row 0 of their 8-row outputs: fp16 operands, fp32 accumulation,
  one fp16 rounding (``kernel/csrc/SpMM_Kernel.cuh:258-265`` GQA addressing
  ``kv_head = q_head // G``; ``:491-519`` the store).
* ``decode_attention_model_order_ref`` repeats the model's decode step with its
  fp16 roundings in the same places (``models/llama_mustafar_kernel.py:394-438``).
* ``decode_attention_ref`` is the same attention in fp32 end to end: dense
  ``softmax(q.K^T / sqrt(D)).V`` on the pruned tensors, which is what the torch
  accuracy path computes (``models/llama_mustafar_Kt_Mag_Vt_Mag.py:873-874,963,974``).
"""
from __future__ import annotations

import math

import numpy as np
import torch


def _t(x, dtype=None):
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(np.ascontiguousarray(x))
    return x if dtype is None else x.to(dtype)


def rel_l2(a, b) -> float:
    a = _t(a, torch.float64).reshape(-1)
    b = _t(b, torch.float64).reshape(-1)
    den = float(torch.linalg.norm(b))
    return float(torch.linalg.norm(a - b)) / (den if den > 0 else 1.0)


def key_formulation_ref(k_dense, q, G: int) -> torch.Tensor:
    """k_dense [Bh,L,D] fp16 (pruned / dequantised), q [Bq,D] fp16 -> S [Bq,L] fp16."""
    k = _t(k_dense).float()
    qf = _t(q).float()
    Bq = qf.shape[0]
    kk = k.repeat_interleave(G, dim=0) if G > 1 else k
    assert kk.shape[0] == Bq
    return torch.bmm(kk, qf.unsqueeze(-1)).squeeze(-1).half()


def value_formulation_ref(v_dense, p, G: int) -> torch.Tensor:
    """v_dense [Bh,L,D] fp16, p [Bq,L] fp16 -> O [Bq,D] fp16."""
    v = _t(v_dense).float()
    pf = _t(p).float()
    vv = v.repeat_interleave(G, dim=0) if G > 1 else v
    return torch.bmm(pf.unsqueeze(1), vv).squeeze(1).half()


def decode_attention_ref(q, k_comp, v_comp, k_win, v_win, G: int) -> torch.Tensor:
    """fp32 attention of one query token per q-head over [compressed ; window].

    q [Bq,D] fp16; k_comp/v_comp [Bh,L,D] fp16 pruned (L may be 0);
    k_win/v_win [Bh,W,D] fp16 dense (W may be 0).  Returns [Bq,D] fp32.
    """
    qf = _t(q).float()
    D = qf.shape[-1]
    ks = [_t(x).float() for x in (k_comp, k_win) if x is not None and x.shape[1] > 0]
    vs = [_t(x).float() for x in (v_comp, v_win) if x is not None and x.shape[1] > 0]
    k = torch.cat(ks, dim=1)
    v = torch.cat(vs, dim=1)
    if G > 1:
        k = k.repeat_interleave(G, dim=0)
        v = v.repeat_interleave(G, dim=0)
    s = torch.bmm(k, qf.unsqueeze(-1)).squeeze(-1) / math.sqrt(D)
    p = torch.softmax(s, dim=-1)
    return torch.bmm(p.unsqueeze(1), v).squeeze(1)


def decode_attention_model_order_ref(q, k_comp, v_comp, k_win, v_win, G: int) -> torch.Tensor:
    """The model's own sequence of fp16 roundings; returns [Bq,D] fp16."""
    qh = _t(q)
    D = qh.shape[-1]
    L = k_comp.shape[1]
    s_c = key_formulation_ref(k_comp, qh, G)                                  # fp16 [Bq,L]
    kw = _t(k_win).float().repeat_interleave(G, dim=0)
    vw = _t(v_win).float().repeat_interleave(G, dim=0)
    s_w = torch.bmm(kw, qh.float().unsqueeze(-1)).squeeze(-1).half()          # fp16 matmul
    s = (torch.cat([s_c, s_w], dim=-1).float() / math.sqrt(D)).half()         # fp16 divide
    p = torch.softmax(s.float(), dim=-1).half()                               # fp32 softmax -> fp16
    o_c = value_formulation_ref(v_comp, p[:, :L].contiguous(), G)             # fp16
    o_w = torch.bmm(p[:, L:].float().unsqueeze(1), vw).squeeze(1).half()      # fp16 matmul
    return (o_c.float() + o_w.float()).half()                                 # fp16 add
