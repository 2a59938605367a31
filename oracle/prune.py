"""Per-token magnitude pruning, CPU restatement (test infrastructure).

Follows ``models/llama_mustafar_kernel.py:194-232`` (``dh_prune_key``; the
value variant at ``:236-274`` is identical):

    num_to_keep = max(1, int(target_sparsity * D))          # despite the name: a RANK
    thr  = kthvalue(|x|, num_to_keep)  along D               # k-th SMALLEST magnitude
    out  = x * (|x| >= thr)                                  # ties at thr are all kept

so a row keeps ``D - k + 1`` elements plus any further ties at the threshold,
and pruned negatives become ``-0.0`` (fp16 multiply by 0).
"""
from __future__ import annotations

import numpy as np
import torch


def keep_count(sparsity: float, D: int = 128) -> int:
    """Rank ``k`` handed to kthvalue (``models/llama_mustafar_kernel.py:215``)."""
    return max(1, int(sparsity * D))


def prune_ref(x: torch.Tensor, sparsity: float) -> torch.Tensor:
    """x: [..., D] fp16 (CPU).  Returns the pruned fp16 tensor, same shape."""
    assert x.dtype == torch.float16
    D = x.shape[-1]
    k = keep_count(sparsity, D)
    flat = x.reshape(-1, D)
    mag = flat.abs().float()  # fp16 -> fp32 is exact and order preserving
    thr, _ = torch.kthvalue(mag, k, dim=-1, keepdim=True)
    mask = mag >= thr
    out = flat * mask.to(flat.dtype)
    return out.view(x.shape)


def prune_np(x: np.ndarray, sparsity: float) -> np.ndarray:
    """Independent numpy restatement (sort based) used to cross-check prune_ref."""
    assert x.dtype == np.float16
    D = x.shape[-1]
    k = keep_count(sparsity, D)
    flat = x.reshape(-1, D)
    mag = np.abs(flat).astype(np.float32)
    thr = np.sort(mag, axis=-1)[:, k - 1:k]
    mask = mag >= thr
    return (flat * mask.astype(np.float16)).reshape(x.shape)
