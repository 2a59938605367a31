"""Seeded synthetic K / V / q generators (test + benchmark infrastructure).

Stand-ins for real model activations: ``K, V ~ N(0,1)`` with four fixed outlier
channels per head scaled x10 in K, ``q ~ N(0,1)``; generated with a CPU
``torch.Generator`` so the CPU oracle and the GPU kernels see identical bits.
The seed scheme (base + 9973 * index) mirrors
``kernel_quant/kernel_bench/benchmark_spmv_detailed.py:77-78,170-171``.
"""
from __future__ import annotations

import torch

BASE_SEED = 20260302
SEED_STRIDE = 9973


def make_kv(Bh: int, L: int, D: int = 128, seed: int = BASE_SEED, outliers: bool = True):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(Bh, L, D, generator=g, dtype=torch.float32)
    v = torch.randn(Bh, L, D, generator=g, dtype=torch.float32)
    if outliers:
        for h in range(Bh):
            ch = torch.randperm(D, generator=g)[:4]
            k[h, :, ch] *= 10.0
    return k.half(), v.half()


def make_query(Bq: int, D: int = 128, seed: int = BASE_SEED + 1):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(Bq, D, generator=g, dtype=torch.float32).half()
