"""Host side of the quantised bitmap format.

``convert_key_batched_quant`` / ``convert_value_batched_quant`` keep the signatures and
return tuples of the reference's ``kernel_quant/compression_quant.py:159-264`` and
``:425-529`` (2-bit, one scale / zero-point per 64-element tile).  ``bits=4`` and
``group=32`` are extensions without a reference counterpart.
"""
from __future__ import annotations

import torch

from . import _lib
from .compression import D, KEY, VALUE, _check_input, _stream


def compress_quant(x: torch.Tensor, kind: int, prune_rank: int = 0, bits: int = 2, group: int = 64):
    """Returns dict(bitmaps, tile_offsets, packed, counts, units, scales, zeros) in the reference's
    compact layout (one flat int32 code buffer shared by all heads)."""
    x = _check_input(x)
    Bh, L, _ = x.shape
    T = 2 * L
    ngrp = 64 // group
    dev = x.device
    bitmaps = torch.empty((Bh, T), dtype=torch.int64, device=dev)
    tile_offsets = torch.empty((Bh, T), dtype=torch.int32, device=dev)
    counts = torch.empty((Bh, T), dtype=torch.int32, device=dev)
    units = torch.empty((Bh, T), dtype=torch.int32, device=dev)
    shape = (Bh, T) if ngrp == 1 else (Bh, T, ngrp)
    scales = torch.empty(shape, dtype=torch.float16, device=dev)
    zeros = torch.empty(shape, dtype=torch.float16, device=dev)
    worst = Bh * T * (64 * bits // 32)
    packed = torch.empty(max(worst, 1), dtype=torch.int32, device=dev)
    info = torch.zeros(Bh + 1, dtype=torch.int32, device=dev)      # per-head end offsets, then dev_status
    if L:
        need = _lib.lib().mfar_compress_scratch_bytes(Bh, L)
        scratch = torch.empty(need, dtype=torch.uint8, device=dev)
        st = _lib.lib().mfar_compress_quant(
            x.data_ptr(), x.stride(0), x.stride(1), Bh, L, kind, prune_rank, bits, group,
            bitmaps.data_ptr(), T, tile_offsets.data_ptr(), counts.data_ptr(), units.data_ptr(),
            scales.data_ptr(), zeros.data_ptr(), T, 0, packed.data_ptr(), 0, worst, info.data_ptr(),
            scratch.data_ptr(), need, info.data_ptr() + 4 * Bh, _stream())
        _lib.check(st, "mfar_compress_quant")
    host = info.tolist()                                            # the one host sync
    _lib.check_dev_status(host[Bh], "mfar_compress_quant")
    total = host[Bh - 1] if (Bh and L) else 0
    return dict(bitmaps=bitmaps, tile_offsets=tile_offsets, packed=packed[:total].clone(), counts=counts,
                units=units, scales=scales, zeros=zeros)


def convert_key_batched_quant(inputs: torch.Tensor, return_metadata: bool = False):
    """Drop-in for ``kernel_quant/compression_quant.py:159-264``: inputs [B*Hkv, L, 128] (already
    pruned) -> (bitmaps, tile_offsets, packed, scales, zeros), with counts and units inserted
    after ``packed`` when ``return_metadata``."""
    r = compress_quant(inputs, KEY)
    if return_metadata:
        return r["bitmaps"], r["tile_offsets"], r["packed"], r["counts"], r["units"], r["scales"], r["zeros"]
    return r["bitmaps"], r["tile_offsets"], r["packed"], r["scales"], r["zeros"]


def convert_value_batched_quant(inputs: torch.Tensor):
    """Drop-in for ``kernel_quant/compression_quant.py:425-529`` (always returns the 7-tuple)."""
    r = compress_quant(inputs, VALUE)
    return r["bitmaps"], r["tile_offsets"], r["packed"], r["counts"], r["units"], r["scales"], r["zeros"]
