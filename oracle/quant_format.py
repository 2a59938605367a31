"""Bitmap + per-tile asymmetric low-bit quantised format, CPU restatement (test infrastructure).

Follows ``kernel_quant/compression_quant.py``:

* bitmap and tile order as the fp16 format (``:23-32`` key, ``:288-303`` value);
* ``counts`` = raw nonzeros per tile, no padding (``:34-35``);
* per tile, over its nonzeros: ``scale = (max - min) / (2**bits - 1)`` (1 when
  that is 0 or the tile is empty), ``zero = floor(-min / scale + 0.5)``
  (``:40-57``); both are *stored* fp16 (``:181-182``);
* codes ``clamp(floor(v / scale_fp16 + 0.5) + zero_fp16, 0, 2**bits - 1)`` with
  fp32 arithmetic on the stored fp16 parameters (``:134-145``);
* ``capacity = 32 // bits`` codes per uint32, LSB first (``:148-152``);
  ``units = ceil(counts / capacity)`` (``:221``); ``tile_offsets`` = global
  uint32 offset of each tile in ONE flat buffer shared by all heads (``:223-238``).

The arithmetic dtype of ``scale`` / ``zero`` before they are stored was fixed by
running the reference's Triton kernels under the interpreter (see
``tests/golden/make_golden.py``): see ``_scale_zero`` below, which reproduces
the interpreter bit for bit.

The reference hard-codes ``bits = 2`` (``:209-210``).  ``bits = 4`` and
``group = 32`` (a fresh scale/zero every 32 nonzeros of a tile, i.e. up to two
groups per tile) are extensions of this build: **parity unpinned**.
"""
from __future__ import annotations

import numpy as np

from .fp16_format import _WEIGHTS, key_tiles, value_tiles


def _scale_zero(xmin: np.ndarray, xmax: np.ndarray, has: np.ndarray, bits: int):
    """xmin/xmax per group -> (scale fp16, zero fp16) exactly as the Triton kernel
    ``calculate_bitmap_and_scale_*`` stores them: ``tl.min`` / ``tl.max`` promote
    fp16 to fp32, so the subtraction, the division by ``2**bits - 1``, the
    ``== 0`` test and ``floor(-min / scale + 0.5)`` all run in fp32 on the
    UNROUNDED scale; only the two stores round to fp16."""
    maxq = np.float32((1 << bits) - 1)
    lo = xmin.astype(np.float32)
    hi = xmax.astype(np.float32)
    with np.errstate(all="ignore"):
        scale = (hi - lo) / maxq
        scale = np.where(scale == 0, np.float32(1.0), scale).astype(np.float32)
        zero = np.floor((-lo) / scale + np.float32(0.5)).astype(np.float32)
    scale = np.where(has, scale, np.float32(1.0)).astype(np.float16)
    zero = np.where(has, zero, np.float32(0.0)).astype(np.float16)
    return scale, zero


def quant_pack_tiles(tiles: np.ndarray, bits: int = 2, group: int = 64):
    """tiles [Bh,T,64] fp16 -> dict of the seven arrays of the quantised format."""
    assert bits in (2, 4) and group in (32, 64)
    Bh, T, _ = tiles.shape
    cap = 32 // bits
    ngrp = 64 // group
    maxq = (1 << bits) - 1
    nz = tiles != 0
    bitmaps = (nz.astype(np.uint64) * _WEIGHTS).sum(axis=-1, dtype=np.uint64).view(np.int64)
    counts = nz.sum(axis=-1).astype(np.int32)
    rank = np.cumsum(nz, axis=-1) - 1                       # index among the tile's nonzeros
    grp = np.where(nz, rank // group, 0)                    # group of each nonzero

    scales = np.ones((Bh, T, ngrp), dtype=np.float16)
    zeros = np.zeros((Bh, T, ngrp), dtype=np.float16)
    for g in range(ngrp):
        sel = nz & (grp == g)
        has = sel.any(axis=-1)
        xmin = np.where(sel, tiles, np.float16(np.inf)).min(axis=-1)
        xmax = np.where(sel, tiles, np.float16(-np.inf)).max(axis=-1)
        scales[..., g], zeros[..., g] = _scale_zero(xmin, xmax, has, bits)

    s32 = np.take_along_axis(scales, grp, axis=-1).astype(np.float32)
    s32 = np.where(s32 == 0, np.float32(1.0), s32)          # ``if scale == 0.0: scale = 1.0`` (``:136-137``)
    z32 = np.take_along_axis(zeros, grp, axis=-1).astype(np.float32)
    with np.errstate(all="ignore"):
        q = np.floor(tiles.astype(np.float32) / s32 + np.float32(0.5)) + z32
    q = np.clip(q, 0.0, float(maxq))
    q = np.where(nz, q, 0.0).astype(np.uint32)

    units = (counts + cap - 1) // cap
    flat_units = units.reshape(-1).astype(np.int64)
    offs = np.zeros(Bh * T, dtype=np.int64)
    np.cumsum(flat_units[:-1], out=offs[1:])
    tile_offsets = offs.reshape(Bh, T).astype(np.int32)
    total = int(flat_units.sum())
    packed = np.zeros(total, dtype=np.uint32)
    word = tile_offsets[..., None].astype(np.int64) + rank // cap
    shift = ((rank % cap) * bits).astype(np.uint32)
    np.bitwise_or.at(packed, word[nz], q[nz] << shift[nz])

    if ngrp == 1:
        scales, zeros = scales[..., 0], zeros[..., 0]
    return dict(bitmaps=bitmaps, tile_offsets=tile_offsets, packed=packed.view(np.int32),
                counts=counts, units=units.astype(np.int32), scales=scales, zeros=zeros)


def quant_compress_key_ref(x, bits: int = 2, group: int = 64):
    """``convert_key_batched_quant`` (``kernel_quant/compression_quant.py:159-264``)."""
    return quant_pack_tiles(key_tiles(x), bits, group)


def quant_compress_value_ref(x, bits: int = 2, group: int = 64):
    """``convert_value_batched_quant`` (``kernel_quant/compression_quant.py:425-529``)."""
    return quant_pack_tiles(value_tiles(x), bits, group)


def _dequant_tiles(fmt: dict, bits: int, group: int, mode: int = 0) -> np.ndarray:
    """Per-element ``(q - zero) * scale`` rounded to fp16, as the reference kernels
    place it in shared memory (``kernel_quant/csrc/SpMM_Kernel_Quant.cuh:235-240``
    for mode 0 = fp32 math; ``:190-193`` for mode 1 = fp16 math)."""
    bitmaps = fmt["bitmaps"].view(np.uint64)
    Bh, T = bitmaps.shape
    cap = 32 // bits
    mask = np.uint32((1 << bits) - 1)
    bit = ((bitmaps[..., None] >> np.arange(63, -1, -1, dtype=np.uint64)) & np.uint64(1)).astype(bool)
    rank = np.cumsum(bit, axis=-1) - 1
    word = fmt["tile_offsets"][..., None].astype(np.int64) + np.where(bit, rank // cap, 0)
    packed = fmt["packed"].view(np.uint32)
    if packed.size == 0:
        return np.zeros((Bh, T, 64), dtype=np.float16)
    word = np.minimum(word, packed.size - 1)
    q = (packed[word] >> ((np.where(bit, rank, 0) % cap) * bits).astype(np.uint32)) & mask
    scales = fmt["scales"].reshape(Bh, T, -1)
    zeros = fmt["zeros"].reshape(Bh, T, -1)
    grp = np.where(bit, rank // group, 0)
    s = np.take_along_axis(scales, grp, axis=-1)
    z = np.take_along_axis(zeros, grp, axis=-1)
    if mode == 0:
        v = ((q.astype(np.float32) - z.astype(np.float32)) * s.astype(np.float32)).astype(np.float16)
    else:
        v = ((q.astype(np.float16) - z).astype(np.float16) * s).astype(np.float16)
    return np.where(bit, v, np.float16(0))


def dequant_key_ref(fmt: dict, L: int, D: int = 128, bits: int = 2, group: int = 64, mode: int = 0):
    tiles = _dequant_tiles(fmt, bits, group, mode)
    Bh = tiles.shape[0]
    return np.ascontiguousarray(tiles.reshape(Bh, L // 64, D, 64).transpose(0, 1, 3, 2)).reshape(Bh, L, D)


def dequant_value_ref(fmt: dict, L: int, D: int = 128, bits: int = 2, group: int = 64, mode: int = 0):
    tiles = _dequant_tiles(fmt, bits, group, mode)
    Bh = tiles.shape[0]
    return np.ascontiguousarray(
        tiles.reshape(Bh, L // 64, D // 64, 64, 64).transpose(0, 1, 3, 2, 4)).reshape(Bh, L, D)
