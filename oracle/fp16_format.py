"""Bitmap + packed-nonzero fp16 format, CPU restatement (test infrastructure).

Follows ``kernel/compression.py``:

* a *tile* is 64 logical elements described by one 64-bit bitmap; bit ``63-i``
  is element ``i`` (``:42-44``, ``:164-165``: ``bitmap >> (63 - offsets)``);
* K tiles run along tokens for a fixed channel of the transposed ``[Bh, D, L]``
  copy: ``tile_id = (t // 64) * D + c`` (``:32-36``, ``:258``);
* V tiles run along channels for a fixed token, ordered
  ``[token_block][col_half][token_in_block]`` (``:87-97``);
* ``counts = ((nnz + 7) & ~7) >> 1`` -- nonzeros padded to 8 halves, expressed
  in uint32 units (``:48``); ``accum_counts = [0, cumsum(counts)]`` per head,
  int32, ``T + 1`` entries (``:297-301``);
* packed values of a head: tile ``i`` starts at half ``2 * accum[i]``, holds its
  nonzeros in element order, padding halves are 0 (``:171-174``, ``:312``).
"""
from __future__ import annotations

import numpy as np
import torch

_WEIGHTS = (np.uint64(1) << np.arange(63, -1, -1, dtype=np.uint64))


def _np16(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        assert x.dtype == torch.float16
        return x.detach().cpu().contiguous().numpy()
    assert x.dtype == np.float16
    return np.ascontiguousarray(x)


def key_tiles(x) -> np.ndarray:
    """[Bh, L, D] -> [Bh, T, 64] tiles in K order (``kernel/compression.py:32-36``)."""
    x = _np16(x)
    Bh, L, D = x.shape
    assert L % 64 == 0
    return np.ascontiguousarray(
        x.reshape(Bh, L // 64, 64, D).transpose(0, 1, 3, 2)).reshape(Bh, L * D // 64, 64)


def value_tiles(x) -> np.ndarray:
    """[Bh, L, D] -> [Bh, T, 64] tiles in V order (``kernel/compression.py:87-97``)."""
    x = _np16(x)
    Bh, L, D = x.shape
    assert L % 64 == 0 and D % 64 == 0
    return np.ascontiguousarray(
        x.reshape(Bh, L // 64, 64, D // 64, 64).transpose(0, 1, 3, 2, 4)).reshape(Bh, L * D // 64, 64)


def pack_tiles(tiles: np.ndarray):
    """tiles [Bh, T, 64] fp16 -> (bitmaps int64 [Bh,T], accum int32 [Bh,T+1], list of fp16 1-D)."""
    Bh, T, _ = tiles.shape
    nz = tiles != 0  # -0.0 compares equal to 0 and is dropped; NaN is kept (``:39``)
    bitmaps = (nz.astype(np.uint64) * _WEIGHTS).sum(axis=-1, dtype=np.uint64).view(np.int64)
    nnz = nz.sum(axis=-1).astype(np.int32)
    counts = ((nnz + 7) & ~7) >> 1
    accum = np.zeros((Bh, T + 1), dtype=np.int32)
    np.cumsum(counts, axis=1, out=accum[:, 1:])
    rank = np.cumsum(nz, axis=-1) - 1
    packed = []
    for b in range(Bh):
        buf = np.zeros(2 * int(accum[b, -1]), dtype=np.float16)
        dest = 2 * accum[b, :-1, None].astype(np.int64) + rank[b]
        buf[dest[nz[b]]] = tiles[b][nz[b]]
        packed.append(buf)
    return bitmaps, accum, packed


def compress_key_ref(x):
    """``convert_key_batched`` (``kernel/compression.py:249-342``) on the CPU."""
    return pack_tiles(key_tiles(x))


def compress_value_ref(x):
    """``convert_value_batched`` (``kernel/compression.py:344-435``) on the CPU."""
    return pack_tiles(value_tiles(x))


def nz_offsets_ref(accum: np.ndarray) -> np.ndarray:
    """Per-head start of the packed values in uint4 units once the per-head
    buffers are concatenated (``models/llama_mustafar_kernel.py:546-548``)."""
    tails = accum[:, -1].astype(np.int64) // 4
    out = np.zeros(accum.shape[0], dtype=np.int32)
    out[1:] = np.cumsum(tails)[:-1]
    return out


def _unpack_tiles(bitmaps: np.ndarray, accum: np.ndarray, packed) -> np.ndarray:
    Bh, T = bitmaps.shape
    bits = ((bitmaps.view(np.uint64)[..., None] >> np.arange(63, -1, -1, dtype=np.uint64)) & np.uint64(1)).astype(bool)
    rank = np.cumsum(bits, axis=-1) - 1
    tiles = np.zeros((Bh, T, 64), dtype=np.float16)
    for b in range(Bh):
        src = 2 * accum[b, :-1, None].astype(np.int64) + rank[b]
        tiles[b][bits[b]] = np.asarray(packed[b])[src[bits[b]]]
    return tiles


def decompress_key_ref(bitmaps, accum, packed, L: int, D: int = 128) -> np.ndarray:
    tiles = _unpack_tiles(np.asarray(bitmaps), np.asarray(accum), packed)
    Bh = tiles.shape[0]
    return np.ascontiguousarray(tiles.reshape(Bh, L // 64, D, 64).transpose(0, 1, 3, 2)).reshape(Bh, L, D)


def decompress_value_ref(bitmaps, accum, packed, L: int, D: int = 128) -> np.ndarray:
    tiles = _unpack_tiles(np.asarray(bitmaps), np.asarray(accum), packed)
    Bh = tiles.shape[0]
    return np.ascontiguousarray(
        tiles.reshape(Bh, L // 64, D // 64, 64, 64).transpose(0, 1, 3, 2, 4)).reshape(Bh, L, D)
