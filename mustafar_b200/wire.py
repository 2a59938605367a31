"""Flat wire / disk format of a compressed K or V cache: one byte blob per ``SparseStore`` that another
process (or a later run) can map back into an arena, for cache offload and prefix reuse.  The reference
keeps its compressed cache only as live Python lists of tensors (``models/llama_mustafar_kernel.py:546-560``)
and has no such format; the sections below are its own arrays, unchanged, laid end to end.

    offset 0    header, 64 bytes, little endian:
                  0  8 bytes  magic b"MFARKV01"
                  8  u32      kind (0 = K tiles: channel x 64 tokens, 1 = V tiles: token x 64 channels)
                 12  u32      n_heads (batch * kv heads)
                 16  u32      tokens (multiple of 64)
                 20  u32      head_dim (128)
                 24  u64      tiles per head (= 2 * tokens)
                 32  u64      total packed halves over all heads
                 40  u32      largest packed size of a 64-token block, halves (staging hint of the decode kernel)
                 44  20 bytes zero
    then, each section starting on a 16-byte boundary:
      bitmaps   int64 [n_heads, tiles]        bit 63 - i <-> element i of the tile
      accum     int32 [n_heads, tiles + 1]    the reference's accum_counts (uint32 units inside the head)
      starts    int64 [n_heads + 1]           first packed half of every head inside `packed`
      packed    fp16  [total]                 heads back to back, each 2 * accum[h, tiles] halves

``pack_store`` copies device -> host once per section; ``unpack_store`` validates every field it relies on
before it allocates (a blob is untrusted input) and rebuilds a ``SparseStore`` on the given device."""
from __future__ import annotations

import struct

import numpy as np
import torch

from .compression import D, KEY, VALUE, SparseStore

MAGIC = b"MFARKV01"
HEADER_BYTES = 64


def _pad16(n: int) -> int:
    return (n + 15) // 16 * 16


def pack_store(st: SparseStore) -> torch.Tensor:
    """-> uint8 CPU tensor holding the store's first ``st.tokens`` tokens."""
    T = st.tiles
    accum = st.accum[:, :T + 1].cpu()
    lengths = (2 * accum[:, T].to(torch.int64)).tolist() if st.n_heads else []
    starts = np.zeros(st.n_heads + 1, dtype=np.int64)
    if st.n_heads:
        starts[1:] = np.cumsum(lengths)
    total = int(starts[-1])
    hint = 0
    if st.tokens and st.bitmaps.is_cuda:
        hint = st.stage_hint()
    elif st.tokens:
        per_block = accum[:, 128::128] - accum[:, :-1:128][:, :accum[:, 128::128].shape[1]]
        hint = int(2 * per_block.max().item()) if per_block.numel() else 0
    sizes = [8 * st.n_heads * T, 4 * st.n_heads * (T + 1), 8 * (st.n_heads + 1), 2 * total]
    offs, o = [], HEADER_BYTES
    for s in sizes:
        offs.append(o)
        o = _pad16(o + s)
    blob = np.zeros(o, dtype=np.uint8)
    blob[:HEADER_BYTES] = np.frombuffer(
        struct.pack("<8sIIIIQQI20x", MAGIC, st.kind, st.n_heads, st.tokens, D, T, total, hint), dtype=np.uint8)
    blob[offs[0]:offs[0] + sizes[0]] = st.bitmaps[:, :T].cpu().contiguous().numpy().view(np.uint8).reshape(-1)
    blob[offs[1]:offs[1] + sizes[1]] = accum.contiguous().numpy().view(np.uint8).reshape(-1)
    blob[offs[2]:offs[2] + sizes[2]] = starts.view(np.uint8)
    if total:
        flat = torch.cat([st.nz[h, :lengths[h]] for h in range(st.n_heads)]).cpu()
        blob[offs[3]:offs[3] + sizes[3]] = flat.numpy().view(np.uint8)
    return torch.from_numpy(blob)


def unpack_store(blob: torch.Tensor, device, max_tokens: int | None = None, nz_capacity: int | None = None) -> SparseStore:
    """Rebuilds a store from ``pack_store``'s blob.  ``max_tokens`` / ``nz_capacity`` size the arena for later
    appends (defaults: exactly what the blob holds, rounded up to the format's granules)."""
    raw = blob.detach().cpu().contiguous().view(torch.uint8).numpy()
    if raw.size < HEADER_BYTES:
        raise ValueError("blob shorter than its header")
    magic, kind, n_heads, tokens, head_dim, tiles, total, hint = struct.unpack("<8sIIIIQQI20x", raw[:HEADER_BYTES].tobytes())
    if magic != MAGIC:
        raise ValueError("not a compressed-cache blob (bad magic)")
    if kind not in (KEY, VALUE) or head_dim != D or tokens % 64 or tiles != 2 * tokens:
        raise ValueError("inconsistent header")
    sizes = [8 * n_heads * tiles, 4 * n_heads * (tiles + 1), 8 * (n_heads + 1), 2 * total]
    offs, o = [], HEADER_BYTES
    for s in sizes:
        offs.append(o)
        o = _pad16(o + s)
    if raw.size < o:
        raise ValueError("blob shorter than its sections")
    bitmaps = raw[offs[0]:offs[0] + sizes[0]].view(np.int64).reshape(n_heads, tiles)
    accum = raw[offs[1]:offs[1] + sizes[1]].view(np.int32).reshape(n_heads, tiles + 1)
    starts = raw[offs[2]:offs[2] + sizes[2]].view(np.int64)
    packed = raw[offs[3]:offs[3] + sizes[3]].view(np.float16)
    # everything the kernels will trust: offsets start at 0, never decrease, step in units of 8 halves
    # that hold the tile's popcount, and the per-head extents tile `packed` exactly
    if n_heads:
        steps = np.diff(accum.astype(np.int64), axis=1)
        if (accum[:, 0] != 0).any() or (steps < 0).any() or (steps % 4).any():
            raise ValueError("corrupt accum section")
        pop = np.unpackbits(bitmaps.view(np.uint8), axis=None).reshape(n_heads, tiles, 64).sum(-1) if tiles else steps
        if tiles and (steps != ((pop + 7) // 8) * 4).any():
            raise ValueError("bitmaps and accum disagree")
        lengths = 2 * accum[:, tiles].astype(np.int64)
        if starts[0] != 0 or (np.diff(starts) != lengths).any() or starts[-1] != total:
            raise ValueError("corrupt starts section")
    else:
        lengths = np.zeros(0, dtype=np.int64)
    cap_tokens = max(64, tokens if max_tokens is None else max_tokens)
    if cap_tokens % 64 or cap_tokens < tokens:
        raise ValueError("max_tokens must be a multiple of 64 and hold the blob's tokens")
    need = int(lengths.max()) if n_heads else 0
    cap = max(8, need if nz_capacity is None else nz_capacity)
    if cap < need:
        raise ValueError("nz_capacity smaller than the largest head in the blob")
    st = SparseStore(n_heads, cap_tokens, kind, device, nz_capacity=cap)
    if n_heads and tokens:
        st.bitmaps[:, :tiles] = torch.from_numpy(bitmaps.copy()).to(device)
        st.accum[:, :tiles + 1] = torch.from_numpy(accum.copy()).to(device)
        flat = torch.from_numpy(packed.copy()).to(device)
        for h in range(n_heads):
            st.nz[h, :lengths[h]] = flat[starts[h]:starts[h + 1]]
    st.tokens = tokens
    st._stage_hint = max(8, (int(hint) + 7) // 8 * 8)
    st.stats[1] = int(hint)
    return st
