"""Host side of the quantised bitmap format.

``convert_key_batched_quant`` / ``convert_value_batched_quant`` keep the signatures and
return tuples of the reference's ``kernel_quant/compression_quant.py:159-264`` and
``:425-529`` (2-bit, one scale / zero-point per 64-element tile).  ``bits=4`` and
``group=32`` are extensions without a reference counterpart.
"""
from __future__ import annotations

import torch

from . import _lib
from .compression import D, KEY, VALUE, _check_input, _source_args, _stream


def compress_quant(x: torch.Tensor, kind: int, prune_rank: int = 0, bits: int = 2, group: int = 64):
    """Returns dict(bitmaps, tile_offsets, packed, counts, units, scales, zeros) in the reference's
    compact layout (one flat int32 code buffer shared by all heads)."""
    x = _check_input(x)
    if x.dim() != 3:
        raise RuntimeError("compress_quant expects [heads, tokens, 128]")
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
            x.data_ptr(), x.stride(0), x.stride(1), 0, 0, Bh, L, kind, prune_rank, bits, group,
            bitmaps.data_ptr(), T, tile_offsets.data_ptr(), counts.data_ptr(), units.data_ptr(),
            scales.data_ptr(), zeros.data_ptr(), T, 0, packed.data_ptr(), 0, worst, info.data_ptr(),
            scratch.data_ptr(), need, info.data_ptr() + 4 * Bh, _stream())
        _lib.check(st, "mfar_compress_quant")
    host = info.tolist()                                            # the one host sync
    _lib.check_dev_status(host[Bh], "mfar_compress_quant")
    total = host[Bh - 1] if (Bh and L) else 0
    return dict(bitmaps=bitmaps, tile_offsets=tile_offsets, packed=packed[:total].clone(), counts=counts,
                units=units, scales=scales, zeros=zeros)


class QuantStore:
    """Arena for the quantised format: the seven arrays of ``compress_quant`` with room for ``max_tokens``,
    filled in place by ``append`` (what the reference does with seven ``torch.cat`` per tensor per layer every
    256 steps, ``models/llama_mustafar_quant_kernel.py:305-345``).

    Code words of head h live at ``packed[h, :head_tail[h]]``; ``tile_offsets`` index the flattened ``packed``
    (the kernels reach every tile through them), so the decode ops take this store as they take a compact one."""

    def __init__(self, n_heads: int, max_tokens: int, kind: int, device, bits: int = 2, group: int = 64,
                 words_capacity: int | None = None):
        assert max_tokens % 64 == 0 and kind in (KEY, VALUE) and bits in (2, 4) and group in (32, 64)
        self.n_heads, self.max_tokens, self.kind, self.bits, self.group = n_heads, max_tokens, kind, bits, group
        self.tiles_cap = 2 * max_tokens
        ngrp = 64 // group
        T = self.tiles_cap
        self.words_capacity = T * (64 * bits // 32) if words_capacity is None else int(words_capacity)
        shape = (n_heads, T) if ngrp == 1 else (n_heads, T, ngrp)
        self.bitmaps = torch.empty((n_heads, T), dtype=torch.int64, device=device)
        self.tile_offsets = torch.empty((n_heads, T), dtype=torch.int32, device=device)
        self.counts = torch.empty((n_heads, T), dtype=torch.int32, device=device)
        self.units = torch.empty((n_heads, T), dtype=torch.int32, device=device)
        self.scales = torch.empty(shape, dtype=torch.float16, device=device)
        self.zeros = torch.empty(shape, dtype=torch.float16, device=device)
        self.packed = torch.empty((n_heads, self.words_capacity), dtype=torch.int32, device=device)
        self.head_tail = torch.zeros(n_heads, dtype=torch.int32, device=device)
        self.stats = torch.zeros(1, dtype=torch.int32, device=device)
        self.tokens = 0
        self._scratch = None

    def append(self, x: torch.Tensor, prune_rank: int = 0) -> None:
        """Prune (``prune_rank`` > 0), quantise and store ``x`` [n_heads, n, 128] or [groups, heads per group, n, 128]
        (n % 64 == 0, strided views read in place) behind the tokens held."""
        x = _check_input(x)
        ptr, hs, ts, hpg, gs, heads, n = _source_args(x)
        if heads != self.n_heads:
            raise RuntimeError("head count mismatch")
        if self.tokens + n > self.max_tokens:
            raise RuntimeError("QuantStore is full")
        if n == 0:
            return
        need = _lib.lib().mfar_compress_scratch_bytes(self.n_heads, n)
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, dtype=torch.uint8, device=self.bitmaps.device)
        T = self.tiles_cap
        st = _lib.lib().mfar_compress_quant(
            ptr, hs, ts, hpg, gs, self.n_heads, n, self.kind, prune_rank, self.bits, self.group,
            self.bitmaps.data_ptr(), T, self.tile_offsets.data_ptr(), self.counts.data_ptr(), self.units.data_ptr(),
            self.scales.data_ptr(), self.zeros.data_ptr(), T, 2 * self.tokens, self.packed.data_ptr(),
            self.words_capacity, self.words_capacity, self.head_tail.data_ptr(),
            self._scratch.data_ptr(), self._scratch.numel(), self.stats.data_ptr(), _stream())
        _lib.check(st, "mfar_compress_quant")
        self.tokens += n

    def check(self) -> None:
        """Synchronises and raises if a kernel reported a device-side error (e.g. the code arena is full)."""
        _lib.check_dev_status(int(self.stats[0].item()), "QuantStore")

    def reset(self) -> None:
        """Forgets the stored tokens (the arena stays allocated): the next append starts at token 0."""
        self.tokens = 0
        self.stats.zero_()
        self.head_tail.zero_()

    def as_dict(self) -> dict:
        """The arrays in the shape ``ops_quant.decode_attention_quant`` takes (no copies)."""
        return dict(bitmaps=self.bitmaps, tile_offsets=self.tile_offsets, packed=self.packed.view(-1), counts=self.counts,
                    units=self.units, scales=self.scales, zeros=self.zeros, head_stride=self.tiles_cap)


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
