"""Host side of the fp16 bitmap + packed-value format.

``convert_key_batched`` / ``convert_value_batched`` keep the signatures and
return structures of the reference's ``kernel/compression.py:249-342`` and
``:344-435``.  ``SparseStore`` is the preallocated arena the fused decode path
appends to in place (prune fused into the compression kernel, no per-head
host loop, no reallocation).
"""
from __future__ import annotations

import torch

from . import _lib

KEY, VALUE = 0, 1
D = 128


def keep_rank(sparsity: float, head_dim: int = D) -> int:
    """Rank handed to the selector: the reference prunes with
    ``kthvalue(|x|, max(1, int(sparsity * D)))`` and keeps ``|x| >= thr``
    (``models/llama_mustafar_kernel.py:215-228``)."""
    return max(1, int(sparsity * head_dim))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check_input(x: torch.Tensor) -> torch.Tensor:
    """[heads, tokens, 128], or [groups, heads per group, tokens, 128] (any strides that are multiples of 8 with a
    unit channel stride, e.g. the [batch, token, kv head, 128] projection output viewed as [batch, kv head, token, 128]):
    read in place; anything else is made contiguous first."""
    if not x.is_cuda:
        raise RuntimeError("mustafar_b200: input must be a CUDA tensor (there is no CPU path)")
    if x.dim() not in (3, 4) or x.shape[-1] != D:
        raise RuntimeError(f"expected [heads, tokens, {D}] or [groups, heads, tokens, {D}], got {tuple(x.shape)}")
    if x.dtype != torch.float16:
        raise RuntimeError("expected float16")
    if x.shape[-2] % 64 != 0:
        raise RuntimeError("token count must be a multiple of 64")
    if x.stride(-1) != 1 or any(st % 8 for st in x.stride()[:-1]) or x.data_ptr() % 16:
        x = x.contiguous()
    return x


def _source_args(x: torch.Tensor):
    """(pointer, head stride, token stride, heads per group, group stride, heads, tokens) of a checked input."""
    if x.dim() == 3:
        return x.data_ptr(), x.stride(0), x.stride(1), 0, 0, x.shape[0], x.shape[1]
    return x.data_ptr(), x.stride(1), x.stride(2), x.shape[1], x.stride(0), x.shape[0] * x.shape[1], x.shape[2]


def prune(x: torch.Tensor, sparsity: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """``dh_prune_key`` / ``dh_prune_value`` (``models/llama_mustafar_kernel.py:194-274``)
    on the GPU: x [..., 128] fp16 -> x * (|x| >= kth smallest |x|)."""
    if not x.is_cuda or x.dtype != torch.float16 or x.shape[-1] != D:
        raise RuntimeError("prune expects a CUDA float16 tensor [..., 128]")
    xc = x.contiguous()
    y = torch.empty_like(xc) if out is None else out
    n_rows = xc.numel() // D
    _lib.check(_lib.lib().mfar_prune_fp16(xc.data_ptr(), y.data_ptr(), n_rows, D, keep_rank(sparsity), _stream()),
               "mfar_prune_fp16")
    return y.view(x.shape)


class SparseStore:
    """Compressed K or V of ``n_heads`` (= batch * kv heads) heads, room for ``max_tokens``.

    Layout in HBM (all contiguous, one allocation each):
      bitmaps  int64 [n_heads, 2*max_tokens]       tile t of head h at [h, t]
      accum    int32 [n_heads, 2*max_tokens + 1]   reference ``accum_counts`` (uint32 units)
      nz       fp16  [n_heads, nz_capacity]        packed values, head h starts at h*nz_capacity
    ``tokens`` compressed so far; the first ``2*tokens`` tiles of every head are valid.
    """

    def __init__(self, n_heads: int, max_tokens: int, kind: int, device, nz_capacity: int | None = None):
        assert max_tokens % 64 == 0 and kind in (KEY, VALUE)
        self.n_heads, self.max_tokens, self.kind = n_heads, max_tokens, kind
        self.tiles_cap = 2 * max_tokens
        self.nz_capacity = max_tokens * D if nz_capacity is None else (nz_capacity + 7) // 8 * 8
        self.bitmaps = torch.empty((n_heads, self.tiles_cap), dtype=torch.int64, device=device)
        self.accum = torch.zeros((n_heads, self.tiles_cap + 1), dtype=torch.int32, device=device)
        self.nz = torch.empty((n_heads, self.nz_capacity), dtype=torch.float16, device=device)
        self.tokens = 0
        # [0] dev_status, [1] running max of packed halves per 64-token block
        self.stats = torch.zeros(2, dtype=torch.int32, device=device)
        self._scratch = None
        self._stage_hint = None

    def _scratch_for(self, n_tokens: int) -> torch.Tensor:
        need = _lib.lib().mfar_compress_scratch_bytes(self.n_heads, n_tokens)
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, dtype=torch.uint8, device=self.bitmaps.device)
        return self._scratch

    def append(self, x: torch.Tensor, prune_rank: int = 0) -> None:
        """Compress ``x`` [n_heads, n, 128] or [groups, heads per group, n, 128] (n % 64 == 0; strided views are read
        in place) behind the tokens already stored.  ``prune_rank`` > 0 fuses the magnitude prune (see ``keep_rank``)."""
        x = _check_input(x)
        ptr, hs, ts, hpg, gs, heads, n = _source_args(x)
        if heads != self.n_heads:
            raise RuntimeError("head count mismatch")
        if self.tokens + n > self.max_tokens:
            raise RuntimeError("SparseStore is full")
        if n == 0:
            return
        scratch = self._scratch_for(n)
        st = _lib.lib().mfar_compress_fp16(
            ptr, hs, ts, hpg, gs, self.n_heads, n, self.kind, prune_rank,
            self.bitmaps.data_ptr(), self.tiles_cap, self.accum.data_ptr(), self.tiles_cap + 1, 2 * self.tokens,
            self.nz.data_ptr(), None, self.nz_capacity, self.nz_capacity,
            scratch.data_ptr(), scratch.numel(), self.stats.data_ptr(), self.stats.data_ptr() + 4, _stream())
        _lib.check(st, "mfar_compress_fp16")
        self.tokens += n
        self._stage_hint = None

    def check(self) -> None:
        """Synchronises and raises if a kernel reported a device-side error."""
        _lib.check_dev_status(int(self.stats[0].item()), "SparseStore")

    def reset(self) -> None:
        """Forgets the stored tokens (the arena stays allocated): the next append starts at token 0."""
        self.tokens = 0
        self.stats.zero_()
        self._stage_hint = None

    def stage_hint(self) -> int:
        """Largest packed size (halves) of any block written so far; synchronises once per append."""
        if self._stage_hint is None:
            s = self.stats.tolist()
            _lib.check_dev_status(s[0], "SparseStore")
            self._stage_hint = max(8, (s[1] + 7) // 8 * 8)
        return self._stage_hint

    # -- views in the reference's shapes
    @property
    def tiles(self) -> int:
        return 2 * self.tokens

    def packed_lengths(self) -> torch.Tensor:
        """Halves used per head (device tensor)."""
        return 2 * self.accum[:, self.tiles]


def _convert(inputs: torch.Tensor, kind: int):
    x = _check_input(inputs)
    if x.dim() != 3:
        raise RuntimeError(f"expected [heads, tokens, {D}], got {tuple(x.shape)}")
    Bh, L, _ = x.shape
    store = SparseStore(Bh, max(L, 64), kind, x.device)
    if L:
        store.append(x, 0)
    T = 2 * L
    host = torch.cat([store.packed_lengths(), store.stats[:1]]).tolist()   # the one host sync (the reference has 2*Bh + 1)
    _lib.check_dev_status(host[-1], "SparseStore")
    lengths = host[:-1]
    bitmaps = store.bitmaps[:, :T].contiguous() if store.tiles_cap != T else store.bitmaps
    accum = store.accum[:, :T + 1].contiguous() if store.tiles_cap != T else store.accum
    # one gather launch puts the heads back to back, then per-head views (the reference clones every head, :334-338)
    flat = torch.empty(sum(lengths), dtype=torch.float16, device=x.device)
    _lib.check(_lib.lib().mfar_compact_heads_fp16(store.nz.data_ptr(), store.nz_capacity, store.accum.data_ptr(),
                                                  store.tiles_cap + 1, T, Bh, flat.data_ptr(), flat.numel(), _stream()),
               "mfar_compact_heads_fp16")
    packed = list(flat.split(lengths)) if Bh else []
    return bitmaps, accum, packed


def convert_key_batched(inputs: torch.Tensor):
    """Drop-in for ``kernel/compression.py:249-342``: inputs [B*Hkv, L, 128] (already pruned)
    -> (bitmaps int64 [Bh, T], accum_counts int32 [Bh, T+1], list of Bh fp16 1-D tensors)."""
    return _convert(inputs, KEY)


def convert_value_batched(inputs: torch.Tensor):
    """Drop-in for ``kernel/compression.py:344-435``."""
    return _convert(inputs, VALUE)
