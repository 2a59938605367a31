"""Llama-3-8B-shaped decoder that keeps its KV cache in the sparse format and decodes through
the fused attention entry (the patched counterpart of the reference's model glue,
``models/llama_mustafar_kernel.py:320-599``, not an edit of it).

What differs from the reference layer:
  * the cache is a pair of preallocated ``SparseStore`` arenas per layer plus a fixed-capacity dense
    window; nothing is ``torch.cat``-ed, padded to 8 rows or copied per step;
  * prune and compression are one kernel (prefill: the first ``((T - residual) // 256) * 256``
    tokens, ``:540-557``; decode: the oldest 256 tokens whenever the window reaches
    ``residual + 256``, ``:445-519``).  That is ``prune_mode="block"``, the reference's kernel model.
    ``prune_mode="step"`` prunes like the reference's torch path instead
    (``models/llama_mustafar_Kt_Mag_Vt_Mag.py:917-926,1015-1024``): every decode step the token that leaves the
    ``residual`` most recent ones is pruned in place in the window (inside the RoPE / append launch), so only
    ``residual`` tokens are ever dense; compression still happens 256 tokens at a time, on rows already pruned;
  * q.K^T over compressed + window, softmax and P.V are one call per layer per step.
Linear layers, RMSNorm, RoPE and the dense causal prefill attention are plain torch (cuBLAS /
SDPA); they are outside the hot path this package accelerates.

Weights are random (normal, std 0.02, seeded) with the Llama-3-8B shapes; with tensor parallelism
every rank slices the SAME full matrices by head (q/k/v/gate/up by column, o/down by row) and the
partial sums meet in an NCCL all-reduce after ``o_proj`` and ``down_proj``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import compression as comp
from . import compression_quant as cq
from . import ops, ops_quant, step_ops

D = 128


@dataclass
class LlamaShape:
    hidden: int = 4096
    n_layers: int = 32
    n_q_heads: int = 32
    n_kv_heads: int = 8
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5


def tiny_shape() -> LlamaShape:
    """Same head layout (head_dim 128, 4 q heads per kv head), small everything else: for tests."""
    return LlamaShape(hidden=256, n_layers=2, n_q_heads=8, n_kv_heads=2, ffn=512, vocab=1000)


def _rms(x, w, eps):
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope(x, pos, theta):
    """x [..., T, D] with positions pos [T] (rotate-half convention)."""
    half = x.shape[-1] // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, device=x.device, dtype=torch.float32) / half))
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


class _Layer:
    __slots__ = ("wqkv", "wo", "wgu", "wd", "n1", "n2", "ks", "vs", "kwin", "vwin")


class SparseLlama:
    """Inference-only model object; one instance per rank."""

    def __init__(self, shape: LlamaShape, batch: int, max_tokens: int, device, sparsity: float = 0.7,
                 residual: int = 128, seed: int = 0, tp_rank: int = 0, tp_world: int = 1, dist=None,
                 sparse: bool = True, cache_bits: int = 16, prune_mode: str = "block", tp_fused: bool = False,
                 lm_head_parallel: bool = False):
        assert shape.n_kv_heads % tp_world == 0 and shape.ffn % tp_world == 0
        self.s, self.B, self.dev = shape, batch, torch.device(device)
        self.sparsity, self.residual, self.sparse = sparsity, residual, sparse
        # 16: pruned values kept as fp16; 2 or 4: pruned values quantised per tile (the reference's quantised model,
        # models/llama_mustafar_quant_kernel.py)
        assert cache_bits in (16, 2, 4) and prune_mode in ("block", "step")
        self.step_prune = prune_mode == "step"
        self.cache_bits, self.quant = cache_bits, sparse and cache_bits != 16
        self.tp_rank, self.tp_world, self.dist = tp_rank, tp_world, dist
        self.hq = shape.n_q_heads // tp_world
        self.hkv = shape.n_kv_heads // tp_world
        self.G = shape.n_q_heads // shape.n_kv_heads
        self.max_tokens = (max_tokens + 255) // 256 * 256
        self.wcap = residual + 256
        self.rank_keep = comp.keep_rank(sparsity)
        self.tokens = 0          # tokens seen so far
        self.compressed = 0      # of which compressed
        self.wlen = 0            # tokens in the dense window
        g = torch.Generator(device=self.dev).manual_seed(seed)

        def rnd(*shape_):
            return (torch.randn(*shape_, generator=g, device=self.dev, dtype=torch.float32) * 0.02).half()

        hd, f = shape.hidden, shape.ffn
        fl = f // tp_world
        q0, k0 = tp_rank * self.hq * D, tp_rank * self.hkv * D
        self.embed = rnd(shape.vocab, hd)
        self.lm_head = rnd(shape.vocab, hd)
        # vocabulary-parallel lm_head (only with the peer buffers, whose arg-max exchange picks the token): this rank
        # keeps the rows of its slice of the vocabulary; logits are then local and `decode_next` returns the ids
        self.vocab_parallel = bool(lm_head_parallel and tp_fused and tp_world > 1 and sparse)
        self.v0 = 0
        if self.vocab_parallel:
            vl = shape.vocab // tp_world
            if shape.vocab % tp_world or vl % 8:
                raise RuntimeError("vocabulary-parallel lm_head needs vocab / ranks to be a multiple of 8")
            self.v0 = tp_rank * vl
            self.lm_head = self.lm_head[self.v0:self.v0 + vl].contiguous()
            self._tok_out = torch.empty(batch, dtype=torch.int64, device=self.dev)
        self.norm = torch.ones(hd, dtype=torch.float16, device=self.dev)
        self.layers = []
        Bh = batch * self.hkv
        for _ in range(shape.n_layers):
            L = _Layer()
            wq, wk, wv = rnd(shape.n_q_heads * D, hd), rnd(shape.n_kv_heads * D, hd), rnd(shape.n_kv_heads * D, hd)
            L.wqkv = torch.cat([wq[q0:q0 + self.hq * D], wk[k0:k0 + self.hkv * D], wv[k0:k0 + self.hkv * D]]).contiguous()
            L.wo = rnd(hd, shape.n_q_heads * D)[:, q0:q0 + self.hq * D].contiguous()
            wg, wu = rnd(f, hd), rnd(f, hd)
            L.wgu = torch.cat([wg[tp_rank * fl:(tp_rank + 1) * fl], wu[tp_rank * fl:(tp_rank + 1) * fl]]).contiguous()
            L.wd = rnd(hd, f)[:, tp_rank * fl:(tp_rank + 1) * fl].contiguous()
            L.n1 = torch.ones(hd, dtype=torch.float16, device=self.dev)
            L.n2 = torch.ones(hd, dtype=torch.float16, device=self.dev)
            del wq, wk, wv, wg, wu
            if sparse:
                if self.quant:
                    # code arena sized for the worst case (every tile full): 64 * bits / 32 words per tile
                    L.ks = cq.QuantStore(Bh, self.max_tokens, comp.KEY, self.dev, cache_bits, 64)
                    L.vs = cq.QuantStore(Bh, self.max_tokens, comp.VALUE, self.dev, cache_bits, 64)
                else:
                    cap = int(self.max_tokens * D * min(1.0, (1.0 - sparsity) + 0.25)) // 8 * 8
                    L.ks = comp.SparseStore(Bh, self.max_tokens, comp.KEY, self.dev, nz_capacity=cap)
                    L.vs = comp.SparseStore(Bh, self.max_tokens, comp.VALUE, self.dev, nz_capacity=cap)
                L.kwin = torch.empty(Bh, self.wcap, D, dtype=torch.float16, device=self.dev)
                L.vwin = torch.empty(Bh, self.wcap, D, dtype=torch.float16, device=self.dev)
            else:   # dense reference cache: pruned tokens kept with their zeros (the torch accuracy path)
                L.ks = torch.empty(Bh, self.max_tokens + self.wcap, D, dtype=torch.float16, device=self.dev)
                L.vs = torch.empty(Bh, self.max_tokens + self.wcap, D, dtype=torch.float16, device=self.dev)
                L.kwin = L.vwin = None
            self.layers.append(L)
        self._stage_hint = None
        self._graph = None
        self._eager_done = False
        self._inv_freq = None
        self._qbuf = None
        # largest packed size of a 64-token block that can still come (what a replayed launch stages for): the kept
        # values of 64 tokens, a few ties, and the worst padding of its 128 tiles
        kept = D - self.rank_keep + 1
        self._stage_bound = min(8192, 64 * (kept + 3) + 7 * 128)
        # the decode calls of this model write their split records here: a buffer of its own, sized for the full
        # cache, so that captured graphs never see it move and other users of the ops cannot grow it away
        self.prefill_compress_ms = self.prefill_attention_ms = 0.0
        # tensor parallel decode: partial sums meet in NCCL all-reduces between CUDA graphs, or (tp_fused) in the
        # peer-buffer reduction fused with the residual add + RMSNorm, which lets the whole step be one graph
        self.peer = None
        if tp_world > 1 and tp_fused and sparse:
            from .peer import PeerGroup
            self.peer = PeerGroup(dist, tp_rank, tp_world, self.dev, batch, shape.hidden, 2 * shape.n_layers,
                                  argmax_call=self.vocab_parallel)
        self._decode_ws = None
        if self.sparse:
            _, nbytes = ops.plan(batch * self.hkv, self.max_tokens, self.wcap, self.G)
            nbytes = max(nbytes, 65536 + batch * self.hkv * (self.max_tokens // 64 + 1) * self.G * 132 * 4)
            self._decode_ws = ops.new_workspace(self.dev, nbytes)

    # ------------------------------------------------------------------ pieces
    def _allreduce(self, x):
        if self.tp_world > 1:
            self.dist.all_reduce(x)
        return x

    def _mlp(self, L, x):
        gu = F.linear(x, L.wgu)
        fl = gu.shape[-1] // 2
        return self._allreduce(F.linear(F.silu(gu[..., :fl]) * gu[..., fl:], L.wd))

    def _qkv(self, L, x, pos):
        """x [B, T, hidden] -> q [B, hq, T, D], k, v [B, hkv, T, D] with RoPE applied to q and k."""
        B, T, _ = x.shape
        qkv = F.linear(x, L.wqkv)
        q, k, v = qkv.split([self.hq * D, self.hkv * D, self.hkv * D], dim=-1)
        q = _rope(q.view(B, T, self.hq, D).transpose(1, 2), pos, self.s.rope_theta)
        k = _rope(k.view(B, T, self.hkv, D).transpose(1, 2), pos, self.s.rope_theta)
        return q, k, v.view(B, T, self.hkv, D).transpose(1, 2)

    def _logits(self, x):
        return F.linear(_rms(x, self.norm, self.s.rms_eps), self.lm_head)

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, T] -> logits of the last position [B, vocab]; fills the caches.

        The cache work of a layer (prune + compression of the first ``Lc`` tokens, copy of the rest into the dense
        window) runs on a side stream straight from the projection outputs - K after RoPE, V as the strided
        [B, T, kv head, 128] view of the fused q|k|v GEMM result, neither is copied or flattened first - while the main
        stream goes on with this layer's attention and MLP and the next layer's GEMMs (the reference compresses
        between layers with the GPU otherwise idle, ``models/llama_mustafar_kernel.py:540-560``).  The device time of
        the cache work and of the dense attention is kept in ``prefill_compress_ms`` / ``prefill_attention_ms``."""
        B, T = tokens.shape
        assert B == self.B and self.tokens == 0 and T <= self.max_tokens + self.residual
        pos = torch.arange(T, device=self.dev)
        Lc = max(0, (T - self.residual) // 256) * 256
        x = self.embed[tokens]
        main = torch.cuda.current_stream(self.dev)
        side = torch.cuda.Stream(self.dev) if self.sparse else None
        marks = []
        for L in self.layers:
            h = _rms(x, L.n1, self.s.rms_eps)
            q, k, v = self._qkv(L, h, pos)
            if self.sparse:
                ready = torch.cuda.Event()
                ready.record(main)
                with torch.cuda.stream(side):
                    side.wait_event(ready)
                    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    c0.record(side)
                    if Lc:
                        L.ks.append(k[:, :, :Lc], self.rank_keep)       # strided 4-D views: nothing is copied
                        L.vs.append(v[:, :, :Lc], self.rank_keep)
                    L.kwin.view(B, self.hkv, self.wcap, D)[:, :, :T - Lc] = k[:, :, Lc:]
                    L.vwin.view(B, self.hkv, self.wcap, D)[:, :, :T - Lc] = v[:, :, Lc:]
                    if self.step_prune and T - Lc > self.residual:      # only the newest `residual` tokens stay dense
                        n = T - Lc - self.residual
                        L.kwin[:, :n] = comp.prune(L.kwin[:, :n].contiguous(), self.sparsity)
                        L.vwin[:, :n] = comp.prune(L.vwin[:, :n].contiguous(), self.sparsity)
                    c1.record(side)
                    marks.append(("compress", c0, c1))
                k.record_stream(side)
                v.record_stream(side)
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(main)
            att = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
            a1.record(main)
            marks.append(("attention", a0, a1))
            x = x + self._allreduce(F.linear(att.transpose(1, 2).reshape(B, T, self.hq * D), L.wo))
            x = x + self._mlp(L, _rms(x, L.n2, self.s.rms_eps))
            if not self.sparse:
                kf, vf = k.reshape(B * self.hkv, T, D), v.reshape(B * self.hkv, T, D)
                L.ks[:, :T], L.vs[:, :T] = kf, vf
                Lp = max(Lc, T - self.residual) if self.step_prune else Lc
                if Lp > 0:
                    L.ks[:, :Lp] = comp.prune(kf[:, :Lp].contiguous(), self.sparsity)
                    L.vs[:, :Lp] = comp.prune(vf[:, :Lp].contiguous(), self.sparsity)
            del q, k, v, att
        if side is not None:
            main.wait_stream(side)
        self.tokens, self.compressed, self.wlen = T, Lc, T - Lc
        self._stage_hint = None
        if self._graph is not None:     # a step graph captured during an earlier generation: point its counters here
            self._state.copy_(torch.tensor([self.tokens, self.wlen, self.wlen + 1, self.compressed], dtype=torch.int32))
        out = self._logits(x[:, -1])
        torch.cuda.synchronize(self.dev)
        self.prefill_compress_ms = sum(a.elapsed_time(b) for n, a, b in marks if n == "compress")
        self.prefill_attention_ms = sum(a.elapsed_time(b) for n, a, b in marks if n == "attention")
        return out

    # ------------------------------------------------------------------ one decode step
    def _hint(self):
        if self._stage_hint is None:
            self._stage_hint = max(max(L.ks.stage_hint(), L.vs.stage_hint()) for L in self.layers) if self.compressed else 8
        return self._stage_hint

    def _step_body(self, token: torch.Tensor, dev_state: bool) -> torch.Tensor:
        """One decode step for token ids [B].  With dev_state the position and the window length are
        read from a device tensor (and advanced on the device), so the launch sequence can be captured
        in a CUDA graph and replayed; otherwise they are the host counters.  The dense comparison arm
        (sparse=False) is plain torch: fp32 attention over the pruned tensors."""
        if self.sparse:
            return self._step_body_fused(token, dev_state)
        B = self.B
        x = self.embed[token].view(B, 1, -1)
        pos = torch.tensor([self.tokens], device=self.dev)
        t = self.tokens
        for L in self.layers:
            h = _rms(x, L.n1, self.s.rms_eps)
            q, k, v = self._qkv(L, h, pos)
            L.ks[:, t], L.vs[:, t] = k.reshape(B * self.hkv, D), v.reshape(B * self.hkv, D)
            if self.step_prune and t - self.residual - 1 >= 0:
                o = t - self.residual - 1
                L.ks[:, o] = comp.prune(L.ks[:, o].contiguous(), self.sparsity)
                L.vs[:, o] = comp.prune(L.vs[:, o].contiguous(), self.sparsity)
            kk = L.ks[:, :t + 1].float().repeat_interleave(self.G, dim=0)
            vv = L.vs[:, :t + 1].float().repeat_interleave(self.G, dim=0)
            sc = torch.bmm(kk, q.reshape(B * self.hq, D, 1).float()).squeeze(-1) / math.sqrt(D)
            att = torch.bmm(torch.softmax(sc, -1).unsqueeze(1), vv).squeeze(1).half()
            x = x + self._allreduce(F.linear(att.view(B, 1, self.hq * D), L.wo))
            x = x + self._mlp(L, _rms(x, L.n2, self.s.rms_eps))
        return self._logits(x[:, 0])

    def _step_segments(self, token: torch.Tensor, dev_state: bool):
        """The sparse-cache step with the glue fused (step_ops): per layer RMSNorm(+residual add), q|k|v GEMM,
        RoPE + window append, sparse attention, o_proj, RMSNorm(+add), gate|up GEMM, SiLU*up, down GEMM.

        A generator: under tensor parallelism it yields every partial sum that needs an all-reduce (in place,
        done by the caller) and resumes after it, so that the stretches between two collectives can each be
        captured in a CUDA graph of their own while NCCL stays outside any capture.  The logits end up in
        ``self._step_out``."""
        B, eps = self.B, self.s.rms_eps
        if self._inv_freq is None:
            self._inv_freq = step_ops.rope_inv_freq(self.s.rope_theta, self.dev)
            self._qbuf = torch.empty(B * self.hq, D, dtype=torch.float16, device=self.dev)
        hint = 0 if (dev_state or self.quant) else self._hint()
        w = self.wlen
        pr = dict(prune_rank=self.rank_keep, prune_back=self.residual) if self.step_prune else {}
        peer = self.peer
        tp = self.tp_world > 1 and peer is None
        x = self.embed[token]                     # [B, hidden], updated in place from here on
        delta = None
        call = 0                                  # peer reductions issued so far in this step

        def add_norm(delta, w):
            """residual add + RMSNorm; with peer buffers `delta` is the partial left in slot(call - 1) by the GEMM"""
            if peer is not None and delta is not None:
                return peer.reduce_add_rmsnorm(x, call - 1, w, eps)
            return step_ops.add_rmsnorm(x, delta, w, eps)

        def row_parallel(inp, w):
            """GEMM whose output is a partial sum over ranks: straight into the peer-visible buffer when there is one"""
            nonlocal call
            if peer is None:
                return F.linear(inp, w)
            out = peer.slot(call)
            torch.mm(inp, w.t(), out=out)
            call += 1
            return out

        for L in self.layers:
            h = add_norm(delta, L.n1)
            qkv = F.linear(h, L.wqkv)
            if dev_state and self.quant:
                step_ops.rope_append(qkv, self._inv_freq, self._state[0:1], self._state[1:2], self.hq, self.hkv,
                                     self._qbuf, L.kwin, L.vwin, **pr)
                att = ops_quant.decode_attention_quant(self._qbuf, L.ks.as_dict(), L.vs.as_dict(), self.max_tokens,
                                                       L.kwin, L.vwin, self.G, self.cache_bits,
                                                       n_tokens_dev=self._state[3:4], window_len=self._state[2:3],
                                                       workspace=self._decode_ws)
            elif dev_state:
                step_ops.rope_append(qkv, self._inv_freq, self._state[0:1], self._state[1:2], self.hq, self.hkv,
                                     self._qbuf, L.kwin, L.vwin, **pr)
                att = ops.decode_attention(self._qbuf, L.ks, L.vs, L.kwin, L.vwin, self.G, stage_halves=self._stage_bound,
                                           window_len=self._state[2:3], n_tokens=self._state[3:4],
                                           workspace=self._decode_ws)
            elif self.quant:
                step_ops.rope_append(qkv, self._inv_freq, self.tokens, w, self.hq, self.hkv, self._qbuf, L.kwin, L.vwin, **pr)
                att = ops_quant.decode_attention_quant(self._qbuf, L.ks.as_dict(), L.vs.as_dict(), self.compressed,
                                                       L.kwin[:, :w + 1], L.vwin[:, :w + 1], self.G, self.cache_bits,
                                                       workspace=self._decode_ws)
            else:
                step_ops.rope_append(qkv, self._inv_freq, self.tokens, w, self.hq, self.hkv, self._qbuf, L.kwin, L.vwin, **pr)
                att = ops.decode_attention(self._qbuf, L.ks, L.vs, L.kwin[:, :w + 1], L.vwin[:, :w + 1], self.G,
                                           stage_halves=hint, workspace=self._decode_ws)
            o = row_parallel(att.view(B, self.hq * D), L.wo)
            if tp:
                yield o
            h = add_norm(o, L.n2)
            delta = row_parallel(step_ops.silu_mul(F.linear(h, L.wgu)), L.wd)
            if tp:
                yield delta
        if dev_state:
            self._state += self._state_step
        self._step_out = F.linear(add_norm(delta, self.norm), self.lm_head)
        if self.vocab_parallel:
            self._step_tok = peer.argmax(self._step_out, self.v0, out=self._tok_out)
        if peer is not None:
            peer.end_step()

    def _step_body_fused(self, token: torch.Tensor, dev_state: bool) -> torch.Tensor:
        for partial in self._step_segments(token, dev_state):
            self.dist.all_reduce(partial)
        return self._step_out

    def _capture_step(self):
        """Captures the step as one CUDA graph per stretch between two collectives (a single graph without
        tensor parallelism).  Returns [(graph, tensor to all-reduce after it or None)]; replay in order."""
        # capture_begin / capture_end on a side stream, without the garbage collection and the allocator purge
        # that `with torch.cuda.graph(...)` adds on entry: after a prefill the purge alone can take most of a second
        pool = torch.cuda.graph_pool_handle()
        gen = self._step_segments(self._tok_buf, True)
        out = []
        side = torch.cuda.Stream(device=self.dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            while True:
                g = torch.cuda.CUDAGraph()
                partial = None
                g.capture_begin(pool=pool)
                try:
                    try:
                        partial = next(gen)
                    except StopIteration:
                        pass
                finally:
                    g.capture_end()
                out.append((g, partial))
                if partial is None:
                    break
        torch.cuda.current_stream().wait_stream(side)
        return out

    def _advance(self):
        self.tokens += 1
        self.wlen += 1
        if self.wlen == self.wcap:
            self._compress_oldest()
            if self._graph is not None:
                # the captured launches read their lengths on the device: move the window back by one block and
                # the compressed length forward; nothing is re-captured
                self._state += self._state_append
                for L in self.layers:
                    L.ks.check()
                    L.vs.check()
                ops.check_device_status()
                # the replayed launches stage `_stage_bound` halves per block; a block with more (tokens with many ties
                # at the pruning threshold) would only be noticed when it is first decoded, one step later: say so now
                need = 0 if self.quant else max(max(L.ks.stage_hint(), L.vs.stage_hint()) for L in self.layers)
                if need > self._stage_bound:
                    raise RuntimeError(f"a compressed block holds {need} halves, the captured decode launches stage "
                                       f"{self._stage_bound}: replay would skip it; decode eagerly (graph=False)")

    @torch.no_grad()
    def decode_step(self, token: torch.Tensor, graph: bool = False) -> torch.Tensor:
        """token [B] (ids of the newest position) -> logits [B, vocab].

        graph=True replays CUDA graphs of the step, captured once after a first eager step: position, window
        length and compressed length live in a device tensor that the captured kernels read, so appending a block
        needs no new capture.  Under tensor parallelism the step is a chain of graphs with the NCCL all-reduces
        launched between them."""
        if not (graph and self.sparse):
            out = self._step_body(token, False)
            self._advance()
            return out
        if self._graph is None:
            if not self._eager_done:
                self._eager_done = True
                out = self._step_body(token, False)       # sizes workspaces, resolves the stage hint
                self._advance()
                return out
            # position, window slot of the new token, window length, compressed length: read on the device
            self._state = torch.tensor([self.tokens, self.wlen, self.wlen + 1, self.compressed], device=self.dev,
                                       dtype=torch.int32)
            self._state_step = torch.tensor([1, 1, 1, 0], device=self.dev, dtype=torch.int32)
            self._state_append = torch.tensor([0, -256, -256, 256], device=self.dev, dtype=torch.int32)
            self._tok_buf = token.clone()
            torch.cuda.synchronize()
            self._graph = self._capture_step()
        self._tok_buf.copy_(token)
        for g, partial in self._graph:
            g.replay()
            if partial is not None:
                self.dist.all_reduce(partial)
        out = self._step_out
        self._advance()
        return out

    def _compress_oldest(self):
        """The window reached residual + 256 tokens: its oldest 256 join the compressed cache."""
        c = self.compressed
        for L in self.layers:
            if self.sparse:
                rank = self.rank_keep
                if self.step_prune:
                    # slots 0..254 were pruned step by step; the last one would have been pruned by the next step
                    L.kwin[:, 255] = comp.prune(L.kwin[:, 255].contiguous(), self.sparsity)
                    L.vwin[:, 255] = comp.prune(L.vwin[:, 255].contiguous(), self.sparsity)
                    rank = 0
                L.ks.append(L.kwin[:, :256], rank)
                L.vs.append(L.vwin[:, :256], rank)
                L.kwin[:, :self.residual] = L.kwin[:, 256:].clone()
                L.vwin[:, :self.residual] = L.vwin[:, 256:].clone()
            elif not self.step_prune:
                L.ks[:, c:c + 256] = comp.prune(L.ks[:, c:c + 256].contiguous(), self.sparsity)
                L.vs[:, c:c + 256] = comp.prune(L.vs[:, c:c + 256].contiguous(), self.sparsity)
        self.compressed += 256
        self.wlen -= 256
        self._stage_hint = None

    @torch.no_grad()
    def reset(self) -> None:
        """Ends a generation: the caches are empty again, allocations and the captured step graph stay, so the next
        ``prefill`` starts a new generation that replays the same graph."""
        self.tokens = self.compressed = self.wlen = 0
        self._stage_hint = None
        if self.sparse:
            for L in self.layers:
                L.ks.reset()
                L.vs.reset()

    @torch.no_grad()
    def warm_up(self, graph: bool = True) -> None:
        """One short throw-away generation (prefill of 448 tokens, a few steps) so that the one-off costs - library
        initialisation, the first eager step, the capture and instantiation of the step graph - are paid before real
        traffic, as a serving process does at start-up.  Collective under tensor parallelism."""
        toks = torch.zeros(self.B, 256 + 128 + 64, dtype=torch.long, device=self.dev)
        nxt = self.prefill_next(toks)
        for _ in range(4):
            nxt = self.decode_next(nxt, graph)
        torch.cuda.synchronize(self.dev)
        self.reset()

    @torch.no_grad()
    def prefill_next(self, tokens: torch.Tensor) -> torch.Tensor:
        """prefill, then the greedy choice for the next position [B] (with a vocabulary-parallel lm_head the ranks'
        local logits meet in the peer arg-max exchange; otherwise a plain arg-max)."""
        logits = self.prefill(tokens)
        if not self.vocab_parallel:
            return logits.argmax(-1)
        self._logits_last = logits = logits.contiguous()
        tok = self.peer.argmax(logits, self.v0).clone()
        self.peer.end_step()
        return tok

    @torch.no_grad()
    def decode_next(self, token: torch.Tensor, graph: bool = False) -> torch.Tensor:
        """One decode step and the greedy choice for the position after it [B] (see prefill_next)."""
        logits = self.decode_step(token, graph)
        return self._step_tok.clone() if self.vocab_parallel else logits.argmax(-1)

    def generate(self, tokens: torch.Tensor, steps: int, graph: bool = False):
        """Greedy decoding; returns the generated ids [B, steps]."""
        nxt = self.prefill_next(tokens)
        out = [nxt]
        for _ in range(steps - 1):
            nxt = self.decode_next(nxt, graph)
            out.append(nxt)
        return torch.stack(out, dim=1)
