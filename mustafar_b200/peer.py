"""Peer-mapped buffers for the fused all-reduce of the tensor-parallel decode step (one process per GPU, one node).

Each rank allocates ONE block through ``mfar_peer_alloc`` (flag array, then two partial buffers ``[rows, hidden]``
fp16) and sends its 64-byte CUDA IPC handle to the others with ``torch.distributed.all_gather_object``; every rank
maps its peers' blocks with ``mfar_peer_open`` while its own GPU is current, which is what makes the memory reachable
from its kernels.  (torch's own tensor sharing opens the mapping with the owner's device current: good for copies, but
a kernel of another GPU that dereferences such a mapping takes an illegal-address fault.)  ``reduce_add_rmsnorm``
then launches ``mfar_peer_reduce_add_rmsnorm_f16`` (``csrc/peer_reduce.cu``): flags and partials cross NVLink as plain
loads and stores, no NCCL call and no multicast object is involved, and the launch can be captured in a CUDA graph.

A step counter in device memory, bumped by ``end_step()``, makes the epochs grow monotonically across graph replays.
Every wait in the kernel is bounded (``wait_ms``); a rank that gives up sets the timeout bit of ``ops`` status word,
which ``ops.check_device_status`` turns into an exception.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

MAX_PEERS = 8
_FLAG_BYTES = 256          # 8 uint32 flags, padded so that the partials start 256-byte aligned


def epoch_of(step: int, calls_per_step: int, call: int) -> int:
    """Epoch the kernel derives for reduction ``call`` of step ``step`` (what it writes into the peers' flags)."""
    return step * calls_per_step + call + 1


def slot_of(call: int) -> int:
    """Partial buffer (0 or 1) reduction ``call`` of a step uses.  The choice is made on the host, at graph-capture
    time, so it cannot depend on the step: consecutive reductions alternate across step boundaries only when the number
    of calls per step is even, which PeerGroup therefore requires."""
    return call & 1


class _DeviceView:
    """Lets torch view a raw device allocation (torch.as_tensor reads ``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


class PeerGroup:
    def __init__(self, dist, rank: int, world: int, device, rows: int, hidden: int, calls_per_step: int,
                 wait_ms: float = 2000.0, argmax_call: bool = False):
        """``calls_per_step`` reductions per step (even), plus one arg-max exchange per step when ``argmax_call``
        (it takes the call index ``calls_per_step`` and has a buffer of its own)."""
        if world > MAX_PEERS:
            raise RuntimeError(f"at most {MAX_PEERS} ranks")
        if calls_per_step <= 0 or calls_per_step % 2:
            raise RuntimeError("calls_per_step must be even: the two partial buffers alternate from call to call, also "
                               "from the last call of a step to the first of the next")
        self.rank, self.world, self.dev = rank, world, torch.device(device)
        self.rows, self.hidden, self.calls_per_step = rows, hidden, calls_per_step
        self.epoch_calls = calls_per_step + (1 if argmax_call else 0)      # flag epochs consumed per step
        self.wait_ns = int(wait_ms * 1e6)
        self._dist = dist
        L = _lib.lib()
        slot_bytes = rows * hidden * 2
        pair_off = _FLAG_BYTES + 2 * slot_bytes                        # (value, index) per row for the arg-max exchange
        nbytes = pair_off + 8 * rows
        self._base = C.c_void_p()
        handle = C.create_string_buffer(64)
        self._mapped: list[int] = []
        # every rank goes through the same collectives whatever fails locally, then all raise together: a rank that
        # left early would pair its next collective with the others' barrier
        failure = None
        with torch.cuda.device(self.dev):
            try:
                _lib.check(L.mfar_peer_alloc(nbytes, C.byref(self._base), handle), "mfar_peer_alloc")
                mine = handle.raw
            except Exception as e:
                failure, mine = e, None
            gathered = [None] * world
            dist.all_gather_object(gathered, mine)
            bases = []
            if failure is None and any(g is None for g in gathered):
                failure = RuntimeError("a peer rank could not allocate its buffers")
            for r in range(world):
                if failure is not None:
                    break
                if r == rank:
                    bases.append(self._base.value)
                    continue
                ptr = C.c_void_p()
                try:
                    _lib.check(L.mfar_peer_open(C.create_string_buffer(gathered[r], 64), C.byref(ptr)), f"mfar_peer_open(rank {r})")
                except Exception as e:
                    failure = e
                    break
                self._mapped.append(ptr.value)
                bases.append(ptr.value)
            everybody = torch.tensor([0.0 if failure is not None else 1.0], device=self.dev)
            dist.all_reduce(everybody, op=dist.ReduceOp.MIN)
            if float(everybody) == 0.0:
                for ptr in self._mapped:
                    L.mfar_peer_close(ptr)
                self._mapped = []
                dist.barrier()          # nobody frees while a peer may still hold a mapping
                if self._base.value:
                    L.mfar_peer_free(self._base)
                self._base = None
                raise RuntimeError(f"peer buffers could not be set up on every rank ({failure or 'another rank failed'})")
        base = self._base.value
        self.flags = torch.as_tensor(_DeviceView(base, (MAX_PEERS,), "<i4"), device=self.dev)
        self.partials = torch.as_tensor(_DeviceView(base + _FLAG_BYTES, (2, rows, hidden), "<f2"), device=self.dev)
        self.step = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self._one = torch.ones(1, dtype=torch.int32, device=self.dev)
        torch.cuda.synchronize(self.dev)
        dist.barrier()      # every rank has opened every handle before anybody writes
        self._ptr_arrays = {slot: (C.c_void_p * world)(*[b + _FLAG_BYTES + slot * slot_bytes for b in bases]) for slot in (0, 1)}
        self._flag_array = (C.c_void_p * world)(*bases)
        self._pair_array = (C.c_void_p * world)(*[b + pair_off for b in bases])

    def close(self) -> None:
        """Collective: unmaps the peers' blocks, then (after a barrier) frees this rank's own."""
        if self._base is None:
            return
        torch.cuda.synchronize(self.dev)
        L = _lib.lib()
        with torch.cuda.device(self.dev):
            for ptr in self._mapped:
                L.mfar_peer_close(ptr)
            self._mapped = []
            self._dist.barrier()
            self.flags = self.partials = None
            L.mfar_peer_free(self._base)
        self._base = None

    def slot(self, call: int) -> torch.Tensor:
        """The local partial buffer of call ``call`` of a step: the producer (a GEMM with ``out=``) writes here."""
        return self.partials[slot_of(call)]

    def reduce_add_rmsnorm(self, x: torch.Tensor, call: int, weight: torch.Tensor, eps: float,
                           out: torch.Tensor | None = None) -> torch.Tensor:
        """``x += sum over ranks of slot(call)`` in place, returns ``rmsnorm(x) * weight``; x [rows, hidden] fp16."""
        from .ops import _dev_status
        if x.shape != (self.rows, self.hidden) or x.dtype != torch.float16 or not x.is_contiguous():
            raise RuntimeError("reduce_add_rmsnorm: x must be contiguous float16 [rows, hidden] as given at construction")
        if out is None:
            out = torch.empty_like(x)
        st = _lib.lib().mfar_peer_reduce_add_rmsnorm_f16(
            x.data_ptr(), self._ptr_arrays[slot_of(call)], self._flag_array, self.world, self.rank, self.step.data_ptr(), 0,
            self.epoch_calls, call, weight.data_ptr(), out.data_ptr(), self.rows, self.hidden, float(eps),
            self.wait_ns, _dev_status(x.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
        _lib.check(st, "mfar_peer_reduce_add_rmsnorm_f16")
        return out

    def argmax(self, logits: torch.Tensor, vocab_offset: int, out: torch.Tensor | None = None) -> torch.Tensor:
        """logits [rows, n_local] fp16: this rank's slice of the vocabulary, starting at ``vocab_offset`` -> int64 [rows],
        the index of the largest logit over all ranks' slices (the smallest index among equals), the same on every
        rank.  Takes the step's last call index; the group must have been built with ``argmax_call=True``."""
        from .ops import _dev_status
        if self.epoch_calls == self.calls_per_step:
            raise RuntimeError("PeerGroup was built without argmax_call=True")
        if logits.dim() != 2 or logits.shape[0] != self.rows or logits.dtype != torch.float16 or logits.stride(1) != 1 \
                or logits.shape[1] % 8 or logits.stride(0) % 8 or logits.data_ptr() % 16:
            raise RuntimeError("argmax: logits must be float16 [rows, n_local], n_local a multiple of 8, rows 16-byte aligned")
        if out is None:
            out = torch.empty(self.rows, dtype=torch.int64, device=logits.device)
        st = _lib.lib().mfar_peer_argmax_f16(
            logits.data_ptr(), logits.stride(0), self.rows, logits.shape[1], int(vocab_offset), self._pair_array,
            self._flag_array, self.world, self.rank, self.step.data_ptr(), 0, self.epoch_calls, self.calls_per_step,
            out.data_ptr(), self.wait_ns, _dev_status(logits.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
        _lib.check(st, "mfar_peer_argmax_f16")
        return out

    def end_step(self) -> None:
        """Advances the step counter on the device (stream ordered, capturable): call once after the last reduction."""
        self.step += self._one
