"""The fused peer reduction + residual add + RMSNorm kernel (mfar_peer_reduce_add_rmsnorm_f16) on ONE GPU.

The kernel of rank 0 of a 2-rank group runs alone: the "peer" partial and the peer's flag array are ordinary local
buffers.  With the peer's flag set by the host beforehand the kernel must produce x + p0 + p1 and its RMSNorm; with the
flag never set the bounded wait must run out, report MFAR_DEV_TIMEOUT and leave x and out untouched (the failure is
made by not signalling, never by faulting).  The two-GPU run of the same kernel is in test_gpu_tensor_parallel.py."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def call(lib, x, parts, flags, step_dev, call_idx, w, out, status, wait_ms):
    pa = (C.c_void_p * 2)(parts[0].data_ptr(), parts[1].data_ptr())
    fa = (C.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    return lib.mfar_peer_reduce_add_rmsnorm_f16(
        x.data_ptr(), pa, fa, 2, 0, step_dev.data_ptr(), 0, 4, call_idx, w.data_ptr(), out.data_ptr(), x.shape[0],
        x.shape[1], 1e-5, int(wait_ms * 1e6), status.data_ptr(), torch.cuda.current_stream().cuda_stream)


def setup(rows=5, hidden=1024):
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(rows, hidden, generator=g, device="cuda").half()
    parts = [torch.randn(rows, hidden, generator=g, device="cuda").half() for _ in range(2)]
    w = (1 + 0.1 * torch.randn(hidden, generator=g, device="cuda")).half()
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    return x, parts, w, flags


def test_sums_partials_in_fp32_then_normalises():
    from mustafar_b200 import _lib
    lib = _lib.lib()
    x, parts, w, flags = setup()
    step = torch.tensor([7], dtype=torch.int32, device="cuda")
    flags[0][1] = 7 * 4 + 2 + 1                       # the peer has announced call 2 of step 7 already
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros_like(x)
    x0 = x.clone()
    assert call(lib, x, parts, flags, step, 2, w, out, status, 1000) == 0
    torch.cuda.synchronize()
    assert int(status) == 0
    want_x = (x0.float() + parts[0].float() + parts[1].float()).half()
    assert torch.equal(x, want_x)
    xf = want_x.float()
    want = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).half() * w
    assert (out.float() - want.float()).abs().max() <= 2e-3 * want.float().abs().max()
    assert int(flags[1][0]) == 7 * 4 + 2 + 1          # this rank's announcement reached the "peer"


def test_missing_peer_signal_times_out_and_writes_nothing():
    from mustafar_b200 import _lib
    lib = _lib.lib()
    x, parts, w, flags = setup()
    step = torch.tensor([1], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros_like(x)
    x0 = x.clone()
    assert call(lib, x, parts, flags, step, 0, w, out, status, 30) == 0     # the peer never signals: 30 ms bound
    torch.cuda.synchronize()
    assert int(status) & _lib.DEV_TIMEOUT
    assert torch.equal(x, x0) and float(out.abs().sum()) == 0.0
    # the bit is sticky: the next unsignalled call gives up at once instead of waiting for its own bound (10 s here)
    import time
    t0 = time.perf_counter()
    assert call(lib, x, parts, flags, step, 1, w, out, status, 10000) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0 and torch.equal(x, x0)
    # the context is still usable and a later, signalled call succeeds
    flags[0][1] = 100
    status.zero_()
    assert call(lib, x, parts, flags, step, 1, w, out, status, 1000) == 0
    torch.cuda.synchronize()
    assert int(status) == 0 and not torch.equal(x, x0)


def test_argument_errors():
    from mustafar_b200 import _lib
    lib = _lib.lib()
    x, parts, w, flags = setup()
    pa = (C.c_void_p * 2)(parts[0].data_ptr(), parts[1].data_ptr())
    fa = (C.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    bad = lib.mfar_peer_reduce_add_rmsnorm_f16(x.data_ptr(), pa, fa, 9, 0, None, 0, 4, 0, w.data_ptr(), x.data_ptr(), 5,
                                               1024, 1e-5, 1000, None, None)
    assert bad == 1
    bad = lib.mfar_peer_reduce_add_rmsnorm_f16(x.data_ptr(), pa, fa, 2, 0, None, 0, 4, 4, w.data_ptr(), x.data_ptr(), 5,
                                               1024, 1e-5, 1000, None, None)
    assert bad == 1


def test_peer_block_allocates_zeroed_and_is_viewable_by_torch():
    """mfar_peer_alloc hands out a zeroed cudaMalloc block plus its 64-byte IPC handle; torch views it in place
    (mapping the handle needs a second process: test_gpu_tensor_parallel.py)."""
    from mustafar_b200 import _lib
    from mustafar_b200.peer import _DeviceView
    lib = _lib.lib()
    base, handle = C.c_void_p(), C.create_string_buffer(64)
    assert lib.mfar_peer_alloc(4096, C.byref(base), handle) == 0 and base.value
    assert any(handle.raw)
    t = torch.as_tensor(_DeviceView(base.value, (1024,), "<i4"), device="cuda")
    assert t.data_ptr() == base.value and int(t.abs().sum()) == 0
    t += 3
    assert int(t.sum()) == 3 * 1024
    del t
    torch.cuda.synchronize()
    assert lib.mfar_peer_free(base) == 0
    assert lib.mfar_peer_alloc(0, C.byref(base), handle) == 1          # MFAR_ERR_ARG
    assert lib.mfar_peer_close(None) == 0 and lib.mfar_peer_free(None) == 0


def test_split_vocabulary_argmax_picks_the_global_best_and_the_lowest_index_of_equals():
    """mfar_peer_argmax_f16 as rank 0 of two on one GPU: the "peer" pair buffer is filled by hand and its flag is set
    beforehand.  Rows exercise: best in the local slice, best in the peer's slice, a tie across slices (the lower
    index wins), a tie inside the local slice."""
    from mustafar_b200 import _lib
    lib = _lib.lib()
    rows, n_local, off = 4, 1024, 0
    g = torch.Generator(device="cuda").manual_seed(11)
    logits = torch.randn(rows, n_local, generator=g, device="cuda").half().clamp_(-3, 3)
    logits[0, 700] = 9.0                                   # local best
    logits[1, 5] = 4.0                                     # the peer has 6.0 for this row
    logits[2, 900] = 7.0                                   # tie with the peer's 7.0: index 900 < 1024 + 3
    logits[3, 10] = 8.0
    logits[3, 400] = 8.0                                   # tie inside the slice: 10 wins
    pairs = [torch.zeros(rows, 2, dtype=torch.int32, device="cuda") for _ in range(2)]
    peer_vals = torch.tensor([1.0, 6.0, 7.0, -1.0], dtype=torch.float32)
    pairs[1][:, 0] = peer_vals.view(torch.int32).cuda()
    pairs[1][:, 1] = torch.tensor([1024 + 1, 1024 + 2, 1024 + 3, 1024 + 4], dtype=torch.int32).cuda()
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    flags[0][1] = 5                                        # epoch of (step 0, call 4 of 5)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tokens = torch.full((rows,), -1, dtype=torch.int64, device="cuda")
    pa = (C.c_void_p * 2)(pairs[0].data_ptr(), pairs[1].data_ptr())
    fa = (C.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    st = lib.mfar_peer_argmax_f16(logits.data_ptr(), logits.stride(0), rows, n_local, off, pa, fa, 2, 0, None, 0, 5, 4,
                                  tokens.data_ptr(), int(1e9), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert int(status) == 0
    assert tokens.tolist() == [700, 1024 + 2, 900, 10]
    assert int(flags[1][0]) == 5                           # announced to the "peer"
    # local pairs are what a peer would read
    assert pairs[0][:, 1].tolist() == [700, 5, 900, 10]
    # the peer never announces the next epoch: bounded wait, tokens untouched
    tokens.fill_(-1)
    st = lib.mfar_peer_argmax_f16(logits.data_ptr(), logits.stride(0), rows, n_local, off, pa, fa, 2, 0, None, 1, 5, 4,
                                  tokens.data_ptr(), int(30e6), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert int(status) & _lib.DEV_TIMEOUT and tokens.tolist() == [-1] * rows
