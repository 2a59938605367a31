"""The allocation-free compression entry point (for hosts that may not call cudaMalloc while
running, e.g. a server that owns all device memory through its own arena) must write exactly what
the regular entry point writes.  Called straight through the C ABI, twice in a row with different
inputs, because both calls share one scratch array inside the library and the second must not be
disturbed by what the first left there."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(lib, x, kind, rank, entry):
    Bh, L, _ = x.shape
    T = 2 * L
    bitmaps = torch.zeros((Bh, T), dtype=torch.int64, device="cuda")
    accum = torch.zeros((Bh, T + 1), dtype=torch.int32, device="cuda")
    nz = torch.zeros((Bh, L * 128), dtype=torch.float16, device="cuda")
    stats = torch.zeros(2, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    src = (x.data_ptr(), x.stride(0), x.stride(1))
    dst = (Bh, L, kind, rank, bitmaps.data_ptr(), T, accum.data_ptr(), T + 1, 0, nz.data_ptr(), None, L * 128, L * 128)
    if entry == "noalloc":
        st = lib.mfar_compress_fp16_noalloc(*src, *dst, stats.data_ptr(), stats.data_ptr() + 4, stream)
    else:
        need = lib.mfar_compress_scratch_bytes(Bh, L)
        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
        st = lib.mfar_compress_fp16(*src, 0, 0, *dst, scratch.data_ptr(), need, stats.data_ptr(), stats.data_ptr() + 4,
                                    stream)
    torch.cuda.synchronize()
    assert st == 0, st
    return bitmaps, accum, nz.view(torch.int16), stats


def test_noalloc_entry_matches_regular_entry_twice():
    from mustafar_b200 import _lib
    lib = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(11)
    shapes = [((6, 1024, 128), 0, 89), ((3, 448, 128), 1, 64)]     # (shape, kind, prune rank); two calls in a row
    for shape, kind, rank in shapes:
        x = torch.randn(shape, generator=g, device="cuda").half()
        want = _run(lib, x, kind, rank, "regular")
        got = _run(lib, x, kind, rank, "noalloc")
        for a, b in zip(got, want):
            assert torch.equal(a, b)
        assert int(got[3][0]) == 0


def test_noalloc_entry_rejects_jobs_beyond_its_limit():
    from mustafar_b200 import _lib
    lib = _lib.lib()
    # 129 heads x 4096 tokens = 8256 blocks > MFAR_NOALLOC_MAX_BLOCKS (8192): refused before any launch
    st = lib.mfar_compress_fp16_noalloc(None, 0, 0, 129, 4096, 0, 0, None, 0, None, 0, 0, None, None, 0, 0, None, None, None)
    assert st == 6
    assert b"limit" in lib.mfar_status_string(st)
