"""Second opinion from the reference's OWN CUDA extensions, compiled for sm_100 into ``oracle/_ref`` by
``python -m oracle.build_ref`` (git-ignored; skipped when absent).

Identical compressed inputs go to the reference's ops and to this library's drop-ins; row 0 of the 8-row outputs must
agree to 2e-3 relative L2 (both accumulate fp16 products in fp32 and round once).  Small shapes only (at most 8 heads
x 1024 tokens).  The fp16 packed buffer gets spare halves at its end because the reference's loader fetches one uint4
past a tile whose count is a multiple of 8 (``kernel/csrc/SpMM_Kernel.cuh:100``).  Of the quantised value kernels only
the 128-row tiling (``value_tile_config=2``) is compared: the 64-row tiling and the ``decode_n1`` prototypes index
tiles in an order the compressor does not emit (``kernel_quant/csrc/SpMM_API_Quant.cu:66,159``) and are never run."""
import pytest
import torch

import oracle
from oracle import build_ref

pytestmark = pytest.mark.gpu
TOL = 2e-3


@pytest.fixture(scope="module")
def m():
    from mustafar_b200 import compression, compression_quant, ops, ops_quant

    class M:
        pass
    M.c, M.cq, M.o, M.oq = compression, compression_quant, ops, ops_quant
    return M


def ref_module(name):
    try:
        mod = build_ref.load(name)
    except ImportError as e:      # built against another torch / python than the one running the tests
        pytest.skip(f"oracle/_ref/{name} does not load here: {e}")
    if mod is None:
        pytest.skip(f"oracle/_ref/{name} was not built (python -m oracle.build_ref)")
    return mod


def call_reference(fn, *args):
    """Host-side refusals of the reference's wrapper (dtype conversions this torch lacks, argument checks) skip the
    comparison; they say nothing about this library."""
    try:
        return fn(*args)
    except (RuntimeError, TypeError) as e:
        if "CUDA error" in str(e):
            raise
        pytest.skip(f"the reference's wrapper refused the call: {str(e).splitlines()[0]}")


def fp16_inputs(m, kind, Bh, L, seed):
    k, v = oracle.make_kv(Bh, L, seed=seed)
    x = oracle.prune_ref(k if kind == "key" else v, 0.7)
    conv = m.c.convert_key_batched if kind == "key" else m.c.convert_value_batched
    bmp, idx, packed = conv(x.cuda())
    nz = torch.cat(packed + [torch.zeros(64, dtype=torch.float16, device="cuda")])   # spare halves for the over-read
    off = torch.zeros(Bh, dtype=torch.int32, device="cuda")
    for i in range(1, Bh):
        off[i] = off[i - 1] + idx[i - 1][-1] // 4
    return x, bmp, nz, idx, off


@pytest.mark.parametrize("G,Bh,L", [(1, 2, 256), (4, 2, 1024)])
def test_fp16_key_op_matches_reference_kernel(m, G, Bh, L):
    ref = ref_module("mustafar_package")
    x, bmp, nz, idx, off = fp16_inputs(m, "key", Bh, L, 501 + L)
    q = oracle.make_query(Bh * G, seed=9).cuda()
    padded = torch.nn.functional.pad(q.view(Bh * G, 1, 128), (0, 0, 0, 7)).contiguous()
    theirs = call_reference(ref.mustafar_key_formulation, bmp, nz, idx, off, padded, L, 128, Bh * G, G)
    ours = m.o.mustafar_key_formulation(bmp, nz, idx, off, padded, L, 128, Bh * G, G)
    torch.cuda.synchronize()
    assert theirs.shape == ours.shape
    assert oracle.rel_l2(ours[:, 0].float().cpu(), theirs[:, 0].float().cpu()) < TOL
    assert oracle.rel_l2(theirs[:, 0].float().cpu(), oracle.key_formulation_ref(x, q.cpu(), G).float()) < TOL


@pytest.mark.parametrize("G,Bh,L", [(1, 2, 256), (4, 2, 1024)])
def test_fp16_value_op_matches_reference_kernel(m, G, Bh, L):
    ref = ref_module("mustafar_package")
    x, bmp, nz, idx, off = fp16_inputs(m, "value", Bh, L, 601 + L)
    g = torch.Generator().manual_seed(3)
    p = torch.softmax(torch.randn(Bh * G, L, generator=g) * 3, dim=-1).half().cuda()
    padded = torch.nn.functional.pad(p.view(Bh * G, 1, L), (0, 0, 0, 7)).contiguous()
    ws = torch.zeros(1, dtype=torch.float16, device="cuda")
    theirs = call_reference(ref.mustafar_value_formulation, bmp, nz, idx, off, padded, ws, 128, L, Bh * G, G)
    ours = m.o.mustafar_value_formulation(bmp, nz, idx, off, padded, ws, 128, L, Bh * G, G)
    torch.cuda.synchronize()
    assert oracle.rel_l2(ours[:, 0].float().cpu(), theirs[:, 0].float().cpu()) < TOL
    assert oracle.rel_l2(theirs[:, 0].float().cpu(), oracle.value_formulation_ref(x, p.cpu(), G).float()) < TOL


def quant_inputs(m, kind, Bh, L, seed):
    k, v = oracle.make_kv(Bh, L, seed=seed)
    x = oracle.prune_ref(k if kind == "key" else v, 0.7)
    if kind == "key":
        return x, m.cq.convert_key_batched_quant(x.cuda(), return_metadata=True)
    return x, m.cq.convert_value_batched_quant(x.cuda())


@pytest.mark.parametrize("G,Bh,L", [(1, 2, 256), (4, 2, 1024)])
def test_quant_key_op_matches_reference_kernel(m, G, Bh, L):
    ref = ref_module("mustafar_package_quant")
    x, (bmp, offs, packed, counts, units, scales, zeros) = quant_inputs(m, "key", Bh, L, 701 + L)
    q = oracle.make_query(Bh * G, seed=10).cuda()
    padded = torch.nn.functional.pad(q.view(Bh * G, 1, 128), (0, 0, 0, 7)).contiguous()
    theirs = call_reference(ref.mustafar_key_formulation_quant, bmp, packed, offs, scales, zeros, padded, L, 128, Bh * G, G, 2, 16, 0)
    ours = m.oq.mustafar_key_formulation_quant(bmp, packed, offs, scales, zeros, padded, L, 128, Bh * G, G, 2, 16, 0)
    meta = call_reference(ref.mustafar_key_formulation_quant_meta, bmp, packed, offs, counts, units, scales, zeros, padded,
                          L, 128, Bh * G, G, 2, 16, 0)
    torch.cuda.synchronize()
    assert oracle.rel_l2(ours[:, 0].float().cpu(), theirs[:, 0].float().cpu()) < TOL
    assert oracle.rel_l2(meta[:, 0].float().cpu(), theirs[:, 0].float().cpu()) < 1e-6


@pytest.mark.parametrize("G,Bh,L", [(1, 2, 256), (4, 2, 1024)])
def test_quant_value_op_matches_reference_kernel(m, G, Bh, L):
    ref = ref_module("mustafar_package_quant")
    x, (bmp, offs, packed, counts, units, scales, zeros) = quant_inputs(m, "value", Bh, L, 801 + L)
    g = torch.Generator().manual_seed(4)
    p = torch.softmax(torch.randn(Bh * G, L, generator=g) * 3, dim=-1).half().cuda()
    padded = torch.nn.functional.pad(p.view(Bh * G, 1, L), (0, 0, 0, 7)).contiguous()
    ws = torch.zeros(1, dtype=torch.float16, device="cuda")
    theirs = call_reference(ref.mustafar_value_formulation_quant, bmp, packed, offs, counts, units, scales, zeros, padded,
                            ws, 128, L, Bh * G, G, 2, 16, 0, 1, 2)
    ours = m.oq.mustafar_value_formulation_quant(bmp, packed, offs, counts, units, scales, zeros, padded, ws, 128, L,
                                                 Bh * G, G, 2, 16, 0, 1, 2)
    torch.cuda.synchronize()
    assert oracle.rel_l2(ours[:, 0].float().cpu(), theirs[:, 0].float().cpu()) < TOL
