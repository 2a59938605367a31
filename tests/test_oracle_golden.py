"""The CPU oracle against fixtures produced by the reference's own Triton kernels
(run under the Triton interpreter by tests/golden/make_golden.py) and by the
reference's own dh_prune_key.  Bit-exact: integer / byte / index work."""
import os

import numpy as np
import pytest
import torch

import oracle
from oracle.prune import prune_np

G = os.path.join(os.path.dirname(__file__), "golden")
F16 = np.load(os.path.join(G, "fp16_cases.npz"))
QNT = np.load(os.path.join(G, "quant_cases.npz"))
PRN = np.load(os.path.join(G, "prune_cases.npz"))
CASES = sorted({k.split("/")[0] for k in F16.files})


def bits16(a):
    return np.ascontiguousarray(a).view(np.uint16)


def test_case_inventory():
    assert len(CASES) >= 20


@pytest.mark.parametrize("s", [0, 10, 50, 70, 90, 99])
def test_prune_matches_reference(s):
    raw = torch.from_numpy(PRN["raw"])
    want = PRN[f"s{s}"]
    got = oracle.prune_ref(raw, s / 100.0).numpy()
    assert np.array_equal(bits16(got), bits16(want))        # includes the sign of pruned zeros
    assert np.array_equal(bits16(prune_np(PRN["raw"], s / 100.0)), bits16(want))


@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("kind", ["key", "value"])
def test_fp16_format_matches_reference(name, kind):
    x = F16[f"{name}/x"]
    fn = oracle.compress_key_ref if kind == "key" else oracle.compress_value_ref
    bitmaps, accum, packed = fn(x)
    assert np.array_equal(bitmaps, F16[f"{name}/{kind}/bitmaps"])
    assert np.array_equal(accum, F16[f"{name}/{kind}/accum"])
    flat = np.concatenate(packed) if packed else np.zeros(0, np.float16)
    assert np.array_equal(bits16(flat), bits16(F16[f"{name}/{kind}/packed_flat"]))
    starts = F16[f"{name}/{kind}/starts"]
    assert np.array_equal(oracle.nz_offsets_ref(accum).astype(np.int64) * 8, starts)
    # round trip
    L = x.shape[1]
    de = oracle.decompress_key_ref if kind == "key" else oracle.decompress_value_ref
    back = de(bitmaps, accum, packed, L)
    assert np.array_equal(back, np.where(x == 0, np.float16(0), x))


@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("kind", ["key", "value"])
def test_quant_format_matches_reference(name, kind):
    x = QNT[f"{name}/x"]
    fn = oracle.quant_compress_key_ref if kind == "key" else oracle.quant_compress_value_ref
    got = fn(x, bits=2, group=64)
    for key in ("bitmaps", "tile_offsets", "counts", "units", "packed"):
        assert np.array_equal(got[key], QNT[f"{name}/{kind}/{key}"]), key
    for key in ("scales", "zeros"):
        assert np.array_equal(bits16(got[key]), bits16(QNT[f"{name}/{kind}/{key}"])), key
