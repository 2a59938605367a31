"""Wire format of a compressed cache: round trip on CPU tensors built from the oracle's compression,
and rejection of damaged blobs."""
import numpy as np
import pytest
import torch

import oracle
from mustafar_b200 import wire
from mustafar_b200.compression import KEY, VALUE, SparseStore


def _store_from_oracle(kind, n_heads=3, tokens=128, seed=5):
    g = torch.Generator().manual_seed(seed)
    x = oracle.prune.prune_ref(torch.randn(n_heads, tokens, 128, generator=g).half(), 0.7)
    fn = oracle.fp16_format.compress_key_ref if kind == KEY else oracle.fp16_format.compress_value_ref
    bitmaps, accum, packed = fn(x)
    packed = [torch.from_numpy(pk) for pk in packed]
    st = SparseStore(n_heads, tokens, kind, "cpu", nz_capacity=max(int(p.numel()) for p in packed))
    T = 2 * tokens
    st.bitmaps[:, :T] = torch.from_numpy(bitmaps)
    st.accum[:, :T + 1] = torch.from_numpy(accum)
    for h, pk in enumerate(packed):
        st.nz[h, :pk.numel()] = pk
    st.tokens = tokens
    return st, packed


@pytest.mark.parametrize("kind", [KEY, VALUE])
def test_round_trip(kind):
    st, packed = _store_from_oracle(kind)
    blob = wire.pack_store(st)
    assert blob.dtype == torch.uint8 and blob.numel() % 16 == 0
    back = wire.unpack_store(blob, "cpu", max_tokens=256)
    T = st.tiles
    assert back.kind == kind and back.tokens == st.tokens and back.max_tokens == 256
    assert torch.equal(back.bitmaps[:, :T], st.bitmaps[:, :T])
    assert torch.equal(back.accum[:, :T + 1], st.accum[:, :T + 1])
    for h, pk in enumerate(packed):
        assert torch.equal(back.nz[h, :pk.numel()], pk)
    # a second trip through the format is byte-identical
    assert torch.equal(wire.pack_store(back), blob)


def test_empty_store():
    st = SparseStore(2, 64, KEY, "cpu")
    back = wire.unpack_store(wire.pack_store(st), "cpu")
    assert back.tokens == 0 and back.n_heads == 2


def test_damaged_blobs_are_rejected():
    st, _ = _store_from_oracle(VALUE)
    blob = wire.pack_store(st)
    bad = blob.clone()
    bad[0] = 0
    with pytest.raises(ValueError):
        wire.unpack_store(bad, "cpu")
    with pytest.raises(ValueError):
        wire.unpack_store(blob[:100], "cpu")
    with pytest.raises(ValueError):
        wire.unpack_store(blob[:-16], "cpu")
    bad = blob.clone()
    bad[wire.HEADER_BYTES:wire.HEADER_BYTES + 8] = 0xff   # first tile claims 64 values: no longer what accum says
    with pytest.raises(ValueError):
        wire.unpack_store(bad, "cpu")
    with pytest.raises(ValueError):
        wire.unpack_store(blob, "cpu", max_tokens=64)
