"""Fused decode-step glue kernels against the torch expressions they replace (same rounding steps)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rms_ref(x, w, eps):
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope_ref(x, pos, theta):
    half = x.shape[-1] // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, device=x.device, dtype=torch.float32) / half))
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


@pytest.mark.parametrize("rows,hidden", [(1, 256), (32, 4096), (5, 1024)])
def test_add_rmsnorm(rows, hidden):
    from mustafar_b200 import step_ops
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(rows, hidden, generator=g, device="cuda").half()
    d = torch.randn(rows, hidden, generator=g, device="cuda").half()
    w = (1 + 0.1 * torch.randn(hidden, generator=g, device="cuda")).half()
    x0 = x.clone()
    out = step_ops.add_rmsnorm(x, None, w, 1e-5)
    assert torch.equal(x, x0)
    ref = _rms_ref(x0, w, 1e-5)
    # the sum of squares is taken in another order: at most an fp16 ulp on a few elements
    assert (out.float() - ref.float()).abs().max() <= 2e-3 * ref.float().abs().max()
    assert (out != ref).float().mean() < 0.01
    out2 = step_ops.add_rmsnorm(x, d, w, 1e-5)
    assert torch.equal(x, x0 + d)
    ref2 = _rms_ref(x0 + d, w, 1e-5)
    assert (out2 != ref2).float().mean() < 0.01


@pytest.mark.parametrize("dev_state", [False, True])
def test_rope_append(dev_state):
    from mustafar_b200 import step_ops
    B, hq, hkv, cap, theta = 3, 8, 2, 16, 500000.0
    g = torch.Generator(device="cuda").manual_seed(2)
    qkv = torch.randn(B, (hq + 2 * hkv) * 128, generator=g, device="cuda").half()
    kwin = torch.zeros(B * hkv, cap, 128, dtype=torch.float16, device="cuda")
    vwin = torch.zeros_like(kwin)
    q_out = torch.empty(B * hq, 128, dtype=torch.float16, device="cuda")
    pos, slot = 4321, 7
    inv = step_ops.rope_inv_freq(theta, "cuda")
    if dev_state:
        st = torch.tensor([pos, slot], dtype=torch.int32, device="cuda")
        step_ops.rope_append(qkv, inv, st[0:1], st[1:2], hq, hkv, q_out, kwin, vwin)
    else:
        step_ops.rope_append(qkv, inv, pos, slot, hq, hkv, q_out, kwin, vwin)
    q, k, v = qkv.split([hq * 128, hkv * 128, hkv * 128], dim=-1)
    p = torch.tensor([pos], device="cuda")
    q_ref = _rope_ref(q.view(B, 1, hq, 128).transpose(1, 2), p, theta).reshape(B * hq, 128)
    k_ref = _rope_ref(k.view(B, 1, hkv, 128).transpose(1, 2), p, theta).reshape(B * hkv, 128)
    # cosf / sinf may differ from torch's by an fp32 ulp, which shows after rounding on a few elements only
    for got, ref in ((q_out, q_ref), (kwin[:, slot], k_ref)):
        assert (got != ref).float().mean() < 0.01
        assert (got.float() - ref.float()).abs().max() < 1e-2
    assert torch.equal(vwin[:, slot], v.reshape(B * hkv, 128))
    mask = torch.ones(cap, dtype=torch.bool)
    mask[slot] = False
    assert kwin[:, mask].abs().sum() == 0 and vwin[:, mask].abs().sum() == 0


def test_rope_append_slot_outside_window_is_reported_not_written():
    """A device-resident slot equal to the window capacity (host and device counters out of step) must leave the
    windows untouched and set the status bit; the query is still produced."""
    from mustafar_b200 import ops, step_ops
    B, hq, hkv, cap = 2, 4, 2, 8
    g = torch.Generator(device="cuda").manual_seed(4)
    qkv = torch.randn(B, (hq + 2 * hkv) * 128, generator=g, device="cuda").half()
    guard = torch.zeros(B * hkv + 1, cap, 128, dtype=torch.float16, device="cuda")   # one spare head behind the window
    kwin, vwin = guard[:B * hkv], torch.zeros(B * hkv, cap, 128, dtype=torch.float16, device="cuda")
    q_out = torch.zeros(B * hq, 128, dtype=torch.float16, device="cuda")
    st = torch.tensor([5, cap], dtype=torch.int32, device="cuda")
    ops.check_device_status()
    step_ops.rope_append(qkv, step_ops.rope_inv_freq(500000.0, "cuda"), st[0:1], st[1:2], hq, hkv, q_out, kwin, vwin)
    with pytest.raises(RuntimeError):
        ops.check_device_status()
    assert guard.abs().sum() == 0 and vwin.abs().sum() == 0
    assert q_out.abs().sum() > 0
    with pytest.raises(RuntimeError):      # a host-side slot is refused before the launch
        step_ops.rope_append(qkv, step_ops.rope_inv_freq(500000.0, "cuda"), 5, cap, hq, hkv, q_out, kwin, vwin)


def test_per_step_prune_builds_the_same_cache_as_block_mode():
    """Feeding the same K / V stream token by token with per-step pruning (prune inside the append launch, then
    compression of already pruned rows with prune_rank = 0) gives bit for bit the cache of block mode (dense window,
    prune fused into the compression of the oldest 256 tokens)."""
    from mustafar_b200 import compression as comp, ops, step_ops
    B, hq, hkv, residual, rank = 2, 4, 2, 128, comp.keep_rank(0.7)
    cap = residual + 256
    Bh = B * hkv
    g = torch.Generator(device="cuda").manual_seed(8)
    inv = step_ops.rope_inv_freq(500000.0, "cuda")
    stores = {}
    for mode in ("block", "step"):
        ks, vs = comp.SparseStore(Bh, 512, comp.KEY, "cuda"), comp.SparseStore(Bh, 512, comp.VALUE, "cuda")
        kwin = torch.zeros(Bh, cap, 128, dtype=torch.float16, device="cuda")
        vwin = torch.zeros_like(kwin)
        q_out = torch.empty(B * hq, 128, dtype=torch.float16, device="cuda")
        g.manual_seed(8)
        w = 0
        for t in range(2 * cap - residual):
            qkv = torch.randn(B, (hq + 2 * hkv) * 128, generator=g, device="cuda").half()
            extra = dict(prune_rank=rank, prune_back=residual) if mode == "step" else {}
            step_ops.rope_append(qkv, inv, 0, w, hq, hkv, q_out, kwin, vwin, **extra)   # position 0: K is not rotated
            w += 1
            if w == cap:
                r = rank
                if mode == "step":
                    kwin[:, 255] = comp.prune(kwin[:, 255].contiguous(), 0.7)
                    vwin[:, 255] = comp.prune(vwin[:, 255].contiguous(), 0.7)
                    r = 0
                ks.append(kwin[:, :256], r)
                vs.append(vwin[:, :256], r)
                kwin[:, :residual] = kwin[:, 256:].clone()
                vwin[:, :residual] = vwin[:, 256:].clone()
                w = residual
        ks.check(); vs.check()
        stores[mode] = (ks, vs)
    ops.check_device_status()
    for a, b in zip(stores["block"], stores["step"]):
        assert a.tokens == b.tokens == 512
        assert torch.equal(a.bitmaps, b.bitmaps) and torch.equal(a.accum, b.accum)
        for h, n in enumerate(a.packed_lengths().tolist()):
            assert torch.equal(a.nz[h, :n].view(torch.int16), b.nz[h, :n].view(torch.int16)), h


def test_silu_mul():
    from mustafar_b200 import step_ops
    g = torch.Generator(device="cuda").manual_seed(3)
    gu = (3 * torch.randn(7, 2 * 1434, generator=g, device="cuda")).half()
    out = step_ops.silu_mul(gu)
    ref = torch.nn.functional.silu(gu[:, :1434]) * gu[:, 1434:]
    assert (out != ref).float().mean() < 0.01
    assert (out.float() - ref.float()).abs().max() <= 2e-3 * ref.float().abs().max()


def test_argument_errors():
    from mustafar_b200 import step_ops
    x = torch.zeros(2, 100, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        step_ops.add_rmsnorm(x, None, torch.ones(100, dtype=torch.float16, device="cuda"), 1e-5)   # hidden % 8
    with pytest.raises(RuntimeError):
        step_ops.add_rmsnorm(x.float(), None, torch.ones(100, dtype=torch.float16, device="cuda"), 1e-5)
