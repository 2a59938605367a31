#!/usr/bin/env python
"""Generate the golden fixtures in this directory FROM THE REFERENCE ITSELF.

Run once, in a container that has the reference checkout (it is not needed at
test time):

    python tests/golden/make_golden.py --reference /path/to/mustafar

What it runs:

* the reference's ``@triton.jit`` compression kernels (``kernel/compression.py``
  and ``kernel_quant/compression_quant.py``) under ``TRITON_INTERPRET=1``.  The
  reference's host wrappers insist on CUDA tensors, so the few lines of host
  arithmetic between the two kernel launches (prefix sums, buffer allocation)
  are redone here on CPU tensors; every bitmap / count / scale / code in the
  fixtures is produced by the reference's own kernels;
* the reference's ``dh_prune_key`` (``models/llama_mustafar_kernel.py:194-232``),
  extracted from the source with ``ast`` and executed unmodified (the module as
  a whole does not import under newer ``transformers``).

Output: ``fp16_cases.npz``, ``quant_cases.npz``, ``prune_cases.npz``.
"""
from __future__ import annotations

import argparse
import ast
import importlib.util
import os
import sys
import textwrap

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _ref_prune(ref_root):
    src = open(os.path.join(ref_root, "models", "llama_mustafar_kernel.py")).read()
    tree = ast.parse(src)
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == "dh_prune_key":
            code = textwrap.dedent(ast.get_source_segment(src, node))
            ns = {"torch": torch}
            exec(compile(code, "dh_prune_key", "exec"), ns)
            return ns["dh_prune_key"]
    raise RuntimeError("dh_prune_key not found")


_SHIFTS = torch.tensor(np.left_shift(np.int64(1), np.arange(63, -1, -1, dtype=np.int64)))


def run_fp16(mod, x: torch.Tensor, kind: str):
    Bh, L, D = x.shape
    T = L * D // 64
    src = (x.transpose(1, 2) if kind == "key" else x).contiguous().view(-1)
    bitmaps = torch.empty((Bh, T), dtype=torch.int64)
    counts = torch.empty((Bh, T), dtype=torch.int32)
    k1 = getattr(mod, f"calculate_bitmap_{kind}_batched")
    k2 = getattr(mod, f"compress_{kind}_batched")
    k1[(T, Bh)](src, bitmaps.view(-1), counts.view(-1), total_elems=Bh * L * D,
                shifts_ptr=_SHIFTS, stride_batch=T * 64, M=L, N=D)
    accum = torch.zeros((Bh, T + 1), dtype=torch.int32)
    accum[:, 1:] = torch.cumsum(counts, dim=1)
    halves = 2 * accum[:, -1].to(torch.int64)
    ends = torch.cumsum(halves, dim=0)
    starts = ends - halves
    flat = torch.zeros(int(ends[-1]), dtype=torch.float16)
    k2[(T, Bh)](src, bitmaps.view(-1), accum.view(-1), flat, starts.to(torch.int32),
                total_elems=Bh * L * D, stride_batch=T * 64, M=L, N=D)
    return bitmaps.numpy(), accum.numpy(), flat.numpy(), starts.numpy().astype(np.int64)


def run_quant(mod, x: torch.Tensor, kind: str):
    Bh, L, D = x.shape
    T = L * D // 64
    src = (x.transpose(1, 2) if kind == "key" else x).contiguous().view(-1)
    bitmaps = torch.empty((Bh, T), dtype=torch.int64)
    counts = torch.empty((Bh, T), dtype=torch.int32)
    scales = torch.empty((Bh, T), dtype=torch.float16)
    zeros = torch.empty((Bh, T), dtype=torch.float16)
    k1 = getattr(mod, f"calculate_bitmap_and_scale_{kind}_batched")
    k2 = getattr(mod, f"compress_{kind}_batched")
    k1[(T, Bh)](src, bitmaps.view(-1), counts.view(-1), scales.view(-1), zeros.view(-1),
                total_elems=Bh * L * D, shifts_ptr=_SHIFTS, stride_batch=T * 64, M=L, N=D)
    units = (counts + 15) // 16
    flat_units = units.view(-1).to(torch.int64)
    offs = torch.cumsum(flat_units, dim=0) - flat_units
    tile_offsets = offs.view(Bh, T).to(torch.int32)
    packed = torch.zeros(int(flat_units.sum()), dtype=torch.int32)
    if packed.numel():
        k2[(T, Bh)](src, bitmaps.view(-1), counts.view(-1), tile_offsets.view(-1), packed,
                    scales.view(-1), zeros.view(-1), 2, 16,
                    total_elems=Bh * L * D, stride_batch=T * 64, M=L, N=D)
    return dict(bitmaps=bitmaps.numpy(), tile_offsets=tile_offsets.numpy(), packed=packed.numpy(),
                counts=counts.numpy(), units=units.numpy().astype(np.int32),
                scales=scales.numpy(), zeros=zeros.numpy())


def cases(prune):
    """Seeded inputs [Bh, L, 128] fp16, already pruned the way the model prunes."""
    out = {}

    def add(name, x):
        out[name] = x.contiguous()

    def randn(seed, Bh, L, scale_outliers=True):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(Bh, L, 128, generator=g)
        if scale_outliers:
            for h in range(Bh):
                x[h, :, torch.randperm(128, generator=g)[:4]] *= 10.0
        return x.half()

    def pr(x, s):
        return prune(None, x.unsqueeze(0), s).squeeze(0)

    i = 0
    for Bh, L in [(1, 64), (2, 64), (3, 64), (2, 128), (1, 192), (2, 256)]:
        for s in (0.5, 0.7):
            add(f"randn_b{Bh}_l{L}_s{int(s * 100)}", pr(randn(1000 + i, Bh, L), s))
            i += 1
    # heavy ties: values on a coarse grid
    g = torch.Generator().manual_seed(77)
    x = (torch.randint(-4, 5, (2, 64, 128), generator=g).float() / 4).half()
    add("ties_grid_s70", pr(x, 0.7))
    add("ties_grid_s50", pr(x, 0.5))
    # unpruned dense block (every tile full), all-zero block, single nonzero per row
    add("dense_unpruned", randn(5, 1, 64, False))
    add("all_zero", torch.zeros(1, 64, 128, dtype=torch.float16))
    x = torch.zeros(2, 64, 128, dtype=torch.float16)
    x[:, torch.arange(64), (torch.arange(64) * 7) % 128] = 1.5
    add("one_per_row", x)
    # rows of equal magnitude (all kept), rows with zeros and negative zeros, mixed sparsity
    x = torch.ones(1, 64, 128, dtype=torch.float16)
    x[:, :, ::2] = -1
    add("equal_magnitude_s70", pr(x, 0.7))
    x = randn(9, 2, 128)
    x[0, :32] = 0
    x[1, 64:, 64:] = 0
    add("zero_rows_s70", pr(x, 0.7))
    add("sparsity_90", pr(randn(10, 2, 64), 0.9))
    add("sparsity_10", pr(randn(11, 1, 64), 0.1))
    # counts exactly multiples of 8 / 16 in some tiles: block-structured masks
    x = randn(12, 1, 128, False)
    m = torch.zeros(128, 128)
    m[:8, :] = 1
    m[64:80, :] = 1
    m[:, 5] = 1
    add("mult8_tiles", (x * m).half())
    # tiny dynamic range tiles (scale underflow paths of the quantiser) and constant tiles
    x = torch.full((1, 64, 128), 0.25, dtype=torch.float16)
    x[:, :, 64:] = randn(13, 1, 64, False)[:, :, 64:] * 1e-3
    add("const_and_tiny", pr(x, 0.5))
    x = randn(14, 1, 64, False) * 200
    add("large_values_s70", pr(x.half(), 0.7))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (Haozon/mustafar)")
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    comp = _load(os.path.join(a.reference, "kernel", "compression.py"), "ref_compression")
    compq = _load(os.path.join(a.reference, "kernel_quant", "compression_quant.py"), "ref_compression_quant")
    prune = _ref_prune(a.reference)

    # --- prune fixtures: raw input -> reference output, several sparsities
    pc = {}
    g = torch.Generator().manual_seed(4242)
    raw = torch.randn(1, 2, 96, 128, generator=g)
    raw[:, :, :, [3, 40, 77, 120]] *= 10
    raw = raw.half()
    raw[0, 0, 0] = 0                      # all-zero row
    raw[0, 0, 1] = 1.0                    # all-equal row
    raw[0, 0, 2, :64] = 0                 # half zeros
    raw[0, 0, 3] = (torch.arange(128) % 5).half()   # many ties
    raw[0, 0, 4, ::2] *= -1
    pc["raw"] = raw.numpy()
    for s in (0.0, 0.1, 0.5, 0.7, 0.9, 0.99):
        pc[f"s{int(s * 100)}"] = prune(None, raw, s).numpy()
    np.savez_compressed(os.path.join(HERE, "prune_cases.npz"), **pc)
    print("prune cases:", len(pc) - 1)

    cs = cases(prune)
    f16, q = {}, {}
    for name, x in cs.items():
        f16[f"{name}/x"] = x.numpy()
        q[f"{name}/x"] = x.numpy()
        for kind in ("key", "value"):
            b, acc, flat, starts = run_fp16(comp, x, kind)
            f16[f"{name}/{kind}/bitmaps"] = b
            f16[f"{name}/{kind}/accum"] = acc
            f16[f"{name}/{kind}/packed_flat"] = flat
            f16[f"{name}/{kind}/starts"] = starts
            for k2, v2 in run_quant(compq, x, kind).items():
                q[f"{name}/{kind}/{k2}"] = v2
        print("done", name, tuple(x.shape))
    np.savez_compressed(os.path.join(HERE, "fp16_cases.npz"), **f16)
    np.savez_compressed(os.path.join(HERE, "quant_cases.npz"), **q)


if __name__ == "__main__":
    main()
