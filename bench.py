#!/usr/bin/env python
"""Benchmark of the sparse KV-cache decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--batch B] [--kv-len L] [--window W] [--sparsity S]

One "step" = one decode-attention layer pass (q.K^T over the compressed cache + dense
window, softmax, P.V) for a batch of B sequences with the Llama-3-8B head shape
(32 query heads, 8 kv heads, head_dim 128).  Default workload = batched decode sparse attention
at its largest point (B=64, L=32768, window 128, 70 % sparsity); inputs are seeded synthetic
tensors (K, V ~ N(0,1), four K outlier channels x10).  After the timed region the step's output
is checked, for a sample of kv heads, against the CPU oracle fed with those heads' slices of the
very cache that was timed ("parity_check"; a failure makes the run exit non-zero).

Prints ONE JSON line (rank 0).  `value` = sequences * steps / device time, i.e. decode
tokens per second through one attention layer, whole job over all ranks (batch-sharded
replicas, no collective on the data path, weak scaling).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HQ, HKV, D = 32, 8, 128
G = HQ // HKV


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--kv-len", type=int, default=32768)
    ap.add_argument("--window", type=int, default=128)
    ap.add_argument("--sparsity", type=float, default=0.7)
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="budget of the CPU baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parity-heads", type=int, default=4, help="kv heads checked against the CPU oracle after timing")
    ap.add_argument("--no-e2e-llama", action="store_true",
                    help="skip the end-to-end Llama-3-8B-shape generation reported under \"e2e_llama\"")
    ap.add_argument("--e2e-llama-new", type=int, default=256, help="generated tokens of the end-to-end run")
    ap.add_argument("--no-other-configs", action="store_true",
                    help="skip the short measurements of the other workloads reported under \"other_configs\"")
    return ap.parse_args()


def other_configs():
    """Short timings of the remaining workloads through the same library (mustafar_b200/kernel_bench.py runs them)."""
    from mustafar_b200 import kernel_bench as kb
    peak, _ = measured_peak_gbs()
    rows = []

    def collect(name, us, nbytes, **kw):
        rows.append({"kernel": name, "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1),
                     "frac_of_hbm_peak": round(nbytes / us / 1e3 / peak, 3), **kw})
    emit, kb.emit = kb.emit, collect
    try:
        kb.bench_compress_fp16(False, iters=10, warmup=3)
        kb.bench_quant(False, 32, 16384, (2,), (0.7,), (64,))
        kb.bench_step(False)
    finally:
        kb.emit = emit
        torch.cuda.empty_cache()
    return rows


# ------------------------------------------------------------------------------------------ peaks / clocks
def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.03)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------ workload
def build_cache(batch, kv_len, window, sparsity, device, seed):
    """Seeded synthetic cache: K, V ~ N(0,1), 4 outlier channels x10 per kv head in K, pruned
    per token by magnitude inside the compression kernel.  Built in token chunks to bound memory."""
    from mustafar_b200 import compression as comp
    Bh = batch * HKV
    gen = torch.Generator(device=device).manual_seed(seed)
    cap = int(kv_len * D * min(1.0, (1.0 - sparsity) + 0.25)) // 8 * 8
    ks = comp.SparseStore(Bh, kv_len, comp.KEY, device, nz_capacity=cap)
    vs = comp.SparseStore(Bh, kv_len, comp.VALUE, device, nz_capacity=cap)
    out_ch = torch.stack([torch.randperm(D, generator=gen, device=device)[:4] for _ in range(Bh)])
    scale = torch.ones(Bh, 1, D, device=device)
    scale.scatter_(2, out_ch[:, None, :], 10.0)
    rank = comp.keep_rank(sparsity)
    chunk = max(256, min(kv_len, (1 << 28) // (Bh * D) // 256 * 256))
    for t0 in range(0, kv_len, chunk):
        n = min(chunk, kv_len - t0)
        k = (torch.randn(Bh, n, D, generator=gen, device=device) * scale).half()
        ks.append(k, rank)
        v = torch.randn(Bh, n, D, generator=gen, device=device).half()
        vs.append(v, rank)
        del k, v
    kw = (torch.randn(Bh, window, D, generator=gen, device=device) * scale).half()
    vw = torch.randn(Bh, window, D, generator=gen, device=device).half()
    ks.check(); vs.check()
    return ks, vs, kw, vw


def algorithmic_bytes(ks, vs, window, batch):
    """Bytes one decode-attention launch has to move: per tensor the bitmaps (8 B/tile), the
    offsets (4 B/tile + 4 B/head) and the packed values actually stored (from the accum tails),
    each kv head once; plus the dense window, q and the output."""
    Bh = batch * HKV
    total = 0
    for st in (ks, vs):
        n_tiles = Bh * st.tiles
        packed_halves = int(st.packed_lengths().sum().item())
        total += 8 * n_tiles + 4 * (n_tiles + Bh) + 2 * packed_halves
    total += 2 * (2 * Bh * window * D) + 2 * (2 * batch * HQ * D)
    return total


def traffic_estimate(alg_bytes):
    """DRAM traffic of one launch: the read + written bytes per algorithmic byte that ncu measured on a smaller
    case of the same kernel (traffic grows with the tokens read), times this launch's algorithmic bytes."""
    p = os.path.join(ROOT, "profiles", "decode_attn_traffic.txt")
    try:
        d = dict(line.split(":", 1) for line in open(p) if ":" in line and not line.startswith("#"))
        return alg_bytes * float(d["dram_bytes"]) / float(d["algorithmic_bytes"])
    except Exception:
        return None


def parity_check(q, out, ks, vs, kw, vw, n_heads, tol=2e-3):
    """Checks the timed configuration itself: for a sample of kv heads, their slices of the compressed cache are
    copied to the host, decompressed by the oracle, and the oracle's fp32 attention over [decompressed ; window]
    is compared with the kernel's output for the G query heads of each sampled kv head."""
    import oracle
    Bh, L = ks.n_heads, ks.tokens
    n_heads = max(1, min(n_heads, Bh))
    heads = sorted({int(round(i * (Bh - 1) / max(1, n_heads - 1))) for i in range(n_heads)})
    T = ks.tiles
    worst = 0.0
    for h in heads:
        dense = []
        for st, fn in ((ks, oracle.decompress_key_ref), (vs, oracle.decompress_value_ref)):
            bmp = st.bitmaps[h:h + 1, :T].cpu().numpy()
            acc = st.accum[h:h + 1, :T + 1].cpu().numpy()
            n = 2 * int(acc[0, -1])
            packed = [st.nz[h, :n].cpu().numpy()]
            dense.append(torch.from_numpy(fn(bmp, acc, packed, L)))
        want = oracle.decode_attention_ref(q[h * G:(h + 1) * G].cpu(), dense[0], dense[1], kw[h:h + 1].cpu(), vw[h:h + 1].cpu(), G)
        worst = max(worst, oracle.rel_l2(out[h * G:(h + 1) * G].float().cpu(), want))
    return {"heads": len(heads), "kv_heads_checked": heads, "rel_l2": worst, "tol": tol, "ok": bool(worst < tol),
            "against": "oracle.decode_attention_ref on the oracle-decompressed cache slices of the sampled heads"}


# ------------------------------------------------------------------------------------------ CPU baseline
def cpu_baseline(kv_len, window, sparsity, budget_s, steps=None, warmup=3):
    """The reference's torch path on the host cores (oracle port): dense
    softmax(q.K~^T / sqrt(d)).V~ on the pruned tensors for ONE sequence (8 kv heads,
    32 q heads) of the same length; K~/V~ held in fp32 so the step is pure attention."""
    import oracle
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    k, v = oracle.make_kv(HKV, kv_len + window, seed=oracle.synth.BASE_SEED)
    kc = oracle.prune_ref(k[:, :kv_len].contiguous(), sparsity).float()
    vc = oracle.prune_ref(v[:, :kv_len].contiguous(), sparsity).float()
    kk = torch.cat([kc, k[:, kv_len:].float()], dim=1).repeat_interleave(G, dim=0)
    vv = torch.cat([vc, v[:, kv_len:].float()], dim=1).repeat_interleave(G, dim=0)
    q = oracle.make_query(HQ).float()

    def step():
        s = torch.bmm(kk, q.unsqueeze(-1)).squeeze(-1) / math.sqrt(D)
        p = torch.softmax(s, dim=-1)
        return torch.bmm(p.unsqueeze(1), vv).squeeze(1)

    for _ in range(max(1, warmup)):
        step()
    times, t_end = [], time.perf_counter() + budget_s
    if steps is not None:                      # reference arm: exactly `steps` timed steps
        for _ in range(steps):
            t0 = time.perf_counter()
            step()
            times.append(time.perf_counter() - t0)
    while steps is None and (len(times) < 10 or (time.perf_counter() < t_end and len(times) < 200)):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() > t_end and len(times) >= 10:
            break
    times.sort()
    med = times[len(times) // 2]
    return {"value": 1.0 / med, "unit": "tok/s/layer", "cores": threads, "kind": "port",
            "sample": f"1 sequence (8 kv heads, 32 q heads) of kv_len {kv_len}+{window}, dense fp32 attention on the "
                      f"pruned tensors, median of {len(times)} steps", "ms_per_step": med * 1e3}


# ------------------------------------------------------------------------------------------ main
def main():
    a = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    workload = f"decode-attn B={a.batch} Hq={HQ} Hkv={HKV} D={D} L={a.kv_len} W={a.window} sparsity={a.sparsity}"
    config = {"workload": workload, "batch_per_gpu": a.batch, "kv_len": a.kv_len, "window": a.window,
              "sparsity": a.sparsity, "sharding": "batch-sharded replicas, no data-path collective",
              "l2": "inputs larger than L2 (126 MB)"}

    if a.impl == "reference":
        if rank != 0:
            return
        cb = cpu_baseline(a.kv_len, a.window, a.sparsity, a.cpu_seconds, steps=a.steps, warmup=a.warmup)
        line = {"impl": "reference", "metric": "sparse_decode_attention_throughput", "value": cb["value"],
                "unit": "tok/s/layer", "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
                "ms_per_step": cb["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "tok/s/layer", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        # NCCL carries only barriers, scalar reductions and (in the NCCL arm) 256 KiB all-reduces here: in-switch
        # reduction buys nothing, and without multicast objects a rank that dies cannot disturb its peers' GPUs
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)

    from mustafar_b200 import ops

    ks, vs, kw, vw = build_cache(a.batch, a.kv_len, a.window, a.sparsity, dev, 20260302 + 9973 * 2 + rank)
    Bq = a.batch * HQ
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    q = torch.randn(Bq, D, generator=gen, device=dev).half()
    out = torch.empty(Bq, D, dtype=torch.float16, device=dev)
    hint = max(ks.stage_hint(), vs.stage_hint())
    alg_bytes = algorithmic_bytes(ks, vs, a.window, a.batch)
    _, ws_bytes = ops.plan(a.batch * HKV, a.kv_len, a.window, G)
    ws = ops.new_workspace(dev, ws_bytes)

    def step():
        ops.decode_attention(q, ks, vs, kw, vw, G, out=out, stage_halves=hint, workspace=ws)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    ev = [torch.cuda.Event(enable_timing=True) for _ in range(a.steps + 1)]
    with ClockSampler(local) as clocks:
        for _ in range(max(a.warmup, 3)):
            step()
        # nvidia-smi takes a while to deliver its first line (longer with eight of them starting at once) and the
        # timed region is only tens of milliseconds: keep the GPU under the same load, untimed, until samples arrive
        t_wait = time.time()
        while len(clocks.rows) < 2 and time.time() - t_wait < 4.0:
            step()
            torch.cuda.synchronize()
        ops.check_device_status(dev)
        barrier()
        ev[0].record()
        for i in range(a.steps):
            step()
            ev[i + 1].record()
        torch.cuda.synchronize()
    total_ms = ev[0].elapsed_time(ev[-1])
    step_ms = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(a.steps))
    per_launch_ms = sum(step_ms) / a.steps
    barrier()
    parity = parity_check(q, out, ks, vs, kw, vw, a.parity_heads) if rank == 0 else None

    # end to end through the public API with host buffers: q from pinned memory, result back to the host
    q_host = q.cpu().pin_memory()
    out_host = torch.empty_like(out, device="cpu").pin_memory()
    q_dev = torch.empty_like(q)

    def e2e_step():
        q_dev.copy_(q_host, non_blocking=True)
        ops.decode_attention(q_dev, ks, vs, kw, vw, G, out=out, stage_halves=hint, workspace=ws)
        out_host.copy_(out, non_blocking=True)

    for _ in range(3):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1)
    ops.check_device_status(dev)

    from mustafar_b200.sharding import max_over_ranks
    total_ms, e2e_ms, per_launch_ms = (max_over_ranks(x, dist, dev) for x in (total_ms, e2e_ms, per_launch_ms))

    # second half of the metric: Llama-3-8B-shape decode tokens/s, end to end (random-init weights, prompt 4096, greedy
    # steps at batch 32 per GPU, batch-sharded at every N; with 8 GPUs also the 8-way head-tensor-parallel arm, whose
    # all-reduces after o_proj / down_proj are the only collectives of this benchmark)
    e2e_llama = None
    if not a.no_e2e_llama:
        from mustafar_b200.e2e_llama import run_e2e
        del ks, vs, kw, vw, ws
        torch.cuda.empty_cache()
        e2e_llama = {}
        arms = [("batch_sharded", "dp")] + ([("tensor_parallel", "tp")] if world == 8 else [])
        for name, par in arms:
            try:        # the headline line is printed whatever happens here
                e2e_llama[name] = run_e2e(dev, rank, world, dist, new=a.e2e_llama_new, parallel=par)
            except Exception as e:
                e2e_llama[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                torch.cuda.empty_cache()

    # the other workloads of the path, a few calls each, so that one bench line shows them all (N = 1 only; their
    # parity is what the -m gpu tests check, here they are only timed): prune + compress of 64 heads x 8192 tokens,
    # the decode over the 2-bit cache at batch 32 x 16384 tokens, the per-step launches around the attention call
    other = None
    if world == 1 and not a.no_other_configs:
        try:
            other = other_configs()
        except Exception as e:
            other = {"error": f"{type(e).__name__}: {e}"[:300]}

    if rank == 0:
        peak, which = measured_peak_gbs()
        achieved = alg_bytes / (per_launch_ms * 1e-3) / 1e9
        line = {
            "metric": "sparse_decode_attention_throughput", "value": world * a.batch * a.steps / (total_ms * 1e-3),
            "unit": "tok/s/layer", "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3),
            "ms_per_step": total_ms / a.steps, "us_per_layer": 1e3 * total_ms / a.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 storage, f32 accumulate",
            "data": "synthetic", "config": config,
            "clocks": clocks.summary(),
            "e2e": {"value": world * a.batch * a.steps / (e2e_ms * 1e-3), "unit": "tok/s/layer",
                    "h2d_bytes_per_step": q.numel() * 2, "d2h_bytes_per_step": out.numel() * 2},
            "step_ms": {"min": step_ms[0], "median": step_ms[len(step_ms) // 2], "max": step_ms[-1]},
            "gpu_launches": a.steps,
            "parity_check": parity,
            "e2e_llama": e2e_llama,
            "other_configs": other,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": which, "frac_of_nominal_8000": achieved / 8000.0,
                         "algorithmic_bytes_per_launch": alg_bytes,
                         # dram bytes read + written per algorithmic byte in the ncu capture of a smaller case
                         # (profiles/decode_attn_traffic.txt), scaled by the units of this launch
                         "traffic": traffic_estimate(alg_bytes),
                         "kernel": "decode_attn_kernel (one launch per step: decode + merge of the split records)"},
        }
        if not a.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(a.kv_len, a.window, a.sparsity, a.cpu_seconds)
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        raise SystemExit(f"parity check failed: {parity}")


if __name__ == "__main__":
    main()
