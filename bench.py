#!/usr/bin/env python
"""Benchmark of the blockwise masked attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl ours|reference]

A step is one forward + backward pass of ``masked_attention_via_map`` over one batch of
synthetic input.  The metric is attention TFLOP/s counted on non-empty (full + partial) blocks
only: forward 4*bq*bk*d per block, backward 2.5x that.  With N > 1 (torchrun, one rank per GPU)
every rank runs the same per-GPU batch on its own data (batch x head shards need no
collective): weak scaling, value = total FLOPs of all ranks / max-over-ranks time.

``--impl reference`` times the CPU restatement of the reference algorithm (oracle/, torch CPU,
all host threads) on a bounded sample of the same workload; rank 0 only.
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np
import torch

METRIC = "attention_fwd_bwd_tflops"
UNIT = "TFLOP/s"

WORKLOADS = {
    # BASELINE.json configs[1]: the dense-causal reference shape the metric is quoted on
    "c2": dict(B=8, L=4096, H=32, d=128, bs=128, mask="causal", dtype="bf16", qkv_scale="rsqrt_d",
               desc="causal bf16 B=8 L=4096 H=32 d=128 block_size=128"),
    # a quarter of c2 (same per-(b,h) work): small enough for multi-pass ncu captures, inputs still exceed L2
    "c2_small": dict(B=2, L=4096, H=32, d=128, bs=128, mask="causal", dtype="bf16", qkv_scale="rsqrt_d",
                     desc="causal bf16 B=2 L=4096 H=32 d=128 block_size=128 (quarter of the dense-causal shape)"),
    # headline target shape of the north star (bf16 causal, L=8192, d=128)
    "t0": dict(B=4, L=8192, H=32, d=128, bs=128, mask="causal", dtype="bf16", qkv_scale="one",
               desc="causal bf16 B=4 L=8192 H=32 d=128 block_size=128"),
    "c3": dict(B=4, L=8192, H=16, d=128, bs=128, mask="sliding256", dtype="bf16", qkv_scale="one",
               desc="sliding window |q-k|<=256 bf16 B=4 L=8192 H=16 d=128 window_size=(256,256) block_size=128"),
    "c4": dict(B=4, L=16384, H=16, d=128, bs=128, mask="documents", dtype="bf16", qkv_scale="one",
               desc="packed documents (segments 256..4096) & causal, bf16 B=4 L=16384 H=16 d=128"),
    # BASELINE.json configs[4]: one long sequence (on one GPU here; the ring partition splits it over ranks)
    "c5": dict(B=1, L=131072, H=32, d=128, bs=128, mask="causal", dtype="bf16", qkv_scale="one",
               desc="causal bf16 B=1 L=131072 H=32 d=128 block_size=128"),
    # head dimension 64 on the tensor-core path (same model width as c2: 64 heads of 64)
    "d64": dict(B=8, L=4096, H=64, d=64, bs=128, mask="causal", dtype="bf16", qkv_scale="rsqrt_d",
                desc="causal bf16 B=8 L=4096 H=64 d=64 block_size=128"),
    "c1": dict(B=2, L=128, H=8, d=64, bs=32, mask="causal", dtype="f32", qkv_scale="one",
               desc="causal fp32 B=2 L=128 H=8 d=64 block_size=32"),
}


def ncu_traffic(workload):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch and kernel, from an ncu capture of the
    quarter-size workload (c2_small), kept as JSON beside the capture's summary.  The full-size shape is the
    captured one times four: every input is read once and every output written once, so traffic grows with the
    units processed.  Workloads without a capture report null."""
    try:
        table = json.loads((ROOT / "profiles" / "ncu_dram_traffic.json").read_text())
    except (OSError, ValueError):
        return {}
    entry = table.get("workloads", {}).get(workload)
    if entry is None:
        return {}
    base = table["captures"][entry["capture"]]
    return {k: v * entry["scale"] for k, v in base.items()}


class numa_local:
    """Runs the enclosed host allocations on CPUs of the NUMA node the GPU hangs off (sysfs: the PCI device's
    numa_node and that node's cpulist), so that pinned buffers are first touched — and therefore placed — next to the
    GPU's PCIe root complex instead of wherever the launcher happened to run.  Does nothing when the node cannot be
    found or the affinity cannot be set.  ``info`` records what was done, for the bench line."""

    def __init__(self, device_index):
        self.index, self.saved, self.info = device_index, None, {"numa_node": None}

    def __enter__(self):
        try:
            pr = torch.cuda.get_device_properties(self.index)
            bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
            node = int(Path(f"/sys/bus/pci/devices/{bdf.lower()}/numa_node").read_text())
            if node < 0:
                return self
            cpus = set()
            for part in Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            allowed = os.sched_getaffinity(0)
            target = cpus & allowed
            if target:
                self.saved = allowed
                os.sched_setaffinity(0, target)
                self.info = {"numa_node": node, "cpus_used": len(target)}
        except Exception as e:           # containers often hide sysfs or forbid the call: measure as is
            self.info = {"numa_node": None, "why": type(e).__name__}
        return self

    def __exit__(self, *exc):
        if self.saved is not None:
            try:
                os.sched_setaffinity(0, self.saved)
            except Exception:
                pass
        return False


def synth(shape, seed, dtype, scale=1.0, device="cpu", pin=False):
    """Seeded N(0,1) tensors: numpy PCG64(seed) -> float32 -> dtype (the configs' definition)."""
    x = np.random.Generator(np.random.PCG64(seed)).standard_normal(shape, dtype=np.float32)
    t = torch.from_numpy(x)
    if scale != 1.0:
        t = t * scale
    t = t.to(dtype)
    if pin:
        t = t.pin_memory()
    return t.to(device) if device != "cpu" else t


def document_segments(B, L, seed=4, lo=256, hi=4096):
    rng = np.random.Generator(np.random.PCG64(seed))
    seg = np.zeros((B, L), dtype=np.int32)
    for b in range(B):
        pos, sid = 0, 0
        while pos < L:
            n = int(rng.integers(lo, hi + 1))
            seg[b, pos:pos + n] = sid
            pos += n
            sid += 1
    return seg


def mask_kwargs(w, masks_mod, B=None, L=None):
    B, L = B or w["B"], L or w["L"]
    if w["mask"] == "causal":
        return dict(is_causal=True, block_size=w["bs"])
    if w["mask"] == "sliding256":
        return dict(mask_fn=masks_mod.sliding_window_mask(256, 256), window_size=(256, 256), block_size=w["bs"])
    if w["mask"] == "documents":
        return dict(mask_fn=masks_mod.document_mask(document_segments(B, L), causal=True), block_size=w["bs"])
    raise KeyError(w["mask"])


def torch_dtype(name):
    return {"bf16": torch.bfloat16, "f32": torch.float32}[name]


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        # keep the samples taken under load (the upper half of the observed clocks)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def flops_of(lists_tensors, w_bs, d, B, H):
    """(fwd, fwd+bwd) FLOPs counted on non-empty blocks from the compiled block lists."""
    n = lists_tensors["kv_num_blocks"].sum(dtype=torch.int64) + lists_tensors["full_kv_num_blocks"].sum(dtype=torch.int64)
    lb, lh = lists_tensors["kv_num_blocks"].shape[:2]
    blocks = int(n) * (B // lb) * (H // lh)
    fwd = 4.0 * w_bs * w_bs * d * blocks
    return fwd, 3.5 * fwd, blocks


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        j = json.loads(p.read_text())
        return j.get("bf16_tflops_sustained", 1385.6), j.get("bf16_tflops", 1648.3), j.get("hbm_gbs", 6548.8), "measured"
    return 1400.0, 1590.0, 6650.0, "fallback"


def cpu_reference_run(w, steps, warmup, threads=None):
    """Times the CPU restatement of the reference (oracle/attention_oracle.py, torch CPU) on a
    bounded sample: one batch row of the workload at full sequence length with as many heads as keep a step to a few
    seconds (8 at L = 4096: one head alone leaves most host threads idle and reads 3.5 times slower per head)."""
    from oracle import attention_oracle as ao
    from jaxmodules_b200 import masks as M
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    L, d = w["L"], w["d"]
    Bs, Hs = 1, max(1, min(w["H"], int(8 * (4096 / L) ** 2)))
    dt = torch_dtype(w["dtype"])
    scale = 1 / math.sqrt(d) if w["qkv_scale"] == "rsqrt_d" else 1.0
    Q, K, V = (synth((Bs, L, Hs, d), s, dt, scale) for s in (0, 1, 2))
    dO = synth((Bs, L, Hs, d), 3, torch.float32)
    kw = mask_kwargs(w, M, B=Bs, L=L)
    # useful FLOPs of the slice (non-empty 128-blocks), from a dense evaluation of the mask per block row
    mask_fn = ao.canonical_mask_fn(kw.get("mask_fn"), kw.get("is_causal", False))
    bs = w["bs"]
    blocks = 0
    for i in range(L // bs):
        row = ao.eval_mask_grid(mask_fn, Bs, Hs, np.arange(i * bs, (i + 1) * bs), np.arange(L))
        if kw.get("window_size") is not None:
            lb, rb = ao.window_blocks(kw["window_size"], bs)
            s = ao.window_start(i, lb, rb, L // bs)
            row[..., : s * bs] = False
            row[..., (s + lb + rb) * bs:] = False
        blocks += int(row.reshape(Bs, Hs, bs, L // bs, bs).any(axis=(2, 4)).sum())
    flops = 3.5 * 4.0 * bs * bs * d * blocks
    times = []
    for i in range(warmup + steps):
        t = time.perf_counter()
        ao.masked_attention_via_map(Q, K, V, dO=dO, **kw)
        if i >= warmup:
            times.append(time.perf_counter() - t)
    sec = float(np.mean(times))
    return dict(value=flops / sec / 1e12, seconds_per_step=sec, cores=threads,
                sample=f"B=1,H={Hs} slice of the workload at full L={L} (fwd+bwd of the reference algorithm, "
                       f"which visits every block; FLOPs counted on the {blocks} non-empty blocks only)")


def device_randn(shape, seed, dtype, scale, dev):
    """Seeded N(0,1) inputs generated on the device (the side workloads of ``extra``; the headline workload
    uses the configs' NumPy PCG64 definition through pinned host memory)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(shape, device=dev, generator=g)
    if scale != 1.0:
        x.mul_(scale)
    return x.to(dtype)


def dense_fp32_slice(q, k, v, do, allowed, scale, chunk=2048):
    """float32 attention of one (batch, head) slice on the GPU, written out densely in query chunks (torch
    float32 matmul, TF32 off): O, dQ, dK, dV from P = exp(s - lse), delta = rowsum(dO*O), dS = P*(dO V^T - delta)."""
    N, L = q.shape[0], k.shape[0]
    O, dQ = torch.empty_like(q), torch.empty_like(q)
    dK, dV = torch.zeros_like(k), torch.zeros_like(v)
    ki = torch.arange(L, device=q.device)[None, :]
    for q0 in range(0, N, chunk):
        sl = slice(q0, min(N, q0 + chunk))
        qi = torch.arange(sl.start, sl.stop, device=q.device)[:, None]
        s = (q[sl] @ k.T) * scale
        s.masked_fill_(~allowed(qi, ki), float("-inf"))
        lse = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[:, None])
        o = p @ v
        ds = p * (do[sl] @ v.T - (do[sl] * o).sum(dim=-1, keepdim=True))
        O[sl], dQ[sl] = o, (ds @ k) * scale
        dK += (ds.T @ q[sl]) * scale
        dV += p.T @ do[sl]
        del s, p, ds
    return dict(O=O, dQ=dQ, dK=dK, dV=dV)


def dense_predicate(w, seg):
    if w["mask"] == "causal":
        return lambda b: (lambda qi, ki: ki <= qi)
    if w["mask"] == "sliding256":
        return lambda b: (lambda qi, ki: (ki >= qi - 256) & (ki <= qi + 256))
    return lambda b: (lambda qi, ki: (seg[b][qi] == seg[b][ki]) & (ki <= qi))


def parity_of_slices(w, Q, K, V, dO, O, grads, seg=None, flex=False):
    """Observed max / mean absolute error of O, dQ, dK, dV on two (batch, head) slices of the benchmarked
    workload against the dense float32 attention of the same slice (slices are independent)."""
    B, H, d = w["B"], w["H"], w["d"]
    pick = (lambda t, b, h: t[b, h]) if flex else (lambda t, b, h: t[b, :, h])
    pred = dense_predicate(w, None if seg is None else torch.from_numpy(seg).to(Q.device))
    out = {}
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for b, h in ((0, 0), (B - 1, H - 1)):
            ref = dense_fp32_slice(pick(Q, b, h).detach().float(), pick(K, b, h).detach().float(), pick(V, b, h).detach().float(),
                                   pick(dO, b, h).float(), pred(b), 1 / math.sqrt(d))
            for name, got in zip(("O", "dQ", "dK", "dV"), (O,) + tuple(grads)):
                err = (pick(got, b, h).detach().float() - ref[name]).abs()
                e = out.setdefault(name, {"max_abs": 0.0, "mean_abs": 0.0, "ref_max_abs": 0.0})
                e["max_abs"] = max(e["max_abs"], float(err.max()))
                e["mean_abs"] = max(e["mean_abs"], float(err.mean()))
                e["ref_max_abs"] = max(e["ref_max_abs"], float(ref[name].abs().max()))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    out["against"] = "dense float32 torch attention of the slices (b,h) = (0,0) and (B-1,H-1); worst of the two"
    out["bound"] = "max-abs 2e-2, mean-abs 2e-3 (bf16 I/O)" if w["dtype"] == "bf16" else "max-abs 1e-4 (fp32 I/O)"
    return out


def _traced_causal(b, h, q, k):
    return k <= q


def measure_config(name, dev, steps=5, warmup=3, seed=100, traced=False):
    """One side workload, device-timed: forward + backward through masked_attention_via_map on inputs generated
    on the device; the launch groups are timed separately with CUDA events on the launching stream.  ``traced``:
    the causal mask as a plain Python lambda instead of ``is_causal`` — it is traced into a mask program, evaluated
    on the device into the tile form of the mask description (once, cached on the function) and read by the kernels
    on the tiles it cuts."""
    import jaxmodules_b200 as jm
    from jaxmodules_b200 import _native as nat, attention as A, masks as M
    from jaxmodules_b200.block_mask import compile_block_lists
    w = WORKLOADS[name]
    B, L, H, d = w["B"], w["L"], w["H"], w["d"]
    dt = torch_dtype(w["dtype"])
    scale = 1 / math.sqrt(d) if w["qkv_scale"] == "rsqrt_d" else 1.0
    Q, K, V = (device_randn((B, L, H, d), seed + i, dt, scale, dev).requires_grad_(True) for i in range(3))
    dO = device_randn((B, L, H, d), seed + 3, torch.float32, 1.0, dev)
    kw = mask_kwargs(w, M)
    if traced:
        assert w["mask"] == "causal"
        kw = dict(mask_fn=_traced_causal, block_size=w["bs"])
    be, tq, tk = A.plan(Q, K, V)
    terms = M.MaskTerms(causal=True) if kw.get("is_causal") else M.terms_from_mask_fn(kw["mask_fn"], B, H, L, L, device=dev)
    if kw.get("window_size") is not None:
        bs = w["bs"]
        terms = terms.merged(M.MaskTerms(window=(bs, (kw["window_size"][0] + bs - 1) // bs, 1 + (kw["window_size"][1] + bs - 1) // bs, L // bs)))
    _, lt = compile_block_lists(M.to_device_mask(terms, L, L, dev), B, H, L, L, tq, tk, dev, q_side=False)
    fwd_flops, step_flops, blocks = flops_of(lt, tq, d, B, H)

    def step():
        O = jm.masked_attention_via_map(Q, K, V, **kw)
        Q.grad = K.grad = V.grad = None
        O.backward(dO)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize(dev)
    # short workloads: keep warming until the GPU has been busy for 0.2 s, or its clocks are still ramping when timing starts
    w0 = time.perf_counter()
    while time.perf_counter() - w0 < 0.2:
        step()
        torch.cuda.synchronize(dev)
    sink = {}
    A.set_profile_sink(sink)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step()
    t1.record()
    torch.cuda.synchronize(dev)
    A.set_profile_sink(None)
    ms = t0.elapsed_time(t1) / steps
    per = {k: float(np.mean([a.elapsed_time(b) for a, b in v])) for k, v in sink.items()}
    _, burst, _, _ = peaks()
    tf = lambda fl, t: fl / (t * 1e-3) / 1e12 if t else None
    if traced:
        t = terms.tiles if terms.tiles is not None else None
        w = dict(w, desc=w["desc"] + ", mask as a traced Python lambda (" + ("tile form: %d cut tiles of 4 KB" % t[2].shape[0] if t else "dense bit table") + ")")
    in_bytes = 3 * B * L * H * d * Q.element_size() + dO.numel() * 4
    out = {"l2": ("inputs (%.0f MB) exceed the 126 MB L2; no flush needed" % (in_bytes / 1e6)) if in_bytes > 126e6 else
                 ("inputs (%.2f MB) fit in L2 and are not flushed: a latency figure, not a bandwidth one" % (in_bytes / 1e6)),
           "workload": w["desc"], "backend": {1: "simt", 2: "tcgen05"}.get(be, str(be)), "steps": steps, "warmup": warmup,
           "nonempty_blocks": blocks, "ms_per_step": ms, "value": tf(step_flops, ms), "fwd_tflops": tf(fwd_flops, per.get("fwd")),
           "bwd_tflops": tf(step_flops - fwd_flops, per.get("bwd")), "kernel_ms": per, "status": A.device_status(dev)}
    if be == 2:
        out["frac_of_burst"] = {"value": out["value"] / burst, "fwd": out["fwd_tflops"] / burst, "bwd": out["bwd_tflops"] / burst}
    else:
        out["us_per_step"] = ms * 1e3      # latency-bound shapes
    del Q, K, V, dO
    torch.cuda.empty_cache()
    return out


def block_mask_build_entry(w, dev, steps, warmup):
    """create_block_mask alone (full [B, H] extents, both list sides): HBM-write bound."""
    import jaxmodules_b200 as jm
    from jaxmodules_b200 import masks as M
    B, L, H, bs = w["B"], w["L"], w["H"], w["bs"]
    if w["mask"] == "causal":
        mask_mod = M.causal_mask()
    elif w["mask"] == "sliding256":
        mask_mod = M.sliding_window_mask(256, 256)
    else:
        mask_mod = M.document_mask(document_segments(B, L), causal=True)
    build = lambda: jm.create_block_mask(mask_mod, B, H, L, L, bs, device=dev)
    for _ in range(warmup):
        build()
    torch.cuda.synchronize(dev)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        build()
    t1.record()
    torch.cuda.synchronize(dev)
    ms = t0.elapsed_time(t1) / steps
    NQ = NKV = L // bs
    out_bytes = 2 * 4 * (2 * B * H * NQ + 2 * B * H * NQ * NKV)
    _, _, hbm, peak_kind = peaks()
    gbs = out_bytes / (ms * 1e-3) / 1e9
    torch.cuda.empty_cache()
    return {"workload": "create_block_mask, " + w["desc"], "ms": ms, "list_bytes_per_build": out_bytes, "GB/s": gbs,
            "frac_of_hbm": gbs / hbm, "peak": hbm, "peak_kind": peak_kind,
            "kernels": "classify_kernel + compact_both_kernel"}


def c5_head_shards(rank, world, dev, dist, steps=3, warmup=2):
    """BASELINE config 5 split by head: each rank takes H/N heads of the ONE B=1 sequence (strong scaling, no
    collective on the data path); value = the whole sequence's FLOPs / max-over-ranks step time."""
    import jaxmodules_b200 as jm
    from jaxmodules_b200 import sharding as S
    w = WORKLOADS["c5"]
    B, L, H, d = w["B"], w["L"], w["H"], w["d"]
    units = S.shard_units(B, H, rank, world)
    shards = []
    for b, h0, h1 in units:      # this rank's heads only are ever materialised
        q, k, v = (device_randn((1, L, h1 - h0, d), 1000 * (b * H + h0) + i, torch.bfloat16, 1.0, dev).requires_grad_(True) for i in range(3))
        shards.append((q, k, v, device_randn((1, L, h1 - h0, d), 1000 * (b * H + h0) + 3, torch.float32, 1.0, dev)))

    def step():
        for q, k, v, do in shards:
            o = jm.masked_attention_via_map(q, k, v, is_causal=True, block_size=w["bs"])
            q.grad = k.grad = v.grad = None
            o.backward(do)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(warmup):
        step()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step()
    t1.record()
    barrier()
    ms = t0.elapsed_time(t1) / steps
    if dist is not None:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    nblk = L // 128
    flops = 3.5 * 4.0 * 128 * 128 * d * (B * H * nblk * (nblk + 1) // 2)
    del shards
    torch.cuda.empty_cache()
    _, burst, _, _ = peaks()
    tfl = flops / (ms * 1e-3) / 1e12
    return {"workload": w["desc"], "parallelism": f"{H} heads of one sequence dealt to {world} GPU(s) (sharding.shard_units), no collective",
            "scaling": "strong", "heads_per_gpu": [h1 - h0 for _, h0, h1 in units], "steps": steps, "warmup": warmup, "ms_per_step": ms, "value": tfl,
            "per_gpu": tfl / world, "frac_of_burst_per_gpu": tfl / world / burst}


def run_reference(args, w, rank):
    if rank != 0:
        return
    r = cpu_reference_run(w, steps=max(1, min(args.steps, 3)), warmup=min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": max(1, min(args.steps, 3)), "warmup": min(args.warmup, 1), "ms_per_step": r["seconds_per_step"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": w["desc"], "note": "reference algorithm restated on CPU (JAX is not installed on this box)"},
        "cpu_baseline": {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port", "sample": r["sample"]},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_block_mask_build(args, w, rank, world, dev, warmup):
    """``--block-mask``: the BlockMask builder alone, as its own JSON line."""
    from jaxmodules_b200 import _native as nat
    launches0 = nat.lib().bma_launch_count()
    e = block_mask_build_entry(w, dev, args.steps, warmup)
    if rank == 0:
        print(json.dumps({
            "metric": "block_mask_build_bandwidth", "value": e["GB/s"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
            "ms_per_step": e["ms"], "higher_is_better": True, "dtype": "int32", "data": "synthetic",
            "config": {"workload": e["workload"], "list_bytes_per_build": e["list_bytes_per_build"],
                       "l2": "each build writes fresh output arrays" + (" larger than the 126 MB L2" if e["list_bytes_per_build"] > 126e6 else " (they fit in L2: latency-bound)")},
            "roofline": {"bound": "hbm", "kernel": e["kernels"], "achieved": e["GB/s"], "peak": e["peak"],
                         "unit": "GB/s", "frac": e["frac_of_hbm"], "traffic": None, "peak_kind": e["peak_kind"]},
            "gpu_launches": int(nat.lib().bma_launch_count() - launches0)}), flush=True)


def ring_entry(w, rank, world, local_rank, dev, dist, steps, warmup, ring="zigzag", sample_clocks=True):
    """Sequence-partition mode: forward and backward of ONE causal sequence set split over the ranks
    (strong scaling); K/V and the dK/dV accumulators travel round the ring over NCCL P2P.  Returns the
    result line (meaningful on rank 0)."""
    from jaxmodules_b200 import _native as nat, masks as M, sharding as S
    B, L, H, d = w["B"], w["L"], w["H"], w["d"]
    assert w["mask"] == "causal" and L % (2 * world * 128) == 0
    dt = torch_dtype(w["dtype"])
    n = L // world
    scale = 1 / math.sqrt(d) if w["qkv_scale"] == "rsqrt_d" else 1.0
    Q, K, V = (device_randn((B, n, H, d), 10 * rank + s, dt, scale, dev) for s in (0, 1, 2))
    dO = device_randn((B, n, H, d), 10 * rank + 3, torch.float32, 1.0, dev)
    layout = (S.zigzag_layout if ring == "zigzag" else S.contiguous_layout)(n)
    terms = M.MaskTerms(causal=True)
    timing = {}

    def step():
        O, lse = S.ring_attention_forward(Q, K, V, rank=rank, world=world, terms=terms, layout=layout)
        return S.ring_attention_backward(Q, K, V, O, lse, dO, rank=rank, world=world, terms=terms, layout=layout)

    # The same ring with one half switched off, to show how much of the transfer hides under the kernels: the kernels
    # alone (the exchange hands back local buffers of the right shape) and the transfers alone (the kernels are stubs).
    local = lambda tensors, dst, src: [torch.empty_like(t) for t in tensors]

    def compute_only():
        O, lse = S.ring_attention_forward(Q, K, V, rank=rank, world=world, terms=terms, layout=layout, exchange=local)
        return S.ring_attention_backward(Q, K, V, O, lse, dO, rank=rank, world=world, terms=terms, layout=layout, exchange=local)

    # stub results, cut to the shape of each call (a ring step joins segments into calls of n/2 or n tokens a side)
    stub_o = torch.zeros((B, n, H, d), dtype=torch.float32, device=dev)
    stub_lse = torch.zeros((B, H, n), dtype=torch.float32, device=dev)
    stub_g = torch.zeros((B, n, H, d), dtype=dt, device=dev)

    def transfer_only():
        O, lse = S.ring_attention_forward(Q, K, V, rank=rank, world=world, terms=terms, layout=layout,
                                          attend=lambda q, k, v, t: (stub_o[:, :q.shape[1]], stub_lse[:, :, :q.shape[1]]),
                                          merge=lambda o, l, o2, l2: (o, l))
        O = torch.zeros((B, n, H, d), dtype=torch.float32, device=dev) if O.shape[1] != n else O
        lse = torch.zeros((B, H, n), dtype=torch.float32, device=dev) if lse.shape[2] != n else lse
        return S.ring_attention_backward(Q, K, V, O, lse, dO, rank=rank, world=world, terms=terms, layout=layout,
                                         backward=lambda q, k, v, o, l, g, t: (stub_g[:, :q.shape[1]], stub_g[:, :k.shape[1]],
                                                                               stub_g[:, :k.shape[1]]))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, reps):
        fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / reps
        if dist is not None:
            tt = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt[0])
        return ms

    nblk = L // 128
    blocks = B * H * nblk * (nblk + 1) // 2                      # non-empty 128x128 blocks of the whole causal sequence
    step_flops = 3.5 * 4.0 * 128 * 128 * d * blocks
    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0 and sample_clocks:
        sampler.start()
    launches0 = nat.lib().bma_launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(steps):
        step()
    t1.record()
    barrier()
    clocks = sampler.stop() if (rank == 0 and sample_clocks) else None
    launches = nat.lib().bma_launch_count() - launches0
    ms_step = t0.elapsed_time(t1) / steps
    if dist is not None:
        t = torch.tensor([ms_step], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t[0])
    sustained, burst, hbm, peak_kind = peaks()
    tf = step_flops / (ms_step * 1e-3) / 1e12
    compute_ms, transfer_ms = timed(compute_only, 2), (timed(transfer_only, 2) if world > 1 else 0.0)
    del Q, K, V, dO
    torch.cuda.empty_cache()
    return {
        "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": w["dtype"],
        "data": "synthetic",
        "config": {"workload": w["desc"], "api": "sharding.ring_attention_forward + ring_attention_backward",
                   "parallelism": f"sequence split over {world} GPU(s), {ring} token layout, K/V and dK/dV ring over NCCL P2P",
                   "tokens_per_gpu": n, "nonempty_blocks_total": blocks, "flop_model": "fwd 4*bq*bk*d per non-empty block, bwd 2.5x fwd",
                   "l2": "inputs exceed the 126 MB L2; no flush needed"},
        "roofline": {"bound": "tensor", "kernel": "forward + backward kernels of all ring steps", "achieved": tf / world,
                     "peak": sustained, "unit": "TFLOP/s per GPU", "frac": tf / world / sustained, "traffic": None,
                     "peak_kind": f"{peak_kind} sustained dense bf16"},
        "per_gpu": tf / world, "frac_of_burst_per_gpu": tf / world / burst,
        # max over ranks each: the whole step, its kernels without any transfer, its transfers without any kernel
        "overlap": {"step_ms": ms_step, "compute_only_ms": compute_ms, "transfer_only_ms": transfer_ms,
                    "transfer_hidden_ms": max(0.0, compute_ms + transfer_ms - ms_step)},
        "clocks": clocks, "gpu_launches": int(launches)}


def run_ring(args, w, rank, world, local_rank, dev, dist, warmup):
    line = ring_entry(w, rank, world, local_rank, dev, dist, args.steps, warmup, args.ring)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--api", default="via_map", choices=["via_map", "flex"],
                    help="public entry point under test: masked_attention_via_map on [B,L,H,d] (default) or "
                         "flex_attention on [B,H,L,d] with a BlockMask built once outside the timed region")
    ap.add_argument("--ring", default=None, choices=["contiguous", "zigzag"],
                    help="sequence partition instead of batch x head shards: every rank holds L/N tokens of ONE sequence "
                         "set (strong scaling); K/V and the dK/dV accumulators travel round the ring")
    ap.add_argument("--block-mask", action="store_true",
                    help="time create_block_mask (the BlockMask builder) at the workload's geometry instead of attention")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the `extra` entries: parity of the benchmarked workload, the other configurations, the "
                         "BlockMask builder at config 5 and (N > 1) config 5 split by head and as a ring")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, w, rank)
        return

    import jaxmodules_b200 as jm
    from jaxmodules_b200 import _native as nat, attention as A, masks as M

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)
    if args.ring:
        run_ring(args, w, rank, world, local_rank, dev, dist, warmup)
        return
    if args.block_mask:
        run_block_mask_build(args, w, rank, world, dev, warmup)
        return

    B, L, H, d = w["B"], w["L"], w["H"], w["d"]
    dt = torch_dtype(w["dtype"])
    scale = 1 / math.sqrt(d) if w["qkv_scale"] == "rsqrt_d" else 1.0
    # every rank owns its own batch (seeds offset by rank): batch x head shards, no collective
    flex = args.api == "flex"
    shape = (B, H, L, d) if flex else (B, L, H, d)
    numa = numa_local(local_rank)
    with numa:          # pinned host buffers next to this GPU's PCIe root (matters once eight ranks share the host)
        hQ, hK, hV = (synth(shape, 10 * rank + s, dt, scale, pin=True) for s in (0, 1, 2))
        hdO = synth(shape, 10 * rank + 3, torch.float32, pin=True)
    Q, K, V = (x.to(dev).requires_grad_(True) for x in (hQ, hK, hV))
    dO = hdO.to(dev)
    kw = mask_kwargs(w, M)
    if flex:
        mask_mod = M.causal_mask() if kw.get("is_causal") else kw["mask_fn"]
        block_mask = jm.create_block_mask(mask_mod, B if w["mask"] == "documents" else 1, 1, L, L, 128, device=dev)
        attend = lambda q, k, v: jm.flex_attention(q, k, v, block_mask=block_mask)
    else:
        attend = lambda q, k, v: jm.masked_attention_via_map(q, k, v, **kw)

    def step():
        O = attend(Q, K, V)
        Q.grad = K.grad = V.grad = None
        O.backward(dO)
        return O

    seg_np = document_segments(B, L) if w["mask"] == "documents" else None

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # FLOP count from the block lists the kernels actually walk
    be, tq, tk = A.plan(*((x.transpose(1, 2) for x in (Q, K, V)) if flex else (Q, K, V)))
    terms = M.MaskTerms(causal=True) if kw.get("is_causal") else M.terms_from_mask_fn(kw["mask_fn"], B, H, L, L)
    if kw.get("window_size") is not None:
        bs = w["bs"]
        lb, rb = (kw["window_size"][0] + bs - 1) // bs, 1 + (kw["window_size"][1] + bs - 1) // bs
        terms = terms.merged(M.MaskTerms(window=(bs, lb, rb, L // bs)))
    from jaxmodules_b200.block_mask import compile_block_lists
    dm = M.to_device_mask(terms, L, L, dev)
    _, lt = compile_block_lists(dm, B, H, L, L, tq, tk, dev, q_side=False)
    fwd_flops, step_flops, blocks = flops_of(lt, tq, d, B, H)

    for _ in range(warmup):
        step()
    barrier()

    sink = {}
    A.set_profile_sink(sink)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = nat.lib().bma_launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(args.steps):
        step()
    t1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    launches = nat.lib().bma_launch_count() - launches0
    A.set_profile_sink(None)
    ms_total = t0.elapsed_time(t1)
    status = A.device_status(dev)      # non-zero: a bounded wait inside a kernel gave up and the results are invalid
    assert status == 0, f"device status {status} after the timed region"
    parity = None
    if rank == 0 and not args.no_extra:
        O_last = step()
        torch.cuda.synchronize(dev)
        parity = parity_of_slices(w, Q, K, V, dO, O_last, (Q.grad, K.grad, V.grad), seg=seg_np, flex=flex)
        del O_last
    per_kernel = {k: float(np.mean([a.elapsed_time(b) for a, b in v])) for k, v in sink.items()}

    # end to end through the public API with host buffers (H2D of inputs, D2H of results inside the timed region)
    e2e = None
    if not args.no_e2e:
        # A training loop prefetches: the inputs of step i+1 travel host -> device on their own stream
        # while step i computes and the results of step i-1 travel device -> host on a third stream
        # (PCIe is full duplex).  Every step still copies all of its inputs in and all of its results
        # out inside the timed region; the two copy directions and the kernels merely overlap.
        main = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        with numa:
            host_out = [[torch.empty(shape, dtype=torch.float32).pin_memory()] +
                        [torch.empty(shape, dtype=dt).pin_memory() for _ in range(3)] for _ in range(2)]
        outs = host_out[0]
        dev_in = [None, None]
        in_ready = [torch.cuda.Event(), torch.cuda.Event()]       # Q, K, V of the slot have arrived
        do_ready = [torch.cuda.Event(), torch.cuda.Event()]       # ... and the cotangent, which only the backward needs
        fwd_done = [torch.cuda.Event(), torch.cuda.Event()]
        computed = [torch.cuda.Event(), torch.cuda.Event()]
        copied_out = [torch.cuda.Event(), torch.cuda.Event()]

        def upload(slot):
            with torch.cuda.stream(s_in):
                s_in.wait_event(computed[slot])          # the step that read this slot last has finished
                dev_in[slot] = [x.to(dev, non_blocking=True) for x in (hQ, hK, hV)]
                in_ready[slot].record(s_in)
                dev_in[slot].append(hdO.to(dev, non_blocking=True))
                do_ready[slot].record(s_in)
                for x in dev_in[slot]:
                    x.record_stream(main)

        kept = []

        def e2e_run(n, compute=True):
            for ev in computed + copied_out:
                ev.record(main)
            upload(0)
            for i in range(n):
                slot = i & 1
                if i + 1 < n:
                    upload(slot ^ 1)
                main.wait_event(in_ready[slot])
                if compute:
                    q, k, v = (x.requires_grad_(True) for x in dev_in[slot][:3])
                    o = attend(q, k, v)
                    fwd_done[slot].record(main)
                    main.wait_event(do_ready[slot])
                    o.backward(dev_in[slot][3])
                    computed[slot].record(main)
                    results = (o.detach(), q.grad, k.grad, v.grad)
                    kept[:] = [results]
                else:
                    # the copies alone: same buffers, streams and ordering, no kernels (results of an earlier step go out)
                    fwd_done[slot].record(main)
                    main.wait_event(do_ready[slot])
                    computed[slot].record(main)
                    results = kept[0]
                with torch.cuda.stream(s_out):
                    s_out.wait_event(fwd_done[slot])         # O leaves while the backward runs
                    host_out[slot][0].copy_(results[0], non_blocking=True)
                    s_out.wait_event(computed[slot])
                    for dst, src in zip(host_out[slot][1:], results[1:]):
                        dst.copy_(src, non_blocking=True)
                    for src in results:
                        src.record_stream(s_out)
                    copied_out[slot].record(s_out)
            main.wait_stream(s_out)

        e2e_steps = max(2, args.steps)   # pipeline fill (first upload) and drain (last download) are inside the timed region
        e2e_run(2)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_run(e2e_steps)
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        c0.record()
        e2e_run(e2e_steps, compute=False)
        c1.record()
        barrier()
        copy_ms = c0.elapsed_time(c1) / e2e_steps
        h2d = sum(x.numel() * x.element_size() for x in (hQ, hK, hV, hdO))
        d2h = sum(x.numel() * x.element_size() for x in outs)
        e2e = (e2e_ms, h2d, d2h, copy_ms)
        del kept[:], dev_in[:], host_out

    ms_step = ms_total / args.steps
    if dist is not None:
        t = torch.tensor([ms_step, e2e[0] if e2e else 0.0, e2e[3] if e2e else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t[0])
        if e2e:
            e2e = (float(t[1]), e2e[1], e2e[2], float(t[2]))

    # ---- `extra`: everything beside the headline workload that a reader of this one line should see ----------
    extra = {}
    if not args.no_extra:
        del Q, K, V, dO, hQ, hK, hV, hdO
        torch.cuda.empty_cache()
        if parity is not None:
            extra["parity"] = parity
        if world == 1:
            extra["per_config"] = {name: measure_config(name, dev) for name in ("t0", "c3", "c4", "c5", "d64", "c1") if name != args.workload}
            extra["traced_mask_t0"] = measure_config("t0", dev, traced=True)
            extra["block_mask_c5"] = block_mask_build_entry(WORKLOADS["c5"], dev, steps=5, warmup=3)
        else:
            extra["c5_head_shards"] = c5_head_shards(rank, world, dev, dist)
            if WORKLOADS["c5"]["L"] % (2 * world * 128) == 0:
                r = ring_entry(WORKLOADS["c5"], rank, world, local_rank, dev, dist, steps=3, warmup=2, ring="zigzag", sample_clocks=False)
                extra["ring_c5"] = {k: r[k] for k in ("value", "ms_per_step", "steps", "warmup", "scaling", "per_gpu", "frac_of_burst_per_gpu", "overlap", "gpu_launches")}
                extra["ring_c5"]["parallelism"] = r["config"]["parallelism"]
                extra["ring_c5"]["workload"] = r["config"]["workload"]

    if rank == 0:
        sustained, burst, hbm, peak_kind = peaks()
        total_flops = step_flops * world
        bwd_ms = per_kernel.get("bwd")
        fwd_ms = per_kernel.get("fwd")
        bwd_tf = (step_flops - fwd_flops) / (bwd_ms * 1e-3) / 1e12 if bwd_ms else None
        fwd_tf = fwd_flops / (fwd_ms * 1e-3) / 1e12 if fwd_ms else None
        traffic = ncu_traffic(args.workload)
        line = {
            "metric": METRIC, "value": total_flops / (ms_step * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": w["desc"], "api": "flex_attention [B,H,L,d] + BlockMask(128)" if flex else "masked_attention_via_map [B,L,H,d]",
                       "per_gpu_batch": B, "global_batch": B * world,
                       "parallelism": f"batch x head shards, {world} GPU(s), no collective",
                       "backend": {1: "simt", 2: "tcgen05"}.get(be, str(be)), "tile": tq, "nonempty_blocks_per_gpu": blocks,
                       "l2": "inputs (Q,K,V,dO > 1 GB) exceed the 126 MB L2; no flush needed",
                       "flop_model": "fwd 4*bq*bk*d per non-empty block, bwd 2.5x fwd"},
            "fwd_tflops": fwd_tf, "bwd_tflops": bwd_tf,
            "kernel_ms": per_kernel,
            "roofline": {"bound": "tensor", "kernel": "backward (bwd_dkdv_kernel + dQ kernel)", "achieved": bwd_tf, "peak": sustained,
                         "unit": "TFLOP/s", "frac": (bwd_tf / sustained) if bwd_tf else None, "traffic": traffic.get("bwd"),
                         "peak_kind": f"{peak_kind} sustained dense bf16 (kernel timed inside a long step)"},
            "roofline_fwd": {"bound": "tensor", "kernel": "forward", "achieved": fwd_tf, "peak": sustained, "unit": "TFLOP/s",
                             "frac": (fwd_tf / sustained) if fwd_tf else None, "traffic": traffic.get("fwd")},
            "clocks": clocks, "gpu_launches": int(launches),
        }
        pre_ms = per_kernel.get("bwd_preprocess")
        if pre_ms and w["dtype"] == "bf16" and be == 2:
            # delta = rowsum(dO * O) and the bf16 copy of the float32 cotangent: reads O and dO (float32), writes dO (bf16) and delta
            pre_bytes = B * L * H * d * (4 + 4 + 2) + 4 * B * H * L
            pre_gbs = pre_bytes / (pre_ms * 1e-3) / 1e9
            line["roofline_preprocess"] = {"bound": "hbm", "kernel": "bwd_preprocess_rows4_kernel", "achieved": pre_gbs, "peak": hbm,
                                           "unit": "GB/s", "frac": pre_gbs / hbm, "traffic": None}
        dkdv_ms, replay_ms = per_kernel.get("bwd_dkdv"), per_kernel.get("bwd_dq_replay")
        if dkdv_ms and replay_ms:
            # The two backward kernels timed separately (the library records an event between them).  The dK/dV kernel
            # runs 4 of the 5 algorithmic MMAs of the backward; the replay kernel runs the fifth and is bound by the HBM
            # stream of the dS tiles: 32 KB per non-empty block, plus K read once and dQ written once.
            dkdv_tf = 0.8 * (step_flops - fwd_flops) / (dkdv_ms * 1e-3) / 1e12
            line["roofline"] = {"bound": "tensor", "kernel": "bwd_dkdv_kernel (dominant: %.0f %% of the step)" % (100 * dkdv_ms / ms_step),
                                "achieved": dkdv_tf, "peak": sustained, "unit": "TFLOP/s", "frac": dkdv_tf / sustained,
                                "traffic": traffic.get("bwd_dkdv"),
                                "peak_kind": f"{peak_kind} sustained dense bf16 (kernel timed inside a long step)"}
            replay_bytes = blocks * 32768 + 2 * B * L * H * d * 2
            replay_gbs = replay_bytes / (replay_ms * 1e-3) / 1e9
            line["roofline_dq_replay"] = {"bound": "hbm", "kernel": "bwd_dq_replay_kernel", "achieved": replay_gbs, "peak": hbm,
                                          "unit": "GB/s", "frac": replay_gbs / hbm, "traffic": traffic.get("bwd_dq_replay")}
            line["roofline_bwd"] = {"bound": "tensor", "kernel": "backward (bwd_dkdv_kernel + bwd_dq_replay_kernel)", "achieved": bwd_tf,
                                    "peak": sustained, "unit": "TFLOP/s", "frac": (bwd_tf / sustained) if bwd_tf else None,
                                    "traffic": traffic.get("bwd")}
        if e2e:
            line["e2e"] = {"value": total_flops / (e2e[0] * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e[0],
                           "h2d_bytes_per_step": e2e[1], "d2h_bytes_per_step": e2e[2],
                           # the same copies on the same streams with no kernel in between: the box's own ceiling
                           "copy_only_ms_per_step": e2e[3], "copy_only_GBps_each_way": e2e[1] / (e2e[3] * 1e-3) / 1e9,
                           "pinned_host_buffers": numa.info}
        if extra:
            line["extra"] = extra
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_reference_run(w, steps=1, warmup=1)
            line["cpu_baseline"] = {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port",
                                    "sample": r["sample"], "seconds": r["seconds_per_step"]}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
