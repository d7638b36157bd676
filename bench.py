#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one pass of the hot path over one batch of synthetic input.  The headline workload is
paged GQA decode at batch 32 (48 query / 8 KV heads, head_dim 128, contexts U{1024..16384}, 16-token
pages scattered through a shared pool, split-KV chunk 512): fused RoPE + KV-append of the current
token, split-KV attention, combine.  `value` is algorithmic KV bytes per second with everything
resident in HBM; `e2e` is the same metric through the public API with host buffers (pinned host ->
device copy of the step's Q/K/V and a device -> host read of the output inside the timed region).
Other workloads of the path are measured in the same run and reported under "workloads".

With N > 1 (torchrun, one rank per GPU) sequences are sharded across ranks -- every rank owns its own
batch and pages, no data-path collective -- and `value` is the sum over ranks divided by the slowest
rank's time (weak scaling).

`--impl reference` times the CPU oracle (a scalar port of the reference's kernels; the reference is
Rust + Metal and cannot be built here) on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 0x1FE2A0


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops"], "tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        rows = []
        for line in self.file:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                rows.append((float(parts[0]), float(parts[1]), float(parts[2]), parts[3:7]))
            except ValueError:
                continue
        self.file.close()
        os.unlink(self.file.name)
        if not rows:
            return out
        pmax = max(r[2] for r in rows)
        loaded = [r for r in rows if r[2] >= 0.6 * pmax] or rows
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in loaded for i in range(4) if r[3][i].lower().startswith("active")})
        out.update(sm_mhz=statistics.median(r[0] for r in loaded), sm_max_mhz=max(r[1] for r in rows), reasons=reasons,
                   samples=len(loaded), power_w_max=pmax)
        return out


# ----------------------------------------------------------------------------- workloads
def decode_lens(rank: int, batch: int = 32):
    rng = np.random.RandomState(SEED + 3 + 7919 * rank)
    return rng.randint(1024, 16384 + 1, size=batch).astype(np.int32)


class GqaDecodeB32:
    """Paged GQA decode, batch 32 (the third benchmark configuration)."""
    name = "gqa_decode_b32"
    metric, unit, bound = "attn_decode_hbm_gbs", "GB/s", "hbm"
    kernel = "gqa_decode_partial_kernel"
    launches_per_step = 3  # rope+append, split-KV partial, combine
    B, Hq, Hkv, D, P, CHUNK, THETA = 32, 48, 8, 128, 16, 512, 500000.0

    def __init__(self, be, rank):
        import torch
        self.torch, self.be = torch, be
        self.lens = decode_lens(rank, self.B)
        pages = (self.lens + self.P - 1) // self.P
        self.num_pages = int(pages.sum()) + 64
        g = torch.Generator(device="cpu").manual_seed(SEED + 5 + rank)
        perm = torch.randperm(self.num_pages, generator=g).to(torch.int32)
        table = torch.full((self.B, int(pages.max())), 0, dtype=torch.int32)
        o = 0
        for b, n in enumerate(pages):
            table[b, :n] = perm[o:o + n]
            o += int(n)
        self.pool = be.prepare_kv_pool(self.num_pages, self.P, self.Hkv, self.D)
        gd = torch.Generator(device=be.device).manual_seed(SEED + 6 + rank)
        self.pool.k.normal_(0, 1, generator=gd)
        self.pool.v.normal_(0, 1, generator=gd)
        self.past = be.page_table(table, self.lens - 1, validate_on_host=False)
        self.full = be.page_table(table, self.lens, validate_on_host=False)
        inv = 1.0 / np.power(np.float32(self.THETA), (2 * np.arange(32)).astype(np.float32) / np.float32(64))
        self.rope = be.prepare_rope_table(inv.astype(np.float32), 64, 1.0)
        self.q = torch.randn((self.B, 1, self.Hq, self.D), generator=gd, device=be.device, dtype=torch.float16)
        self.k = torch.randn((self.B, 1, self.Hkv, self.D), generator=gd, device=be.device, dtype=torch.float16)
        self.v = torch.randn((self.B, 1, self.Hkv, self.D), generator=gd, device=be.device, dtype=torch.float16)
        self.out = torch.empty((self.B, self.Hq, self.D), dtype=torch.float32, device=be.device)
        self.hq, self.hk, self.hv = (t.cpu().pin_memory() for t in (self.q, self.k, self.v))
        self.hout = torch.empty((self.B, self.Hq, self.D), dtype=torch.float32).pin_memory()
        self.max_len = int(self.lens.max())
        self.units_per_step = float(self.lens.astype(np.int64).sum()) * self.Hkv * self.D * 2 * 2  # KV bytes
        self.h2d = sum(t.numel() * t.element_size() for t in (self.hq, self.hk, self.hv))
        self.d2h = self.hout.numel() * 4
        self.config = {"workload": self.name, "batch": self.B, "q_heads": self.Hq, "kv_heads": self.Hkv,
                       "head_dim": self.D, "page_size": self.P, "split_chunk": self.CHUNK,
                       "context": "U{1024..16384} seeded", "sum_context": int(self.lens.sum()),
                       "rope_theta": self.THETA, "kv_bytes_per_step": int(self.units_per_step),
                       "l2": "inputs larger than L2 (KV bytes per step >> 126 MB)", "sharding": "by sequence"}

    def step(self):
        q16 = self.be.rope_append_gqa(self.q, self.k, self.v, self.rope, self.pool, self.past)
        self.be.gqa_decode_paged(q16.view(self.B, self.Hq, self.D), self.pool, self.full, self.max_len, self.CHUNK,
                                 out=self.out)

    def step_e2e(self):
        self.q.copy_(self.hq, non_blocking=True)
        self.k.copy_(self.hk, non_blocking=True)
        self.v.copy_(self.hv, non_blocking=True)
        self.step()
        self.hout.copy_(self.out, non_blocking=True)

    # ---- CPU arm: the oracle on host arrays of the same shapes
    @staticmethod
    def cpu_sample(rank=0, max_sequences=32):
        from oracle import pyoracle as orc
        c = GqaDecodeB32
        lens = decode_lens(rank, c.B)[:max_sequences]
        pages = (lens + c.P - 1) // c.P
        num_pages = int(pages.sum()) + 8
        perm = np.random.RandomState(SEED + 9).permutation(num_pages).astype(np.int32)
        table = np.zeros((len(lens), int(pages.max())), np.int32)
        o = 0
        for b, n in enumerate(pages):
            table[b, :n] = perm[o:o + n]
            o += int(n)
        block = np.random.RandomState(SEED + 10).standard_normal(1 << 22).astype(np.float16).view(np.uint16)
        n_el = num_pages * c.Hkv * c.P * c.D
        kp = np.resize(block, n_el).reshape(num_pages, c.Hkv, c.P, c.D)
        vp = np.resize(block[::-1], n_el).reshape(num_pages, c.Hkv, c.P, c.D)
        q = orc.fill_normal((len(lens), 1, c.Hq, c.D), SEED + 11)
        k = orc.fill_normal((len(lens), 1, c.Hkv, c.D), SEED + 12)
        v = orc.fill_normal((len(lens), 1, c.Hkv, c.D), SEED + 13)
        inv = orc.default_inv_freq(c.THETA, 64)
        past = (lens - 1).astype(np.int32)
        units = float(lens.astype(np.int64).sum()) * c.Hkv * c.D * 2 * 2

        def run():
            qr = orc.qk_norm_rope(q, None, inv, 64, 0, positions=past)
            kr = orc.qk_norm_rope(k, None, inv, 64, 0, positions=past)
            return orc.gqa_paged_attention(qr, kr, v, None, kp, vp, table, past, c.P)

        return run, units, f"{len(lens)} of 32 sequences, all heads, full contexts"


WORKLOADS = {w.name: w for w in (GqaDecodeB32,)}
EXTRA_WORKLOADS: list = []  # measured in the same run and reported under "workloads"


# ----------------------------------------------------------------------------- measurement
def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def timed(torch, dist, world, fn, steps, warmup):
    """W warm-up steps, then K steps between barrier + synchronize, device time by CUDA events, max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def kernel_time(be, torch, wl, steps):
    """Average device time of the dominant kernel, from CUDA event pairs recorded around each launch."""
    be.device_profile_boundary(True)
    for _ in range(steps):
        wl.step()
    be.device_profile_boundary(False)
    ms, n = be.profile_read(wl.kernel)
    return (ms / n) if n else None, n


def cpu_baseline(wl_cls, budget_s=12.0):
    from oracle import pyoracle as orc
    run, units, sample = wl_cls.cpu_sample()
    t0 = time.perf_counter()
    run()
    first = time.perf_counter() - t0
    reps = max(1, min(8, int(budget_s / max(first, 1e-3)) - 1))
    best = first
    for _ in range(reps):
        t0 = time.perf_counter()
        run()
        best = min(best, time.perf_counter() - t0)
    scale = 1e-9 if wl_cls.unit == "GB/s" else 1e-12
    return {"value": units / best * scale, "unit": wl_cls.unit, "cores": orc.max_threads(), "kind": "port",
            "sample": sample, "seconds_per_pass": best}


def measure(be, torch, dist, world, rank, wl, steps, warmup, peaks, with_cpu, profile_steps=100):
    ms = timed(torch, dist, world, wl.step, steps, warmup)
    ms_e2e = timed(torch, dist, world, wl.step_e2e, steps, warmup)
    units = wl.units_per_step
    if world > 1:
        t = torch.tensor([units], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        total_units = float(t.item())
    else:
        total_units = units
    scale = 1e-9 if wl.unit == "GB/s" else 1e-12
    value = total_units * steps / (ms * 1e-3) * scale
    e2e = total_units * steps / (ms_e2e * 1e-3) * scale
    k_ms, k_n = kernel_time(be, torch, wl, profile_steps)
    peak = peaks["hbm_gbs"] if wl.bound == "hbm" else peaks["tflops"] * 1.0
    achieved = units / (k_ms * 1e-3) * scale if k_ms else None
    res = {"metric": wl.metric, "value": value, "unit": wl.unit, "ms_per_step": ms / steps,
           "e2e": {"value": e2e, "unit": wl.unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                   "ms_per_step": ms_e2e / steps},
           "roofline": {"bound": wl.bound, "achieved": achieved, "peak": peak,
                        "unit": "GB/s" if wl.bound == "hbm" else "TFLOP/s",
                        "frac": (achieved / peak) if achieved else None, "traffic": getattr(wl, "traffic", None),
                        "kernel": wl.kernel, "kernel_ms": k_ms, "kernel_launches_timed": k_n,
                        "peak_source": f"{peaks['source']} ({'copy bandwidth' if wl.bound == 'hbm' else 'cuBLAS bf16 burst'})"},
           "gpu_launches": wl.launches_per_step * steps, "config": wl.config}
    if with_cpu and rank == 0:
        res["cpu_baseline"] = cpu_baseline(type(wl))
    return res


def run_ours(args):
    import torch
    import torch.distributed as dist
    rank, local_rank, world = dist_env()
    if world > 1:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from inferno_b200 import CudaBackend
    be = CudaBackend(local_rank if world > 1 else 0)
    peaks = load_peaks()
    sampler = ClockSampler(local_rank if world > 1 else 0) if rank == 0 else None
    wl = WORKLOADS[args.workload](be, rank)
    head = measure(be, torch, dist, world, rank, wl, args.steps, args.warmup, peaks,
                   with_cpu=(world == 1 and not args.no_cpu), profile_steps=args.profile_steps)
    extras = []
    if not args.no_extras:
        for cls in EXTRA_WORKLOADS:
            if cls.name == args.workload:
                continue
            del wl
            torch.cuda.empty_cache()
            wl = cls(be, rank)
            extras.append(measure(be, torch, dist, world, rank, wl, min(args.steps, cls.max_steps), args.warmup, peaks,
                                  with_cpu=False, profile_steps=min(args.profile_steps, cls.max_steps)))
    be.device_flush()
    clocks = sampler.stop() if sampler else None
    if rank == 0:
        line = {"metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
                "data": "synthetic", "config": head["config"], "e2e": head["e2e"], "roofline": head["roofline"],
                "gpu_launches": head["gpu_launches"], "clocks": clocks}
        if "cpu_baseline" in head:
            line["cpu_baseline"] = head["cpu_baseline"]
        if extras:
            line["workloads"] = [{k: e[k] for k in ("metric", "value", "unit", "ms_per_step", "e2e", "roofline", "config")}
                                 for e in extras]
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    """The CPU arm: the oracle port on all host threads; rank 0 only."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    from oracle import pyoracle as orc
    cls = WORKLOADS[args.workload]
    run, units, sample = cls.cpu_sample()
    for _ in range(min(args.warmup, 1)):
        run()
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = time.perf_counter() - t0
    scale = 1e-9 if cls.unit == "GB/s" else 1e-12
    value = units * steps / dt * scale
    line = {"impl": "reference", "metric": cls.metric, "value": value, "unit": cls.unit, "n_gpus": world,
            "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": cls.name, "sample": sample,
                       "note": "reference is Rust + Metal and cannot be built here; this is the scalar CPU port of its kernels"},
            "cpu_baseline": {"value": value, "unit": cls.unit, "cores": orc.max_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="gqa_decode_b32", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg (profiler runs)")
    ap.add_argument("--profile-steps", type=int, default=100, help="launches timed per kernel for the roofline")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
