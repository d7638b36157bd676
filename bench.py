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

With N > 1 (torchrun, one rank per GPU) the headline shards by sequence with fixed work per GPU -- every rank
owns its own batch of 32 (the same 32 context lengths, its own pages), no data-path collective -- and `value` is
the sum over ranks divided by the slowest rank's time (weak scaling).  The same run also measures, under
"workloads", the strong-scaled forms of the path: the batch of 32 split 32/N sequences per rank (blocks balanced
by context length) with the [32, 48, 128] output gathered on every rank, and both prefills head-sharded with the
gather of the attention output inside the step.  The gather is fused into the kernels (their last stores go into
every rank's copy of the gathered tensor over NVLink, inf_comm_barrier ends the step); the same steps with the
library's NCCL all-gather (inf_allgather_heads) and with no exchange at all are timed beside it under
"collective".  torch.distributed only carries the rendezvous, the peer-memory handles, the barriers and the
reductions of the timings.

Every timed figure is the median of several regions of exactly K steps, each region bracketed by a barrier and a
synchronize on both sides and taken as the maximum over ranks.

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
    """Paged GQA decode, batch 32 (the third benchmark configuration).  Weak scaling: every rank owns its own batch
    of 32 (the same seeded context lengths on every rank, its own pages and values).  Strong scaling (`strong=True`): rank 0's batch of 32 is split into
    32/N sequences per rank and the [32, 48, 128] fp16 output is gathered on every rank: the combine kernel stores
    each row into every rank's copy (peer stores), and inf_comm_barrier ends the step."""
    name = "gqa_decode_b32"
    metric, unit, bound = "attn_decode_hbm_gbs", "GB/s", "hbm"
    kernel = "gqa_decode_partial_kernel"
    launches_per_step = 3  # rope+append, split-KV partial, combine
    traffic = 1.0320e9 + 15.5e6  # DRAM bytes read + written per launch of the full batch, from an ncu capture
    B, Hq, Hkv, D, P, CHUNK, THETA = 32, 48, 8, 128, 16, 512, 500000.0

    @classmethod
    def describe(cls, lens, strong=False):
        units = float(np.asarray(lens, np.int64).sum()) * cls.Hkv * cls.D * 2 * 2
        return {"workload": cls.name + ("_strong" if strong else ""), "batch": cls.B, "q_heads": cls.Hq,
                "kv_heads": cls.Hkv, "head_dim": cls.D, "page_size": cls.P, "split_chunk": cls.CHUNK,
                "context": "U{1024..16384} seeded", "sum_context": int(np.asarray(lens).sum()),
                "rope_theta": cls.THETA, "output": "fp16, fp32 accumulation", "kv_bytes_per_step": int(units),
                "l2": "inputs larger than L2 (KV bytes per step >> 126 MB)",
                "sharding": "by sequence, 32/N per rank in blocks balanced by context length, output gathered on every rank"
                            if strong else "by sequence"}

    def __init__(self, be, rank, world=1, strong=False, dist=None):
        import torch
        from inferno_b200.sharding import balanced_sequence_order, shard_sequences
        self.torch, self.be, self.world, self.strong = torch, be, world, strong
        # weak scaling keeps the work per GPU fixed: every rank draws the same 32 context lengths (its pages, page
        # order and values are its own)
        all_lens = decode_lens(0, self.B)
        if strong:
            # the batch is put in an order whose equal blocks hold about the same number of cached keys
            all_lens = all_lens[balanced_sequence_order(all_lens, world)]
            b0, b1 = shard_sequences(self.B, world, rank)
            assert self.B % world == 0, "the gather wants equal blocks"
            self.lens = all_lens[b0:b1]
            self.name = self.name + "_strong"
            self.scaling = "strong"
        else:
            self.lens = all_lens
        Bl = self.Bl = len(self.lens)
        pages = (self.lens + self.P - 1) // self.P
        self.num_pages = int(pages.sum()) + 64
        g = torch.Generator(device="cpu").manual_seed(SEED + 5 + rank)
        perm = torch.randperm(self.num_pages, generator=g).to(torch.int32)
        table = torch.full((Bl, int(pages.max())), 0, dtype=torch.int32)
        o = 0
        for b, n in enumerate(pages):
            table[b, :n] = perm[o:o + n]
            o += int(n)
        self.pool = be.prepare_kv_pool(self.num_pages, self.P, self.Hkv, self.D)
        gd = torch.Generator(device=be.device).manual_seed(SEED + 6 + rank)
        self.pool.k.normal_(0, 1, generator=gd)
        self.pool.v.normal_(0, 1, generator=gd)
        self.past = be.page_table(table, self.lens - 1, validate_on_host=False)
        self.table_full = be.page_table(table, self.lens, validate_on_host=False)
        inv = 1.0 / np.power(np.float32(self.THETA), (2 * np.arange(32)).astype(np.float32) / np.float32(64))
        self.rope = be.prepare_rope_table(inv.astype(np.float32), 64, 1.0)
        # q, k and v of a step are three views of one device buffer (and of one pinned host buffer), so that the
        # end-to-end step moves its inputs with a single host-to-device copy
        nq, nk = Bl * self.Hq * self.D, Bl * self.Hkv * self.D
        self.qkv = torch.randn((nq + 2 * nk,), generator=gd, device=be.device, dtype=torch.float16)
        self.q = self.qkv[:nq].view(Bl, 1, self.Hq, self.D)
        self.k = self.qkv[nq:nq + nk].view(Bl, 1, self.Hkv, self.D)
        self.v = self.qkv[nq + nk:].view(Bl, 1, self.Hkv, self.D)
        # fp16 output with fp32 accumulation: the precision the stated tolerance is written for
        self.out = torch.empty((Bl, self.Hq, self.D), dtype=torch.float16, device=be.device)
        self.hqkv = self.qkv.cpu().pin_memory()
        self.hq, self.hk, self.hv = self.hqkv[:nq], self.hqkv[nq:nq + nk], self.hqkv[nq + nk:]
        self.collective = strong and world > 1
        self.gather_bytes = self.out.numel() * 2 if self.collective else 0
        self.gathered = torch.empty((world, Bl, self.Hq, self.D), dtype=torch.float16, device=be.device) if self.collective else None
        if self.collective:
            self.exchange = "fused"   # "fused" (peer stores in the combine kernel), "nccl", "none"
            # two gathered outputs alternate: a peer may still read the one the previous step filled
            self.n_variants = 2
            self.full = [torch.zeros((self.B, self.Hq, self.D), dtype=torch.float16, device=be.device) for _ in range(2)]
            self.peers = [map_peers(be, dist, t) for t in self.full]
            use_fused_exchange(self, be)
            self.mine = [t[b0:b1] for t in self.full]
        result = self.gathered if self.collective else self.out
        self.hout = torch.empty(result.shape, dtype=torch.float16).pin_memory()
        self.max_len = int(self.lens.max())
        self.i = 0
        self.units_per_step = float(self.lens.astype(np.int64).sum()) * self.Hkv * self.D * 2 * 2  # KV bytes
        if strong:
            self.traffic = None
        self.h2d = sum(t.numel() * t.element_size() for t in (self.hq, self.hk, self.hv))
        self.d2h = self.hout.numel() * 2
        self.config = self.describe(all_lens, strong)

    def step(self):
        q16 = self.be.rope_append_gqa(self.q, self.k, self.v, self.rope, self.pool, self.past)
        self.i += 1
        if self.collective and self.exchange == "fused":
            self.result = self.full[self.i & 1]
            self.be.gqa_decode_paged(q16.view(self.Bl, self.Hq, self.D), self.pool, self.table_full, self.max_len,
                                     self.CHUNK, out=self.mine[self.i & 1], peers=self.peers[self.i & 1])
            self.be.comm_barrier()
            return
        self.be.gqa_decode_paged(q16.view(self.Bl, self.Hq, self.D), self.pool, self.table_full, self.max_len, self.CHUNK,
                                 out=self.out)
        self.result = self.out
        if self.collective and self.exchange == "nccl":
            self.be.allgather_into(self.out, self.gathered)
            self.result = self.gathered

    def step_e2e(self):
        self.qkv.copy_(self.hqkv, non_blocking=True)
        self.step()
        self.hout.view(-1).copy_(self.result.view(-1), non_blocking=True)

    # ---- CPU arm: the oracle on host arrays of the same shapes
    @classmethod
    def cpu_sample(cls, rank=0, max_sequences=32):
        from oracle import pyoracle as orc
        c = cls
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



class GqaDecodeB32Fp8(GqaDecodeB32):
    """The batch-32 decode configuration over FP8 E4M3FN pages: the same sequences, half the KV bytes.  The current
    token enters the softmax at full precision (its roped key and value travel beside the query); its FP8 copy is
    appended by the same fused kernel."""
    name = "gqa_decode_b32_fp8"
    metric = "attn_decode_fp8_hbm_gbs"
    kernel = "gqa_decode_partial_fp8_kernel"
    traffic = 516.2e6 + 14.7e6  # DRAM bytes read + written per launch, from an ncu capture
    KS, VS = 0.03, 0.03

    def __init__(self, be, rank, world=1):
        super().__init__(be, rank, world)
        torch = self.torch
        del self.pool
        torch.cuda.empty_cache()
        self.pool = be.prepare_kv_pool_fp8(self.num_pages, self.P, self.Hkv, self.KS, self.VS)
        gd = torch.Generator(device=be.device).manual_seed(SEED + 8 + rank)
        # bytes drawn uniformly from the codes below 0x78 in magnitude (finite values up to 240), both signs
        for t in (self.pool.k, self.pool.v):
            t.copy_(torch.randint(0, 0x78, t.shape, generator=gd, device=be.device, dtype=torch.uint8) |
                    (torch.randint(0, 2, t.shape, generator=gd, device=be.device, dtype=torch.uint8) << 7))
        self.cur_k = torch.empty((self.Bl, 1, self.Hkv, self.D), dtype=torch.float16, device=be.device)
        self.cur_v = torch.empty_like(self.cur_k)
        self.units_per_step = float(self.lens.astype(np.int64).sum()) * self.Hkv * self.D * 1 * 2  # KV bytes, one per value
        self.config = dict(self.config, workload=self.name, kv_dtype="fp8 e4m3fn, one scale per tensor",
                           kv_bytes_per_step=int(self.units_per_step))

    def step(self):
        q16, k16, v16 = self.be.rope_append_gqa_fp8(self.q, self.k, self.v, self.rope, self.pool, self.past,
                                                     cur_k=self.cur_k, cur_v=self.cur_v)
        self.be.gqa_decode_paged_fp8(q16.view(self.Bl, self.Hq, self.D), k16.view(self.Bl, self.Hkv, self.D),
                                     v16.view(self.Bl, self.Hkv, self.D), self.pool, self.past, self.max_len, self.CHUNK,
                                     out=self.out)
        self.result = self.out

    @classmethod
    def cpu_sample(cls, rank=0, max_sequences=32):
        from oracle import pyoracle as orc
        c = cls
        lens = decode_lens(rank, c.B)[:max_sequences]
        pages = (lens + c.P - 1) // c.P
        num_pages = int(pages.sum()) + 8
        perm = np.random.RandomState(SEED + 9).permutation(num_pages).astype(np.int32)
        table = np.zeros((len(lens), int(pages.max())), np.int32)
        o = 0
        for b, n in enumerate(pages):
            table[b, :n] = perm[o:o + n]
            o += int(n)
        n_el = num_pages * c.Hkv * c.P * c.D
        block = np.random.RandomState(SEED + 10).randint(0, 0x78, 1 << 22).astype(np.uint8)
        kp = np.resize(block, n_el).reshape(num_pages, c.Hkv, c.P, c.D)
        vp = np.resize(block[::-1], n_el).reshape(num_pages, c.Hkv, c.P, c.D)
        q = orc.fill_normal((len(lens), 1, c.Hq, c.D), SEED + 11)
        k = orc.fill_normal((len(lens), 1, c.Hkv, c.D), SEED + 12)
        v = orc.fill_normal((len(lens), 1, c.Hkv, c.D), SEED + 13)
        inv = orc.default_inv_freq(c.THETA, 64)
        past = (lens - 1).astype(np.int32)
        units = float(lens.astype(np.int64).sum()) * c.Hkv * c.D * 2

        def run():
            qr = orc.qk_norm_rope(q, None, inv, 64, 0, positions=past)
            kr = orc.qk_norm_rope(k, None, inv, 64, 0, positions=past)
            return orc.gqa_paged_attention_fp8(qr, kr, v, None, kp, vp, c.KS, c.VS, table, past, c.P)

        return run, units, f"{len(lens)} of 32 sequences, all heads, full contexts"


class GlmPagedDecode:
    """paged_decode_attention_resident_device at the GLM expanded layout: MHA decode, 64 heads, key and value dim
    256, 4095 cached keys + the current token, fp16 cache [pages][batch][heads][page][dim] in identity page order.
    No sharing between heads: 268 MB of K and V rows stream once."""
    name = "glm_paged_decode_4k"
    metric, unit, bound = "glm_paged_decode_hbm_gbs", "GB/s", "hbm"
    kernel = "glm_paged_decode_split_kernel"
    launches_per_step = 2
    traffic = 268.46e6 + 6.24e6  # DRAM bytes read + written per launch, from an ncu capture
    B, H, D, DV, P, PAST = 1, 64, 256, 256, 64, 4095
    max_steps = 200

    def __init__(self, be, rank):
        import torch
        self.torch, self.be = torch, be
        gd = torch.Generator(device=be.device).manual_seed(SEED + 61 + rank)
        pages = (self.PAST + self.P - 1) // self.P
        self.n_variants = 2  # two caches of 268 MB in rotation: more than L2
        self.pk = [torch.randn((pages, self.B, self.H, self.P, self.D), generator=gd, device=be.device, dtype=torch.float16)
                   for _ in range(2)]
        self.pv = [torch.randn((pages, self.B, self.H, self.P, self.DV), generator=gd, device=be.device, dtype=torch.float16)
                   for _ in range(2)]
        n = self.B * self.H
        self.inputs = torch.randn((n * (2 * self.D + self.DV),), generator=gd, device=be.device, dtype=torch.float32)
        self.q = self.inputs[:n * self.D].view(self.B, self.H, self.D)
        self.ck = self.inputs[n * self.D:2 * n * self.D].view(self.B, self.H, self.D)
        self.cv = self.inputs[2 * n * self.D:].view(self.B, self.H, self.DV)
        self.hinputs = self.inputs.cpu().pin_memory()
        self.out = None
        self.hout = torch.empty((self.B, self.H, self.DV), dtype=torch.float32).pin_memory()
        self.i = 0
        self.units_per_step = float(self.PAST) * self.B * self.H * (self.D + self.DV) * 2
        self.h2d, self.d2h = self.hinputs.numel() * 4, self.hout.numel() * 4
        self.config = {"workload": self.name, "batch": self.B, "heads": self.H, "head_dim": self.D, "value_dim": self.DV,
                       "cached_keys": self.PAST, "page_size": self.P, "kv_bytes_per_step": int(self.units_per_step),
                       "l2": "rotates through 2 caches (537 MB > L2)", "sharding": "replicas"}

    def step(self):
        v = self.i % 2
        self.i += 1
        self.out = self.be.paged_decode_attention_resident_device(self.q, self.pk[v], self.ck, self.pv[v], self.cv,
                                                                  self.PAST, self.P)

    def step_e2e(self):
        self.inputs.copy_(self.hinputs, non_blocking=True)
        self.step()
        self.hout.copy_(self.out, non_blocking=True)

    def cpu_sample(self):
        from oracle import pyoracle as orc
        rng = np.random.RandomState(SEED + 62)
        pages = (self.PAST + self.P - 1) // self.P
        blk = rng.standard_normal(1 << 22).astype(np.float16).view(np.uint16)
        pk = np.resize(blk, pages * self.B * self.H * self.P * self.D).reshape(pages, self.B, self.H, self.P, self.D)
        pv = np.resize(blk[::-1], pages * self.B * self.H * self.P * self.DV).reshape(pages, self.B, self.H, self.P, self.DV)
        q = rng.standard_normal((self.B, self.H, self.D)).astype(np.float32)
        ck = rng.standard_normal((self.B, self.H, self.D)).astype(np.float32)
        cv = rng.standard_normal((self.B, self.H, self.DV)).astype(np.float32)
        run = lambda: orc.paged_decode_mha_f16(q, pk, ck, pv, cv, self.PAST, self.P)
        return run, self.units_per_step, "whole workload (64 heads, 4095 cached keys)"


class MlaDecode:
    """Absorbed-MLA decode, batch 1, 64 heads over the paged 512+64 latent (second benchmark configuration)."""
    metric, unit, bound = "mla_decode_hbm_gbs", "GB/s", "hbm"
    kernel = "mla_decode_partial_kernel"
    launches_per_step = 3  # post-process + append, split partial, combine
    H, L, R, P = 64, 512, 64, 64
    max_steps = 400

    def __init__(self, be, rank, ctx_len):
        import torch
        self.torch, self.be, self.ctx_len = torch, be, ctx_len
        self.name = f"mla_decode_{ctx_len // 1024}k"
        # DRAM bytes per launch from ncu at 32k context; proportional to context
        self.traffic = (37.89e6 + 0.12e6) * ctx_len / 32768
        row_bytes = (self.L + self.R) * 2
        self.n_caches = max(2, int(np.ceil(320e6 / (ctx_len * row_bytes))))  # rotate through > L2 worth of caches
        pages_per = (ctx_len + self.P - 1) // self.P
        num_pages = self.n_caches * pages_per + 8
        g = torch.Generator(device="cpu").manual_seed(SEED + 21 + rank)
        perm = torch.randperm(num_pages, generator=g).to(torch.int32)
        self.pool = be.prepare_mla_pool(num_pages)
        gd = torch.Generator(device=be.device).manual_seed(SEED + 22 + rank)
        self.pool.rows.normal_(0, 0.5, generator=gd)
        self.tables = [be.page_table(perm[i * pages_per:(i + 1) * pages_per].view(1, -1), [ctx_len - 1],
                                     validate_on_host=False) for i in range(self.n_caches)]
        # the step's inputs (q fp16, the new token's f32 row) are views of one byte buffer on the device and of one
        # pinned buffer on the host: the end-to-end step moves them with a single copy
        q_bytes, x_bytes = self.H * (self.L + self.R) * 2, (self.L + self.R) * 4
        self.inputs = torch.empty((q_bytes + x_bytes,), dtype=torch.uint8, device=be.device)
        self.q = self.inputs[:q_bytes].view(torch.float16).view(1, 1, self.H, self.L + self.R)
        self.x = self.inputs[q_bytes:].view(torch.float32).view(1, 1, self.L + self.R)
        self.q.normal_(0, 1, generator=gd)
        self.x.normal_(0, 1, generator=gd)
        self.w = torch.ones((self.L,), device=be.device, dtype=torch.float32)
        self.out = torch.empty((1, 1, self.H, self.L), dtype=torch.float32, device=be.device)
        self.hinputs = self.inputs.cpu().pin_memory()
        self.hq = self.hinputs[:q_bytes].view(torch.float16).view(1, 1, self.H, self.L + self.R)
        self.hx = self.hinputs[q_bytes:].view(torch.float32).view(1, 1, self.L + self.R)
        self.hout = torch.empty(self.out.shape, dtype=torch.float32).pin_memory()
        self.scale = 1.0 / float(np.sqrt(192.0))
        self.i = 0
        self.n_variants = self.n_caches
        self.units_per_step = float(ctx_len) * row_bytes
        self.flops_per_step = 2.0 * self.H * (self.L + self.R + self.L) * ctx_len
        self.h2d = self.hq.numel() * 2 + self.hx.numel() * 4
        self.d2h = self.hout.numel() * 4
        self.config = self.describe(ctx_len)

    @classmethod
    def describe(cls, ctx_len):
        row_bytes = (cls.L + cls.R) * 2
        n_caches = max(2, int(np.ceil(320e6 / (ctx_len * row_bytes))))
        return {"workload": f"mla_decode_{ctx_len // 1024}k", "batch": 1, "heads": cls.H, "latent_dim": cls.L,
                "rope_dim": cls.R, "context": ctx_len, "page_size": cls.P, "kv_sigma": 0.5, "scale": "1/sqrt(192)",
                "kv_bytes_per_step": int(ctx_len * row_bytes),
                "flops_per_step": 2.0 * cls.H * (cls.L + cls.R + cls.L) * ctx_len,
                "l2": f"rotates through {n_caches} distinct caches ({n_caches * ctx_len * row_bytes / 1e6:.0f} MB > L2)",
                "sharding": "replicas"}

    def step(self):
        t = self.tables[self.i % self.n_caches]
        self.i += 1
        self.be.mla_kv_postprocess_device(self.x, self.w, 1e-6, 1.0e7, self.pool, t, want_outputs=False)
        self.be.mla_decode_absorbed(self.q, self.pool, t, self.ctx_len, self.scale, out=self.out)

    def step_e2e(self):
        self.inputs.copy_(self.hinputs, non_blocking=True)
        self.step()
        self.hout.copy_(self.out, non_blocking=True)

    def cpu_sample(self):
        from oracle import pyoracle as orc
        n, W = self.ctx_len, self.L + self.R
        table = np.random.RandomState(SEED + 23).permutation((n + self.P - 1) // self.P).astype(np.int32)[None]
        pool = np.resize(np.random.RandomState(SEED + 24).standard_normal(1 << 20).astype(np.float16).view(np.uint16),
                         table.size * self.P * W).reshape(-1, self.P, W)
        q = orc.fill_normal((1, 1, self.H, W), SEED + 25)
        cur = orc.fill_normal((1, 1, W), SEED + 26, 0.5)
        run = lambda: orc.mla_absorbed_paged(q, cur, pool, table, [n - 1], self.P, self.L, self.R, self.scale)
        return run, self.units_per_step, "whole workload (1 sequence, 64 heads, full context)"


class MlaAbsorbedDecode(MlaDecode):
    """q8_0_absorbed_mla_device as one call at the GLM decode shape (64 heads, q_no_rope 192, latent 512, value
    256): K_b Q8_0 matvec, append of the current row, absorbed MLA over the pages, V_b Q8_0 matvec.  The bytes
    that must move are the cached rows plus both weight matrices."""
    metric = "mla_absorbed_decode_hbm_gbs"
    launches_per_step = 6  # append, K_b matvec, rope pack, split partial, combine, V_b matvec
    QN, DV = 192, 256

    def __init__(self, be, rank, ctx_len):
        super().__init__(be, rank, ctx_len)
        torch = self.torch
        self.name = f"mla_absorbed_decode_{ctx_len // 1024}k"
        self.traffic = None
        gd = torch.Generator(device=be.device).manual_seed(SEED + 27 + rank)

        def q8(heads, fout, fin, scale):
            nblk = heads * fout * fin // 32
            blocks = torch.empty((nblk, 34), dtype=torch.uint8, device=be.device)
            sc = torch.full((nblk,), scale, dtype=torch.float16, device=be.device)
            blocks[:, :2] = sc.view(torch.uint8).view(nblk, 2)
            blocks[:, 2:] = torch.randint(0, 256, (nblk, 32), generator=gd, device=be.device, dtype=torch.uint8)
            return blocks.view(-1)
        self.k_b = q8(self.H, self.L, self.QN, 1.0e-3)
        self.v_b = q8(self.H, self.DV, self.L, 1.0e-3)
        # the four f32 inputs of the operator are views of one buffer (device and pinned host): one copy per step
        sizes = [self.H * self.QN, self.H * self.R, self.L, self.R]
        offs = np.concatenate([[0], np.cumsum(sizes)]).tolist()
        self.inputs_f32 = torch.randn((offs[-1],), generator=gd, device=be.device, dtype=torch.float32)
        self.inputs_f32[offs[2]:] *= 0.5
        self.hinputs_f32 = self.inputs_f32.cpu().pin_memory()
        shapes = [(1, 1, self.H, self.QN), (1, 1, self.H, self.R), (1, 1, self.L), (1, 1, self.R)]
        self.q_no, self.q_rope, self.cur_lat, self.cur_rope = (
            self.inputs_f32[offs[i]:offs[i + 1]].view(shapes[i]) for i in range(4))
        self.hqn, self.hqr, self.hcl, self.hcr = (
            self.hinputs_f32[offs[i]:offs[i + 1]].view(shapes[i]) for i in range(4))
        self.hout = torch.empty((1, 1, self.H, self.DV), dtype=torch.float32).pin_memory()
        self.weight_bytes = self.k_b.numel() + self.v_b.numel()
        self.kernel_units_per_launch = self.units_per_step  # the attention kernel itself moves only the cached rows
        self.units_per_step += self.weight_bytes
        self.flops_per_step += 2.0 * self.H * self.L * (self.QN + self.DV)
        self.h2d = 4 * (self.hqn.numel() + self.hqr.numel() + self.hcl.numel() + self.hcr.numel())
        self.d2h = self.hout.numel() * 4
        self.config.update({"workload": self.name, "q_no_rope_dim": self.QN, "value_dim": self.DV,
                            "weights": "Q8_0 K_b [64][512][192] + V_b [64][256][512]",
                            "weight_bytes_per_step": int(self.weight_bytes), "flops_per_step": self.flops_per_step,
                            "bytes_per_step": int(self.units_per_step)})
        self.out = torch.empty((1, 1, self.H, self.DV), dtype=torch.float32, device=be.device)

    def step(self):
        t = self.tables[self.i % self.n_caches]
        self.i += 1
        self.be.q8_0_absorbed_mla_device(self.k_b, self.v_b, self.q_no, self.q_rope, self.cur_lat, self.cur_rope,
                                         self.pool, t, self.QN + self.R, self.DV, max_len=self.ctx_len, out=self.out)

    def step_e2e(self):
        self.inputs_f32.copy_(self.hinputs_f32, non_blocking=True)
        self.step()
        self.hout.copy_(self.out, non_blocking=True)

    def cpu_sample(self):
        from oracle import pyoracle as orc
        n, W = self.ctx_len, self.L + self.R
        table = np.random.RandomState(SEED + 23).permutation((n + self.P - 1) // self.P).astype(np.int32)[None]
        pool = np.resize(np.random.RandomState(SEED + 24).standard_normal(1 << 20).astype(np.float16).view(np.uint16),
                         table.size * self.P * W).reshape(-1, self.P, W)
        k_b, v_b = self.k_b.cpu().numpy(), self.v_b.cpu().numpy()
        q_no = orc.fill_normal((1, self.H, self.QN), SEED + 28, 1.0, False)
        q_rope = orc.fill_normal((1, 1, self.H, self.R), SEED + 29, 1.0, False)
        cur = orc.fill_normal((1, 1, W), SEED + 26, 0.5)

        def run():
            q_lat = orc.q8_0_heads_matvec(k_b, q_no, self.H, self.QN, self.L).reshape(1, 1, self.H, self.L)
            q = np.concatenate([q_lat, q_rope], axis=-1)
            ctx = orc.mla_absorbed_paged(q, cur, pool, table, [n - 1], self.P, self.L, self.R, self.scale)
            return orc.q8_0_heads_matvec(v_b, ctx.reshape(1, self.H, self.L), self.H, self.L, self.DV)
        return run, self.units_per_step, "whole workload (1 sequence, 64 heads, full context, both projections)"


class MlaSelectedDecode(MlaDecode):
    """DSA sparse decode, attention step: absorbed MLA over 2048 selected rows (seeded choice, newest row always
    kept) of a 32 768-row paged latent cache, the gather fused into the kernel.  Only the selected rows move."""
    metric = "mla_selected_decode_hbm_gbs"
    N_SEL = 2048

    def __init__(self, be, rank, ctx_len):
        super().__init__(be, rank, ctx_len)
        torch = self.torch
        self.name = f"mla_selected_decode_{self.N_SEL}_of_{ctx_len // 1024}k"
        self.traffic = 2.51e6 if (self.N_SEL, ctx_len) == (2048, 32768) else None  # ncu
        g = torch.Generator(device="cpu").manual_seed(SEED + 31 + rank)
        ids = torch.randperm(ctx_len - 1, generator=g)[: self.N_SEL - 1].sort().values.to(torch.int32)
        self.sel = torch.cat([ids, torch.tensor([ctx_len - 1], dtype=torch.int32)]).view(1, -1).to(be.device)
        self.counts = torch.tensor([self.N_SEL], dtype=torch.int32, device=be.device)
        row_bytes = (self.L + self.R) * 2
        self.units_per_step = float(self.N_SEL) * row_bytes
        self.flops_per_step = 2.0 * self.H * (self.L + self.R + self.L) * self.N_SEL
        self.config.update({"workload": self.name, "selected_rows": self.N_SEL, "kv_bytes_per_step": int(self.units_per_step),
                            "flops_per_step": self.flops_per_step})

    def step(self):
        t = self.tables[self.i % self.n_caches]
        self.i += 1
        self.be.mla_kv_postprocess_device(self.x, self.w, 1e-6, 1.0e7, self.pool, t, want_outputs=False)
        self.be.mla_decode_absorbed_selected(self.q, self.pool, t, self.sel, self.counts, self.scale, out=self.out)

    def cpu_sample(self):
        from oracle import pyoracle as orc
        n, W = self.N_SEL, self.L + self.R  # the oracle runs on the gathered rows, as the reference does
        table = np.arange((n + self.P - 1) // self.P, dtype=np.int32)[None]
        pool = np.resize(np.random.RandomState(SEED + 24).standard_normal(1 << 20).astype(np.float16).view(np.uint16),
                         table.size * self.P * W).reshape(-1, self.P, W)
        q = orc.fill_normal((1, 1, self.H, W), SEED + 25)
        cur = orc.fill_normal((1, 1, W), SEED + 26, 0.5)
        run = lambda: orc.mla_absorbed_paged(q, cur, pool, table, [n - 1], self.P, self.L, self.R, self.scale)
        return run, self.units_per_step, "whole workload (2048 gathered rows, 64 heads)"


class DsaSparseDecode(MlaSelectedDecode):
    """One DSA sparse decode step: index scores over all 32 768 cached tokens (32 index heads x 128), top-2048,
    absorbed MLA over the selected rows.  Bytes that must move: the f32 index keys plus the selected latent rows."""
    metric = "dsa_sparse_decode_hbm_gbs"
    kernel = "dsa_scores_kernel"
    launches_per_step = 5  # append, scores, top-k, split partial, combine
    HI, DI = 32, 128

    def __init__(self, be, rank, ctx_len):
        super().__init__(be, rank, ctx_len)
        torch = self.torch
        self.name = f"dsa_sparse_decode_{ctx_len // 1024}k"
        gd = torch.Generator(device=be.device).manual_seed(SEED + 33 + rank)
        self.n_key_sets = 8  # 8 x 16.8 MB of index keys > L2
        self.idx_keys = [torch.randn((1, ctx_len - 1, self.DI), generator=gd, device=be.device, dtype=torch.float32)
                         for _ in range(self.n_key_sets)]
        self.idx_cur = torch.randn((1, self.DI), generator=gd, device=be.device, dtype=torch.float32)
        self.idx_q = torch.randn((1, self.HI, self.DI), generator=gd, device=be.device, dtype=torch.float32)
        self.idx_w = torch.rand((1, self.HI), generator=gd, device=be.device, dtype=torch.float32)
        self.scores = torch.empty((1, ctx_len), dtype=torch.float32, device=be.device)
        self.ids = torch.empty((1, self.N_SEL), dtype=torch.int32, device=be.device)
        self.n_variants = max(self.n_caches, self.n_key_sets)
        self.key_bytes = float(ctx_len) * self.DI * 4
        self.kernel_units_per_launch = self.key_bytes
        self.traffic = 16.83e6 * ctx_len / 32768  # DRAM bytes read by the scores kernel, from an ncu capture
        self.units_per_step = self.key_bytes + float(self.N_SEL) * (self.L + self.R) * 2
        self.flops_per_step += 2.0 * self.HI * self.DI * ctx_len
        self.config.update({"workload": self.name, "index_heads": self.HI, "index_dim": self.DI,
                            "index_key_bytes_per_step": int(self.key_bytes), "bytes_per_step": int(self.units_per_step),
                            "flops_per_step": self.flops_per_step,
                            "l2": f"rotates through {self.n_key_sets} index-key sets ({self.n_key_sets * self.key_bytes / 1e6:.0f} MB > L2)"})

    def step(self):
        t = self.tables[self.i % self.n_caches]
        keys = self.idx_keys[self.i % self.n_key_sets]
        self.i += 1
        self.be.mla_kv_postprocess_device(self.x, self.w, 1e-6, 1.0e7, self.pool, t, want_outputs=False)
        self.be.dsa_scores(self.idx_q, self.idx_w, keys, self.idx_cur, out=self.scores)
        self.be.dsa_topk(self.scores, self.N_SEL, out=self.ids)
        self.be.mla_decode_absorbed_selected(self.q, self.pool, t, self.ids, self.counts, self.scale, out=self.out)

    def cpu_sample(self):
        from oracle import pyoracle as orc
        run_attn, _, _ = super().cpu_sample()
        q = orc.fill_normal((1, self.HI, self.DI), SEED + 34, 1.0, False)
        w = np.abs(orc.fill_normal((1, self.HI), SEED + 35, 1.0, False))
        pk = orc.fill_normal((1, self.ctx_len - 1, self.DI), SEED + 36, 1.0, False)
        ck = orc.fill_normal((1, self.DI), SEED + 37, 1.0, False)

        def run():
            sc = orc.dsa_scores(q, w, pk, ck)
            orc.dsa_topk(sc, self.N_SEL)
            return run_attn()
        return run, self.units_per_step, "whole step (numpy index scores and top-k, oracle attention over 2048 rows)"


class GqaPrefill2k:
    """Causal GQA prefill, one 2048-token prompt, 48 q / 8 kv heads, fused RoPE + KV-append (fourth configuration).
    With N > 1 ranks the heads are sharded (48/N query heads with their 8/N KV heads per rank) and the output is
    all-gathered through the library's collective: strong scaling."""
    name = "gqa_prefill_2k"
    metric, unit, bound = "gqa_prefill_tflops", "TFLOP/s", "tensor"
    kernel = "flash_prefill_gqa_kernel"
    launches_per_step = 2  # rope+append, flash prefill
    traffic = 33.64e6 + 0.35e6  # DRAM bytes per launch, from an ncu capture
    T, Hq, Hkv, D, P, THETA = 2048, 48, 8, 128, 16, 500000.0
    max_steps = 400
    N_SETS = 8
    scaling = "strong"

    @classmethod
    def describe(cls, world=1):
        set_mb = (cls.T * (cls.Hq + 2 * cls.Hkv) // world * cls.D * 2 * 2) / 1e6
        return {"workload": cls.name, "tokens": cls.T, "q_heads": cls.Hq, "kv_heads": cls.Hkv,
                "head_dim": cls.D, "page_size": cls.P, "rope_theta": cls.THETA, "causal": True,
                "flops_per_step": 4.0 * cls.D * cls.Hq * cls.T * (cls.T + 1) / 2,
                "append_bytes_per_step": cls.T * cls.Hkv * cls.D * 2 * 2,
                "l2": f"rotates through {cls.N_SETS} distinct input sets and pools ({cls.N_SETS * set_mb:.0f} MB)",
                "sharding": "heads" if world > 1 else "none",
                "collective": "all-gather of the output fused into the kernel's epilogue (peer stores over NVLink) + barrier"
                              if world > 1 else None}

    def __init__(self, be, rank, world=1, dist=None):
        import torch
        self.torch, self.be, self.world = torch, be, world
        self.hq_local, self.hkv_local = self.Hq // world, self.Hkv // world
        pages = self.T // self.P
        gd = torch.Generator(device=be.device).manual_seed(SEED + 31 + rank)
        inv = 1.0 / np.power(np.float32(self.THETA), (2 * np.arange(32)).astype(np.float32) / np.float32(64))
        self.rope = be.prepare_rope_table(inv.astype(np.float32), 64, 1.0)
        self.sets = []
        for i in range(self.N_SETS):  # distinct inputs and pools per iteration: more than L2 in rotation
            pool = be.prepare_kv_pool(pages + 4, self.P, self.hkv_local, self.D)
            perm = torch.randperm(pages + 4, generator=torch.Generator().manual_seed(SEED + 32 + i)).to(torch.int32)
            table = be.page_table(perm[:pages].view(1, -1), [0], validate_on_host=False)
            q = torch.randn((1, self.T, self.hq_local, self.D), generator=gd, device=be.device, dtype=torch.float16)
            k = torch.randn((1, self.T, self.hkv_local, self.D), generator=gd, device=be.device, dtype=torch.float16)
            v = torch.randn((1, self.T, self.hkv_local, self.D), generator=gd, device=be.device, dtype=torch.float16)
            self.sets.append((pool, table, q, k, v))
        self.out = torch.empty((1, self.T, self.hq_local, self.D), dtype=torch.float16, device=be.device)
        self.collective = world > 1
        self.gather_bytes = self.out.numel() * 2 if world > 1 else 0
        self.gathered = torch.empty((world, self.T, self.hq_local, self.D), dtype=torch.float16, device=be.device) if world > 1 else None
        self.exchange = "fused"   # how the heads get to every rank: "fused" (peer stores in the epilogue), "nccl", "none"
        if world > 1:
            self.full = [torch.zeros((1, self.T, self.Hq, self.D), dtype=torch.float16, device=be.device) for _ in range(2)]
            self.peers = [map_peers(be, dist, t) for t in self.full]
            use_fused_exchange(self, be)
            self.mine = [t[:, :, rank * self.hq_local:(rank + 1) * self.hq_local] for t in self.full]
        q, k, v = self.sets[0][2:]
        self.hq, self.hk, self.hv = q.cpu().pin_memory(), k.cpu().pin_memory(), v.cpu().pin_memory()
        self.hout = torch.empty((self.gathered if world > 1 else self.out).shape, dtype=torch.float16).pin_memory()
        self.i = 0
        self.n_variants = self.N_SETS
        total_flops = 4.0 * self.D * self.Hq * self.T * (self.T + 1) / 2
        self.units_per_step = total_flops / world  # per rank; summed over ranks by the harness
        self.h2d = sum(t.numel() * 2 for t in (self.hq, self.hk, self.hv))
        self.d2h = self.hout.numel() * 2
        self.config = self.describe(world)
        if world == 1:
            self._init_overlap(gd)

    def step(self):
        pool, table, q, k, v = self.sets[self.i % self.N_SETS]
        self.i += 1
        q16 = self.be.rope_append_gqa(q, k, v, self.rope, pool, table)
        if self.collective and self.exchange == "fused":
            # the two gathered tensors alternate: a peer may still read the one the previous step filled
            self.result = self.full[self.i & 1]
            self.be.gqa_prefill_paged(q16, pool, table, out=self.mine[self.i & 1], peers=self.peers[self.i & 1])
            self.be.comm_barrier()
            return
        self.be.gqa_prefill_paged(q16, pool, table, out=self.out)
        self.result = self.out
        if self.collective and self.exchange == "nccl":
            self.be.allgather_into(self.out, self.gathered)
            self.result = self.gathered

    def step_e2e(self):
        pool, table, q, k, v = self.sets[self.i % self.N_SETS]  # the same set step() is about to use
        q.copy_(self.hq, non_blocking=True)
        k.copy_(self.hk, non_blocking=True)
        v.copy_(self.hv, non_blocking=True)
        self.step()
        self.hout.view(-1).copy_(self.result.view(-1), non_blocking=True)

    # ---- the same end-to-end step, head group by head group: every KV head with its six query heads has its own
    # host buffers, device buffers and pool, so that the upload of group g + 1 and the download of group g - 1 run
    # under the kernels of group g (three streams; the host layout is group-major)
    def _init_overlap(self, gd):
        torch, be = self.torch, self.be
        self.overlap_groups = self.Hkv
        grp, pages = self.Hq // self.Hkv, self.T // self.P
        self.ov = []
        for g in range(self.overlap_groups):
            pool = be.prepare_kv_pool(pages + 4, self.P, 1, self.D)
            perm = torch.randperm(pages + 4, generator=torch.Generator().manual_seed(SEED + 52 + g)).to(torch.int32)
            table = be.page_table(perm[:pages].view(1, -1), [0], validate_on_host=False)
            n_q, n_kv = self.T * grp * self.D, self.T * self.D
            dev = torch.randn((n_q + 2 * n_kv,), generator=gd, device=be.device, dtype=torch.float16)
            host = dev.cpu().pin_memory()
            out = torch.empty((1, self.T, grp, self.D), dtype=torch.float16, device=be.device)
            self.ov.append({"pool": pool, "table": table, "dev": dev, "host": host, "out": out,
                            "q": dev[:n_q].view(1, self.T, grp, self.D), "k": dev[n_q:n_q + n_kv].view(1, self.T, 1, self.D),
                            "v": dev[n_q + n_kv:].view(1, self.T, 1, self.D),
                            "hout": torch.empty(out.shape, dtype=torch.float16).pin_memory(),
                            "up": torch.cuda.Event(), "done": torch.cuda.Event()})
        self.s_up, self.s_down = torch.cuda.Stream(be.device), torch.cuda.Stream(be.device)

    def step_e2e_overlapped(self):
        torch = self.torch
        cur = torch.cuda.current_stream(self.be.device)
        self.s_up.wait_stream(cur)
        for o in self.ov:
            with torch.cuda.stream(self.s_up):
                o["dev"].copy_(o["host"], non_blocking=True)
                o["up"].record(self.s_up)
        for o in self.ov:
            cur.wait_event(o["up"])
            q16 = self.be.rope_append_gqa(o["q"], o["k"], o["v"], self.rope, o["pool"], o["table"])
            self.be.gqa_prefill_paged(q16, o["pool"], o["table"], out=o["out"])
            o["done"].record(cur)
            self.s_down.wait_event(o["done"])
            with torch.cuda.stream(self.s_down):
                o["hout"].copy_(o["out"], non_blocking=True)
        cur.wait_stream(self.s_up)
        cur.wait_stream(self.s_down)

    @classmethod
    def cpu_sample(cls):
        from oracle import pyoracle as orc
        c = cls
        q = orc.fill_normal((1, c.T, c.Hq, c.D), SEED + 33)
        k = orc.fill_normal((1, c.T, c.Hkv, c.D), SEED + 34)
        v = orc.fill_normal((1, c.T, c.Hkv, c.D), SEED + 35)
        inv = orc.default_inv_freq(c.THETA, 64)
        pages = c.T // c.P
        table = np.random.RandomState(SEED + 36).permutation(pages).astype(np.int32)[None]
        kp = np.zeros((pages, c.Hkv, c.P, c.D), np.uint16)
        vp = np.zeros_like(kp)

        def run():
            qr = orc.qk_norm_rope(q, None, inv, 64, 0)
            kr = orc.qk_norm_rope(k, None, inv, 64, 0)
            return orc.gqa_paged_attention(qr, kr, v, None, kp, vp, table, [0], c.P)

        return run, 4.0 * c.D * c.Hq * c.T * (c.T + 1) / 2, "whole workload (2048 tokens, 48 heads)"


class MlaPrefill32k:
    """Causal MLA prefill, 32768-token prompt, 64 heads, qk 128+64, v 128 (fifth configuration).  With N > 1
    ranks the heads are sharded 64/N per rank and the [32768, 64, 128] output is all-gathered through the
    library's collective."""
    name = "mla_prefill_32k"
    metric, unit, bound = "mla_prefill_tflops", "TFLOP/s", "tensor"
    kernel = "flash_prefill_mla_kernel"
    launches_per_step = 1
    traffic = None  # set per prompt length in __init__, from an ncu capture at 8192 tokens
    T, H = 32768, 64
    max_steps = 3
    max_regions = 5
    scaling = "strong"

    @classmethod
    def describe(cls, world=1, tokens=None):
        T = tokens or cls.T
        return {"workload": cls.name if T == cls.T else f"mla_prefill_{T}", "tokens": T, "heads": cls.H, "qk_dim": 192,
                "v_dim": 128, "causal": True, "flops_per_step": T * (T + 1) / 2 * cls.H * 2.0 * (192 + 128),
                "l2": "inputs larger than L2 (2.4 GB of Q/K/V)" if T == cls.T else "inputs of this prompt length",
                "sharding": "heads" if world > 1 else "none",
                "collective": "all-gather of the output fused into the kernel's epilogue (peer stores over NVLink) + barrier"
                              if world > 1 else None}

    def __init__(self, be, rank, world=1, dist=None):
        import torch
        self.torch, self.be, self.world = torch, be, world
        hl = self.H // world
        self.hl = hl
        gd = torch.Generator(device=be.device).manual_seed(SEED + 41 + rank)
        self.q = torch.randn((self.T, hl, 192), generator=gd, device=be.device, dtype=torch.float16)
        self.kn = torch.randn((self.T, hl, 128), generator=gd, device=be.device, dtype=torch.float16)
        self.kr = torch.randn((self.T, 64), generator=gd, device=be.device, dtype=torch.float16)
        self.v = torch.randn((self.T, hl, 128), generator=gd, device=be.device, dtype=torch.float16)
        self.out = torch.empty((self.T, hl, 128), dtype=torch.float16, device=be.device)
        self.collective = world > 1
        self.gather_bytes = self.out.numel() * 2 if world > 1 else 0
        self.gathered = torch.empty((world, self.T, hl, 128), dtype=torch.float16, device=be.device) if world > 1 else None
        self.exchange = "fused"   # "fused" (peer stores in the epilogue), "nccl", "none"
        if world > 1:
            self.full = [torch.zeros((self.T, self.H, 128), dtype=torch.float16, device=be.device) for _ in range(2)]
            self.peers = [map_peers(be, dist, t) for t in self.full]
            use_fused_exchange(self, be)
            self.mine = [t[:, rank * hl:(rank + 1) * hl] for t in self.full]
        self.host = [t.cpu().pin_memory() for t in (self.q, self.kn, self.kr, self.v)]
        self.hout = torch.empty((self.gathered if world > 1 else self.out).shape, dtype=torch.float16).pin_memory()
        self.scale = 1.0 / float(np.sqrt(192.0))
        # DRAM bytes per launch from an ncu capture at 8 192 tokens (518.2 MB read, 126.1 MB written): with the work
        # items ordered by head group the inputs cross HBM about once, so traffic grows with the prompt length
        self.traffic = (518.2e6 + 126.1e6) * self.T / 8192 / world
        total_flops = self.T * (self.T + 1) / 2 * self.H * 2.0 * (192 + 128)
        self.units_per_step = total_flops / world
        self.h2d = sum(t.numel() * 2 for t in self.host)
        self.d2h = self.hout.numel() * 2
        self.i = 0
        self.config = self.describe(world, self.T)
        if world == 1:
            self._init_overlap(gd)

    def step(self):
        self.i += 1
        if self.collective and self.exchange == "fused":
            # the two gathered tensors alternate: a peer may still read the one the previous step filled
            self.result = self.full[self.i & 1]
            self.be.causal_sequence_attention_device(self.q, self.kn, self.kr, self.v, self.scale, out=self.mine[self.i & 1],
                                                     peers=self.peers[self.i & 1])
            self.be.comm_barrier()
            return
        self.be.causal_sequence_attention_device(self.q, self.kn, self.kr, self.v, self.scale, out=self.out)
        self.result = self.out
        if self.collective and self.exchange == "nccl":
            self.be.allgather_into(self.out, self.gathered)
            self.result = self.gathered

    def step_e2e(self):
        for d, h in zip((self.q, self.kn, self.kr, self.v), self.host):
            d.copy_(h, non_blocking=True)
        self.step()
        self.hout.view(-1).copy_(self.result.view(-1), non_blocking=True)

    # ---- the same end-to-end step in groups of eight heads with a group-major host layout: the upload of group
    # g + 1 and the download of group g - 1 run under the kernel of group g (three streams)
    def _init_overlap(self, gd):
        torch, be = self.torch, self.be
        self.overlap_groups = G = 8
        hg = self.hl // G
        self.ov = []
        for g in range(G):
            dev = [torch.randn((self.T, hg, d), generator=gd, device=be.device, dtype=torch.float16) for d in (192, 128, 128)]
            out = torch.empty((self.T, hg, 128), dtype=torch.float16, device=be.device)
            self.ov.append({"dev": dev, "host": [t.cpu().pin_memory() for t in dev], "out": out,
                            "hout": torch.empty(out.shape, dtype=torch.float16).pin_memory(),
                            "up": torch.cuda.Event(), "done": torch.cuda.Event()})
        self.s_up, self.s_down = torch.cuda.Stream(be.device), torch.cuda.Stream(be.device)

    def step_e2e_overlapped(self):
        torch = self.torch
        cur = torch.cuda.current_stream(self.be.device)
        self.s_up.wait_stream(cur)
        with torch.cuda.stream(self.s_up):
            self.kr.copy_(self.host[2], non_blocking=True)  # the rope tail every head shares goes up first
        for o in self.ov:
            with torch.cuda.stream(self.s_up):
                for d, h in zip(o["dev"], o["host"]):
                    d.copy_(h, non_blocking=True)
                o["up"].record(self.s_up)
        for o in self.ov:
            cur.wait_event(o["up"])
            q, kn, v = o["dev"]
            self.be.causal_sequence_attention_device(q, kn, self.kr, v, self.scale, out=o["out"])
            o["done"].record(cur)
            self.s_down.wait_event(o["done"])
            with torch.cuda.stream(self.s_down):
                o["hout"].copy_(o["out"], non_blocking=True)
        cur.wait_stream(self.s_up)
        cur.wait_stream(self.s_down)

    @classmethod
    def cpu_sample(cls):
        from oracle import pyoracle as orc
        scale = 1.0 / float(np.sqrt(192.0))
        T, H = cls.T, 8  # 8 of the 64 heads, 48 sampled rows with their full causal key ranges
        rows = np.sort(np.random.RandomState(SEED + 42).randint(0, T, size=48)).astype(np.int32)
        blk = np.random.RandomState(SEED + 43).standard_normal(1 << 22).astype(np.float16).astype(np.float32)
        q = np.resize(blk, T * H * 192).reshape(T, H, 192)
        kn = np.resize(blk[::-1], T * H * 128).reshape(T, H, 128)
        kr = np.resize(blk[7:], T * 64).reshape(T, 64)
        v = np.resize(blk[13:], T * H * 128).reshape(T, H, 128)
        flops = float(np.sum(rows.astype(np.int64) + 1)) * H * 2.0 * (192 + 128)
        run = lambda: orc.causal_mha(q, kn, kr, v, scale, rows=rows)
        return run, flops, "48 sampled query rows x 8 of 64 heads, full causal key ranges (sampled)"


def map_peers(be, dist, tensor):
    """Every rank exports `tensor` (its copy of a gathered output) and maps the other ranks' copies: the device
    addresses, in rank order without this rank, that the fused gather stores into.  torch.distributed only carries
    the 72-byte handles.  None on every rank when any rank could not map a peer (no peer access between the GPUs):
    the workload then gathers with the library's NCCL collective instead."""
    import torch
    world, rank = dist.get_world_size(), dist.get_rank()
    handles = [None] * world
    mapped, ok = None, 1
    try:
        dist.all_gather_object(handles, be.peer_export(tensor))
        mapped = [be.peer_open(handles[r]) for r in range(world) if r != rank]
    except Exception as e:  # InfernoError from the export / open calls
        sys.stderr.write(f"rank {rank}: peer mapping failed ({e}); gathering with NCCL\n")
        ok = 0
    agreed = torch.tensor([ok], dtype=torch.int32, device="cuda")
    dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
    return mapped if int(agreed.item()) == 1 else None


def use_fused_exchange(wl, be):
    """Called by the sharded workloads after map_peers: falls back to the NCCL gather when the peers are not mapped."""
    if any(p is None for p in wl.peers) or not wl.peers:
        wl.exchange = "nccl"
        wl.fused_ok = False
    else:
        wl.exchange = "fused"
        wl.fused_ok = True


def make_workload(name, be, rank, world=1, tokens=0, dist=None):
    if name == "gqa_decode_b32":
        return GqaDecodeB32(be, rank, world)
    if name == "gqa_decode_b32_strong":
        return GqaDecodeB32(be, rank, world, strong=True, dist=dist)
    if name == "gqa_decode_b32_fp8":
        return GqaDecodeB32Fp8(be, rank, world)
    if name == "glm_paged_decode_4k":
        return GlmPagedDecode(be, rank)
    if name == "mla_decode_4k":
        return MlaDecode(be, rank, 4096)
    if name == "mla_decode_32k":
        return MlaDecode(be, rank, 32768)
    if name == "dsa_sparse_decode_32k":
        return DsaSparseDecode(be, rank, 32768)
    if name == "mla_selected_decode_32k":
        return MlaSelectedDecode(be, rank, 32768)
    if name == "mla_absorbed_decode_32k":
        return MlaAbsorbedDecode(be, rank, 32768)
    if name == "gqa_prefill_2k":
        return GqaPrefill2k(be, rank, world, dist)
    if name == "mla_prefill_32k":
        wl = MlaPrefill32k.__new__(MlaPrefill32k)
        if tokens:
            wl.T = tokens  # smaller prompt for profiler captures; the name in `config` reflects it
            wl.max_steps = 50
        wl.__init__(be, rank, world, dist)
        return wl
    raise KeyError(name)


WORKLOAD_NAMES = ["gqa_decode_b32", "gqa_decode_b32_fp8", "glm_paged_decode_4k", "mla_decode_4k", "mla_decode_32k", "mla_absorbed_decode_32k", "mla_selected_decode_32k",
                  "dsa_sparse_decode_32k", "gqa_prefill_2k", "mla_prefill_32k", "gqa_decode_b32_strong"]
# head-sharded (or sequence-split) with an all-gather: strong scaling, the collective inside the step
STRONG = {"gqa_prefill_2k", "mla_prefill_32k", "gqa_decode_b32_strong"}
# what a multi-GPU run measures besides the weak-scaled headline: the sharded forms of the path
MULTI_GPU_EXTRAS = ["gqa_decode_b32_strong", "gqa_prefill_2k", "mla_prefill_32k"]
SINGLE_GPU_EXTRAS = [n for n in WORKLOAD_NAMES if n != "gqa_decode_b32_strong"]


# ----------------------------------------------------------------------------- measurement
def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


class GraphedStep:
    """A workload step captured into CUDA graphs, one per input set the workload rotates through, so that a
    launch-bound step costs one driver call instead of one per kernel."""

    def __init__(self, be, wl, fn_name):
        self.n = getattr(wl, "n_variants", 1)
        self.graphs = []
        for v in range(self.n):
            wl.i = v
            self.graphs.append(be.capture_graph(getattr(wl, fn_name)))
        self.k = 0

    def __call__(self):
        self.graphs[self.k % self.n].replay()
        self.k += 1


def timed(torch, dist, world, fn, steps, warmup, regions=1):
    """W warm-up steps, then `regions` regions of exactly K steps, each between barrier + synchronize, device time
    by CUDA events.  Returns (median over regions of the max over ranks, per-rank medians, all region maxima)."""
    if world > 1:
        # the ranks enter the warm-up together: a step that ends in the peer-flag barrier waits at most two seconds
        torch.cuda.synchronize()
        dist.barrier()
    for _ in range(warmup):
        fn()
    mine = []
    for _ in range(regions):
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
        mine.append(a.elapsed_time(b))
    if world > 1:
        t = torch.tensor(mine, dtype=torch.float64, device="cuda")
        every = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        table = torch.stack(every).cpu().numpy()  # [rank][region]
    else:
        table = np.array([mine], dtype=np.float64)
    region_max = table.max(axis=0)
    return float(np.median(region_max)), [float(x) for x in np.median(table, axis=1)], [float(x) for x in region_max]


def spread(values):
    return {"min": float(min(values)), "median": float(statistics.median(values)), "max": float(max(values))}


def kernel_time(be, torch, wl, steps):
    """Average device time of the dominant kernel, from CUDA event pairs recorded around each launch."""
    be.device_profile_boundary(True)
    for _ in range(steps):
        # keep the stream busy while the host enqueues the step, so that the event pair around a kernel brackets its
        # device time and not the host's launch latency
        torch.cuda._sleep(400000)
        wl.step()
    be.device_profile_boundary(False)
    ms, n = be.profile_read(wl.kernel)
    return (ms / n) if n else None, n


def cpu_baseline(wl, budget_s=12.0):
    """The oracle (a scalar port of the reference kernels) on all host threads, on a bounded sample."""
    from oracle import pyoracle as orc
    orc.use_all_host_threads()
    run, units, sample = wl.cpu_sample()
    t0 = time.perf_counter()
    run()
    first = time.perf_counter() - t0
    reps = max(0, min(6, int(budget_s / max(first, 1e-3)) - 1))
    best = first
    for _ in range(reps):
        t0 = time.perf_counter()
        run()
        best = min(best, time.perf_counter() - t0)
    scale = 1e-9 if wl.unit == "GB/s" else 1e-12
    return {"value": units / best * scale, "unit": wl.unit, "cores": orc.max_threads(), "kind": "port",
            "sample": sample, "seconds_per_pass": best}


def measure(be, torch, dist, world, rank, wl, steps, warmup, peaks, with_cpu, profile_steps=100, use_graph=True,
            regions=10):
    steps = max(1, min(steps, getattr(wl, "max_steps", steps)))
    profile_steps = max(1, min(profile_steps, getattr(wl, "max_steps", profile_steps)))
    regions = max(1, min(regions, getattr(wl, "max_regions", regions)))
    if use_graph:
        for _ in range(2):
            wl.step()
            wl.step_e2e()
        step, step_e2e = GraphedStep(be, wl, "step"), GraphedStep(be, wl, "step_e2e")
    else:
        step, step_e2e = wl.step, wl.step_e2e
    ms, rank_ms, region_ms = timed(torch, dist, world, step, steps, warmup, regions)
    ms_e2e, _, _ = timed(torch, dist, world, step_e2e, steps, warmup, regions)
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
    peak = peaks["hbm_gbs"] if wl.bound == "hbm" else peaks["tflops"]
    k_units = getattr(wl, "kernel_units_per_launch", units)  # algorithmic units of the dominant kernel's launch
    achieved = k_units / (k_ms * 1e-3) * scale if k_ms else None
    roof = {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": "GB/s" if wl.bound == "hbm" else "TFLOP/s",
            "frac": (achieved / peak) if achieved else None, "traffic": getattr(wl, "traffic", None),
            "traffic_source": "ncu capture of this kernel (dram__bytes_read.sum + dram__bytes_write.sum), not measured by this run"
                              if getattr(wl, "traffic", None) else None,
            "kernel": wl.kernel, "kernel_ms": k_ms, "kernel_launches_timed": k_n,
            "peak_source": f"{peaks['source']} ({'copy bandwidth' if wl.bound == 'hbm' else 'cuBLAS bf16 burst'})"}
    if wl.bound == "hbm" and hasattr(wl, "flops_per_step") and k_ms:
        roof["tensor_tflops"] = wl.flops_per_step / (k_ms * 1e-3) * 1e-12
        roof["tensor_frac_of_burst_peak"] = roof["tensor_tflops"] / peaks["tflops"]
    if wl.bound == "tensor" and achieved and peaks.get("tflops_sustained"):
        roof["frac_of_sustained_peak"] = achieved / peaks["tflops_sustained"]
    res = {"metric": wl.metric, "value": value, "unit": wl.unit, "steps": steps, "ms_per_step": ms / steps,
           "regions": regions, "region_ms_per_step": spread([r / steps for r in region_ms]),
           "e2e": {"value": e2e, "unit": wl.unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                   "ms_per_step": ms_e2e / steps},
           "roofline": roof, "gpu_launches": wl.launches_per_step * steps * regions, "config": wl.config,
           "launch": "cuda graph replay (one per input set)" if use_graph else "eager",
           "scaling": getattr(wl, "scaling", "weak")}
    if getattr(wl, "overlap_groups", 0):
        # the same end-to-end step with the copies of one head group running under the kernels of its neighbours
        for _ in range(2):
            wl.step_e2e_overlapped()
        ms_ov, _, _ = timed(torch, dist, world, wl.step_e2e_overlapped, steps, warmup, regions)
        res["e2e_overlapped"] = {"value": total_units * steps / (ms_ov * 1e-3) * scale, "unit": wl.unit,
                                 "ms_per_step": ms_ov / steps, "head_groups": wl.overlap_groups,
                                 "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h, "launch": "eager, three streams"}
    if world > 1:
        # what every rank saw: its own median region time and its own kernel time
        kt = torch.tensor([k_ms or 0.0], dtype=torch.float64, device="cuda")
        every = [torch.empty_like(kt) for _ in range(world)]
        dist.all_gather(every, kt)
        res["per_rank"] = {"ms_per_step": spread([r / steps for r in rank_ms]),
                           "kernel_ms": spread([float(x.item()) for x in every])}
        if getattr(wl, "gather_bytes", 0):
            def eager_ms(mode):
                if hasattr(wl, "exchange"):
                    wl.exchange = mode
                else:
                    wl.collective = mode != "none"
                t_ms, _, _ = timed(torch, dist, world, wl.step, steps, warmup, regions)
                return t_ms / steps
            coll = {"bytes_sent_per_rank_to_each_peer": wl.gather_bytes,
                    "bytes_received_per_rank": wl.gather_bytes * (world - 1)}
            if hasattr(wl, "exchange"):
                coll["what"] = ("the step's last kernel stores its output into every rank's gathered tensor (peer stores "
                                "over NVLink, tile by tile) and the step ends with inf_comm_barrier; beside it, the same "
                                "step with inf_allgather_heads (NCCL) after the kernel, and with no exchange at all")
                coll["barrier"] = "peer-flag kernel" if be.comm_barrier_is_p2p() else "nccl all-reduce"
                fused_ok = getattr(wl, "fused_ok", True)
                if fused_ok:
                    coll["ms_per_step_fused_gather"] = eager_ms("fused")
                else:
                    coll["fused_gather"] = "unavailable: the peers' memory could not be mapped; the step gathers with NCCL"
                coll["ms_per_step_nccl_allgather"] = eager_ms("nccl")
                coll["ms_per_step_without"] = eager_ms("none")
                wl.exchange = "fused" if fused_ok else "nccl"
                if fused_ok:
                    coll["ms_exchange_fused"] = coll["ms_per_step_fused_gather"] - coll["ms_per_step_without"]
                coll["ms_exchange_nccl"] = coll["ms_per_step_nccl_allgather"] - coll["ms_per_step_without"]
            else:
                coll["what"] = "inf_allgather_heads (NCCL all-gather behind the C ABI) after the kernels"
                coll["ms_per_step_with"] = eager_ms("nccl")
                coll["ms_per_step_without"] = eager_ms("none")
                wl.collective = True
                coll["ms_collective"] = coll["ms_per_step_with"] - coll["ms_per_step_without"]
            res["collective"] = coll
    if with_cpu and rank == 0:
        res["cpu_baseline"] = cpu_baseline(wl)
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
    if world > 1:
        # the library's own communicator: rank 0 makes the id, torch.distributed only carries it to the others
        box = [be.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        be.comm_init(box[0], rank, world)
    peaks = load_peaks()
    sampler = ClockSampler(local_rank if world > 1 else 0) if rank == 0 else None
    wl = make_workload(args.workload, be, rank, world, args.tokens, dist)
    graph_ok = lambda name: not args.no_graph and not (world > 1 and name in STRONG)  # steps with NCCL stay eager
    head = measure(be, torch, dist, world, rank, wl, args.steps, args.warmup, peaks,
                   with_cpu=(world == 1 and not args.no_cpu), profile_steps=args.profile_steps,
                   use_graph=graph_ok(args.workload), regions=args.regions)
    extras = []
    if not args.no_extras:
        names = MULTI_GPU_EXTRAS if world > 1 else SINGLE_GPU_EXTRAS
        for name in names:
            if name == args.workload:
                continue
            del wl
            torch.cuda.empty_cache()
            wl = make_workload(name, be, rank, world, 0, dist)
            extras.append(measure(be, torch, dist, world, rank, wl, args.steps, args.warmup, peaks,
                                  with_cpu=(world == 1 and not args.no_cpu), profile_steps=args.profile_steps,
                                  use_graph=graph_ok(name), regions=args.regions))
    be.device_flush()
    clocks = sampler.stop() if sampler else None
    if rank == 0:
        line = {"metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": world,
                "steps": head["steps"], "warmup": args.warmup, "ms_per_step": head["ms_per_step"],
                "higher_is_better": True, "scaling": head["scaling"],
                "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": head["config"],
                "e2e": head["e2e"], "roofline": head["roofline"], "gpu_launches": head["gpu_launches"],
                "clocks": clocks}
        for k in ("regions", "region_ms_per_step", "launch", "per_rank", "collective", "e2e_overlapped", "cpu_baseline"):
            if k in head:
                line[k] = head[k]
        if extras:
            keys = ("metric", "value", "unit", "steps", "ms_per_step", "regions", "region_ms_per_step", "scaling", "e2e",
                    "e2e_overlapped", "roofline", "gpu_launches", "config", "launch", "per_rank", "collective",
                    "cpu_baseline")
            line["workloads"] = [{k: e[k] for k in keys if k in e} for e in extras]
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        be.comm_destroy()
        dist.destroy_process_group()


def run_reference(args):
    """The CPU arm: the oracle port on all host threads; rank 0 only, the other ranks exit at once.  One step is
    one pass of the oracle over the bounded sample its `cpu_baseline.sample` names."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    from oracle import pyoracle as orc
    cores = orc.use_all_host_threads()  # the same thread count at every N: a launcher's OMP_NUM_THREADS=1 does not apply
    name = args.workload
    if name in ("gqa_decode_b32", "gqa_decode_b32_strong"):
        cls, config = GqaDecodeB32, GqaDecodeB32.describe(decode_lens(0), name.endswith("strong"))
        run, units, sample = cls.cpu_sample()
    elif name in ("mla_decode_4k", "mla_decode_32k"):
        cls = MlaDecode
        wl = cls.__new__(cls)  # no device set-up: only the shape constants and cpu_sample() are used
        wl.ctx_len = 4096 if name.endswith("4k") else 32768
        wl.scale = 1.0 / float(np.sqrt(192.0))
        wl.units_per_step = float(wl.ctx_len) * (wl.L + wl.R) * 2
        config = cls.describe(wl.ctx_len)
        run, units, sample = wl.cpu_sample()
    elif name == "gqa_prefill_2k":
        cls, config = GqaPrefill2k, GqaPrefill2k.describe(world)
        run, units, sample = cls.cpu_sample()
    elif name == "mla_prefill_32k":
        cls, config = MlaPrefill32k, MlaPrefill32k.describe(world)
        run, units, sample = cls.cpu_sample()
    else:
        print(json.dumps({"impl": "reference", "unavailable": f"no CPU arm for workload {name}"}), flush=True)
        return
    for _ in range(args.warmup):
        run()
    steps = args.steps
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = time.perf_counter() - t0
    scale = 1e-9 if cls.unit == "GB/s" else 1e-12
    value = units * steps / dt * scale
    line = {"impl": "reference", "metric": cls.metric, "value": value, "unit": cls.unit, "n_gpus": world,
            "steps": steps, "warmup": args.warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
            "scaling": "strong" if name in STRONG else "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config,
            "note": "the reference is Rust + Metal and cannot be built here; this is the scalar CPU port of its kernels",
            "cpu_baseline": {"value": value, "unit": cls.unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="gqa_decode_b32", choices=WORKLOAD_NAMES)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="only the selected workload")
    ap.add_argument("--regions", type=int, default=10, help="timed regions of K steps each; the median is reported")
    ap.add_argument("--tokens", type=int, default=0, help="prompt length override for mla_prefill_32k (profiler captures)")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly instead of replaying CUDA graphs")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg (profiler runs)")
    ap.add_argument("--profile-steps", type=int, default=100, help="launches timed per kernel for the roofline")
    args = ap.parse_args()
    if args.impl == "reference":
        # one oracle pass over the sample takes 0.3-2 s: bound the run to a couple of minutes whatever K and W say
        args.steps, args.warmup = max(1, min(args.steps, 40)), max(0, min(args.warmup, 5))
        run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        run_ours(args)


if __name__ == "__main__":
    main()
