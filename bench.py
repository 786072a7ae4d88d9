#!/usr/bin/env python3
"""Benchmark of the TurboQuant hot paths on B200: packed paged decode attention and KV compression.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg3|cfg2|cfg4|cfg5] [--impl reference]

Default workload (cfg3): turbo3 batched decode, batch 64 x 8192 tokens, 64 query / 8 KV heads, head_dim 128,
block 16, random block table over a shared pool, fp16 K/V ~ N(0,1) with 4 outlier channels x10 per head, the
cache written by the CUDA compress kernel, one decode step per layer over 62 layers with independent caches.
A "step" is one pass over the 62 layers.  Inputs are synthetic (seeded).  With --gpus N (launched under
torch.distributed.run) the 8 KV heads are split over the ranks; there is no data-path collective.

Prints ONE JSON line: metric = decode HBM GB/s (algorithmic packed bytes / device time, all ranks),
plus us/layer, tokens/s, compress GB/s, roofline, cpu_baseline, e2e, clocks.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "turboquant-amd_b200"), ROOT):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402
import torch  # noqa: E402

OUTLIER_CHANNELS = [5, 50, 90, 127]

WORKLOADS = {
    # name: (format, batch, q heads, kv heads, layers, description)
    "cfg2": dict(fmt="turbo4", batch=1, hq=32, hkv=8, layers=1, lens="fixed:4096", sparse=0.0,
                 desc="turbo4 single sequence, ctx 4096, 32q/8kv heads (latency-bound)"),
    "cfg3": dict(fmt="turbo3", batch=64, hq=64, hkv=8, layers=62, lens="fixed:8192", sparse=0.0,
                 desc="turbo3 batched decode, batch 64 x 8192, 64q/8kv heads, 62 layers"),
    "cfg4": dict(fmt="turbo3", batch=64, hq=64, hkv=8, layers=4, lens="uniform:16384:32768", sparse=1e-6,
                 desc="turbo3 Sparse-V, batch 64, lengths U[16384,32768], 64q/8kv heads"),
    "cfg5": dict(fmt="turbo2", batch=256, hq=32, hkv=8, layers=4, lens="lognormal:4096:1.0:128:65536", sparse=0.0,
                 desc="turbo2 mixed-length decode, batch 256, lognormal lengths, 32q/8kv heads"),
}


def make_lengths(spec: str, batch: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    kind, *a = spec.split(":")
    if kind == "fixed":
        return torch.full((batch,), int(a[0]), dtype=torch.int32)
    if kind == "uniform":
        return torch.randint(int(a[0]), int(a[1]) + 1, (batch,), generator=g, dtype=torch.int32)
    if kind == "lognormal":
        z = torch.randn(batch, generator=g) * float(a[1]) + math.log(float(a[0]))
        return z.exp().clamp(float(a[2]), float(a[3])).to(torch.int32)
    raise ValueError(spec)


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# Workload construction (per rank: its share of the KV heads)
# ------------------------------------------------------------------------------------------------
class Workload:
    def __init__(self, name: str, rank: int, world: int, device: torch.device, layers_override: int | None = None):
        from turboquant.kernels.paged import CacheFormat, Codebooks
        w = WORKLOADS[name]
        self.name, self.spec = name, w
        self.device = device
        self.fmt = CacheFormat.named(w["fmt"])
        self.books = Codebooks(self.fmt, device)
        self.block_size = 16
        self.batch = w["batch"]
        if w["hkv"] % world:
            raise SystemExit(f"--gpus {world} must divide the {w['hkv']} KV heads")
        self.hkv = w["hkv"] // world            # this rank's KV heads
        self.hq = w["hq"] // world
        self.layers = layers_override or w["layers"]
        self.sparse = w["sparse"]
        self.lens = make_lengths(w["lens"], self.batch, seed=1234)
        self.pages = (self.lens + 15) // 16
        self.max_blocks = int(self.pages.max())
        self.num_blocks = int(self.pages.sum())
        self.tok_heads_rank = int(self.lens.sum()) * self.hkv
        self.tok_heads_total = int(self.lens.sum()) * w["hkv"]
        self.bytes_per_tok_head = self.fmt.page_bytes / 16
        g = torch.Generator().manual_seed(99)
        perm = torch.randperm(self.num_blocks, generator=g).to(torch.int32)     # shared pool, random placement
        bt = torch.zeros(self.batch, self.max_blocks, dtype=torch.int32)
        o = 0
        for s in range(self.batch):
            n = int(self.pages[s])
            bt[s, :n] = perm[o:o + n]
            o += n
        self.block_tables = bt.to(device)
        self.seq_lens = self.lens.to(device)
        self.rank, self.world = rank, world
        self.caches: list[torch.Tensor] = []
        self.compress_ms: list[float] = []
        self.compress_bytes = 0

    def build_caches(self):
        """Generate K/V sequence by sequence (bounded temporaries) and compress them into each layer's cache."""
        from turboquant.kernels.paged import allocate_cache, compress_and_scatter
        dev = self.device
        bs = self.block_size
        for layer in range(self.layers):
            cache = allocate_cache(self.num_blocks, bs, self.hkv, self.fmt, dev)
            g = torch.Generator(device=dev).manual_seed(1000 * layer + 17 * self.rank + 1)
            # chunks of sequences so that fp16 K + V temporaries stay under ~2.2 GB
            per_tok = self.hkv * 128 * 2 * 2
            group, acc, groups = [], 0, []
            for s in range(self.batch):
                if acc + int(self.lens[s]) * per_tok > (2200 << 20) and group:
                    groups.append(group)
                    group, acc = [], 0
                group.append(s)
                acc += int(self.lens[s]) * per_tok
            groups.append(group)
            t_layer, b_layer = 0.0, 0
            for grp in groups:
                T = int(self.lens[grp].sum())
                K = torch.randn(T, self.hkv, 128, generator=g, device=dev, dtype=torch.float16)
                V = torch.randn(T, self.hkv, 128, generator=g, device=dev, dtype=torch.float16)
                K[..., OUTLIER_CHANNELS] *= 10
                V[..., OUTLIER_CHANNELS] *= 10
                slots = torch.cat([(self.block_tables[s, :int(self.pages[s])].long().repeat_interleave(bs)[:int(self.lens[s])] * bs
                                    + torch.arange(int(self.lens[s]), device=dev) % bs) for s in grp])
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                compress_and_scatter(K, V, cache, slots, self.books, bs)
                e1.record()
                e1.synchronize()
                t_layer += e0.elapsed_time(e1)
                b_layer += T * self.hkv * (2 * 128 * 2 + self.bytes_per_tok_head)
                del K, V, slots
            self.caches.append(cache)
            self.compress_ms.append(t_layer)
            self.compress_bytes = b_layer

    def make_queries(self, seed: int) -> torch.Tensor:
        g = torch.Generator().manual_seed(seed + 31 * self.rank)
        return torch.randn(self.layers, self.batch, self.hq, 128, generator=g).half()
