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
QUERY_PUSH = 8.0

WORKLOADS = {
    # name: (format, batch, q heads, kv heads, layers, description)
    "cfg2": dict(fmt="turbo4", batch=1, hq=32, hkv=8, layers=1, lens="fixed:4096", sparse=0.0,
                 desc="turbo4 single sequence, ctx 4096, 32q/8kv heads (latency-bound)"),
    "cfg3": dict(fmt="turbo3", batch=64, hq=64, hkv=8, layers=62, lens="fixed:8192", sparse=0.0,
                 desc="turbo3 batched decode, batch 64 x 8192, 64q/8kv heads, 62 layers"),
    "cfg4": dict(fmt="turbo3", batch=64, hq=64, hkv=8, layers=4, lens="uniform:16384:32768", sparse=1e-6,
                 desc="turbo3 Sparse-V, batch 64, lengths U[16384,32768], 64q/8kv heads"),
    "cfg4s": dict(fmt="turbo3", batch=64, hq=64, hkv=8, layers=4, lens="uniform:16384:32768", sparse=1e-6, bias=30.0,
                  desc="cfg4 with a sharper softmax: +30 logit bias on 2% of the 16-token pages (labelled variant; "
                       "with +6 on 2% of positions no page of any sequence falls under the 1e-6 threshold)"),
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


def shard_heads(hq: int, hkv: int, rank: int, world: int):
    """KV heads [lo, hi) and query heads [qlo, qhi) owned by `rank`: contiguous head-major slices, no overlap."""
    if hkv % world:
        raise SystemExit(f"--gpus {world} must divide the {hkv} KV heads")
    per = hkv // world
    g = hq // hkv
    return per * rank, per * (rank + 1), g * per * rank, g * per * (rank + 1)


def make_block_tables(pages: torch.Tensor, seed: int = 99) -> torch.Tensor:
    """Random placement of every sequence's pages in one shared pool (identical on every rank)."""
    num_blocks = int(pages.sum())
    perm = torch.randperm(num_blocks, generator=torch.Generator().manual_seed(seed)).to(torch.int32)
    bt = torch.zeros(len(pages), int(pages.max()), dtype=torch.int32)
    o = 0
    for s in range(len(pages)):
        n = int(pages[s])
        bt[s, :n] = perm[o:o + n]
        o += n
    return bt


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
        lo, hi, qlo, qhi = shard_heads(w["hq"], w["hkv"], rank, world)
        self.hkv = hi - lo                      # this rank's KV heads
        self.hq = qhi - qlo
        self.layers = layers_override or w["layers"]
        self.sparse = w["sparse"]
        self.lens = make_lengths(w["lens"], self.batch, seed=1234)
        self.pages = (self.lens + 15) // 16
        self.max_blocks = int(self.pages.max())
        self.num_blocks = int(self.pages.sum())
        self.tok_heads_rank = int(self.lens.sum()) * self.hkv
        self.tok_heads_total = int(self.lens.sum()) * w["hkv"]
        self.bytes_per_tok_head = self.fmt.page_bytes / 16
        self.block_tables = make_block_tables(self.pages).to(device)
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
                if self.spec.get("bias"):
                    # The reference API has no logit-bias argument, so the bias lives in the data: the queries of
                    # a sequence share a component of size QUERY_PUSH along a per-sequence direction u, and the
                    # keys of the hot pages get bias * sqrt(128) / QUERY_PUSH along u.
                    o = 0
                    for s_ in grp:
                        n = int(self.lens[s_])
                        hot = self.hot_pages(s_)
                        tok = (hot[:, None] * 16 + torch.arange(16)).reshape(-1)
                        tok = tok[tok < n].to(dev)
                        u = self.direction(s_).to(dev)
                        K[o + tok] += (self.spec["bias"] * math.sqrt(128) / QUERY_PUSH * u).half()
                        o += n
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
        if self.layers < 4 and len(groups) == 1:
            # too few layers for a warm sample: time the same compression again into a scratch cache
            scratch = allocate_cache(self.num_blocks, bs, self.hkv, self.fmt, dev)
            T = int(self.lens.sum())
            K = torch.randn(T, self.hkv, 128, device=dev, dtype=torch.float16)
            V = torch.randn(T, self.hkv, 128, device=dev, dtype=torch.float16)
            slots = torch.cat([(self.block_tables[s, :int(self.pages[s])].long().repeat_interleave(bs)[:int(self.lens[s])] * bs
                                + torch.arange(int(self.lens[s]), device=dev) % bs) for s in range(self.batch)])
            for _ in range(8):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                compress_and_scatter(K, V, scratch, slots, self.books, bs)
                e1.record()
                e1.synchronize()
                self.compress_ms.append(e0.elapsed_time(e1))
            del scratch, K, V

    def direction(self, s: int) -> torch.Tensor:
        u = torch.randn(128, generator=torch.Generator().manual_seed(7000 + s))
        return u / u.norm()

    def hot_pages(self, s: int) -> torch.Tensor:
        n = int(self.pages[s])
        k = max(1, n // 50)
        return torch.randperm(n, generator=torch.Generator().manual_seed(9000 + s))[:k]

    def make_queries(self, seed: int) -> torch.Tensor:
        """Queries in rotated space (the decode kernel's input); biased workloads push them along H u."""
        g = torch.Generator().manual_seed(seed + 31 * self.rank)
        q = torch.randn(self.layers, self.batch, self.hq, 128, generator=g)
        if self.spec.get("bias"):
            from turboquant.core.rotation import make_wht_matrix
            H = make_wht_matrix(128)
            for s in range(self.batch):
                q[:, s] += QUERY_PUSH * (self.direction(s) @ H)
        return q.half()


# ------------------------------------------------------------------------------------------------
# Timed loops
# ------------------------------------------------------------------------------------------------
DECODE_FLAGS = 0      # set from --decode-kernel: IO_TCGEN05 selects the tensor-memory variant of the decode kernel


def decode_layers(wl: Workload, q_dev: torch.Tensor, outs: torch.Tensor, stats=None):
    """One step: one decode launch pair (partial + merge) per layer, device-resident inputs."""
    from turboquant.kernels import _native
    f = wl.fmt
    sm, cs = 1.0 / math.sqrt(128), math.sqrt(math.pi / 2) / 128
    for layer in range(wl.layers):
        _native._decode_paged_impl(outs[layer], q_dev[layer], None, wl.caches[layer], wl.block_tables, wl.seq_lens,
                                   wl.books.kc, wl.books.vc, sm, cs, wl.sparse, wl.block_size, f.k_bits, f.v_bits,
                                   f.use_qjl, 0, skip_stats=stats, io_flags=DECODE_FLAGS)


def time_device_steps(wl: Workload, steps: int, warmup: int, dist_barrier):
    """value leg: q already rotated and resident in HBM; CUDA events around exactly `steps` steps."""
    dev = wl.device
    q_dev = wl.make_queries(7).to(dev)
    outs = torch.empty_like(q_dev)
    stats = torch.zeros(2, dtype=torch.int32, device=dev) if wl.sparse > 0 else None
    decode_layers(wl, q_dev, outs, stats)          # sizes the cached workspace before anything is captured
    torch.cuda.synchronize()
    # One step (all layers) is captured once in a CUDA graph and replayed: the launcher library allocates
    # nothing and does not synchronise, so the captured work is exactly the eager work without launch gaps.
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        decode_layers(wl, q_dev, outs, stats)
    for _ in range(warmup):
        graph.replay()
    if stats is not None:
        stats.zero_()
    torch.cuda.synchronize()
    dist_barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    dist_barrier()
    ms = e0.elapsed_time(e1)
    skip = None
    if stats is not None:
        seen, skipped = stats.cpu().tolist()
        skip = {"v_pages_seen": seen, "v_pages_skipped": skipped, "fraction": (skipped / seen if seen else 0.0)}
    time_device_steps.last_queries = q_dev
    return ms, skip, outs


def time_e2e_steps(wl: Workload, steps: int, warmup: int, dist_barrier):
    """e2e leg: per layer, the step's inputs come from pinned host memory (the query and the new token's
    K/V for every sequence), the new K/V is compressed into the cache at the last position, the query is
    rotated, attention runs, the output is de-rotated and copied back to pinned host memory."""
    from turboquant.kernels.paged import compress_and_scatter, paged_decode_attention
    dev = wl.device
    g = torch.Generator().manual_seed(5 + wl.rank)
    q_host = torch.randn(wl.layers, wl.batch, wl.hq, 128, generator=g).half().pin_memory()
    k_host = torch.randn(wl.layers, wl.batch, wl.hkv, 128, generator=g).half().pin_memory()
    v_host = torch.randn(wl.layers, wl.batch, wl.hkv, 128, generator=g).half().pin_memory()
    out_host = torch.empty(wl.layers, wl.batch, wl.hq, 128, dtype=torch.float16).pin_memory()
    # Double-buffered: a copy-in stream, the compute stream and a copy-out stream, as an engine would overlap
    # the transfers of neighbouring layers with attention.  Every byte still crosses PCIe inside the timed region.
    q_dev = [torch.empty(wl.batch, wl.hq, 128, dtype=torch.float16, device=dev) for _ in range(2)]
    k_dev = [torch.empty(wl.batch, wl.hkv, 128, dtype=torch.float16, device=dev) for _ in range(2)]
    v_dev = [torch.empty_like(k_dev[0]) for _ in range(2)]
    o_dev = [torch.empty_like(q_dev[0]) for _ in range(2)]
    last = (wl.lens - 1).long()
    slots = (wl.block_tables.cpu()[torch.arange(wl.batch), (last // 16)].long() * 16 + last % 16).to(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_ready = [torch.cuda.Event() for _ in range(2)]
    out_free = [torch.cuda.Event() for _ in range(2)]

    def step():
        main = torch.cuda.current_stream(dev)
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        for layer in range(wl.layers):
            b = layer & 1
            with torch.cuda.stream(s_in):
                if layer >= 2:
                    s_in.wait_event(in_free[b])
                q_dev[b].copy_(q_host[layer], non_blocking=True)
                k_dev[b].copy_(k_host[layer], non_blocking=True)
                v_dev[b].copy_(v_host[layer], non_blocking=True)
                # the new token is compressed into this layer's cache behind the previous layer's attention
                compress_and_scatter(k_dev[b], v_dev[b], wl.caches[layer], slots, wl.books, wl.block_size)
                in_ready[b].record(s_in)
            main.wait_event(in_ready[b])
            if layer >= 2:
                main.wait_event(out_free[b])
            paged_decode_attention(q_dev[b], wl.caches[layer], wl.block_tables, wl.seq_lens, wl.books, wl.block_size,
                                   sparse_thresh=wl.sparse, rotate_q=True, derotate_out=True, out=o_dev[b])
            in_free[b].record(main)
            out_ready[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(out_ready[b])
                out_host[layer].copy_(o_dev[b], non_blocking=True)
                out_free[b].record(s_out)
        main.wait_stream(s_in)
        main.wait_stream(s_out)

    step()                                         # eager once: sizes the cached workspaces
    torch.cuda.synchronize()
    # The whole step - copies on their streams included - is captured once and replayed, as a serving engine
    # replays its decode step: the pinned host buffers are read and written again by every replay.
    run, how = step, "eager launches"
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        run, how = graph.replay, "one CUDA graph per step"
    except Exception as exc:                        # capture not possible here: time the eager step
        print(f"bench: e2e step not captured ({type(exc).__name__}: {exc}); timing eager launches", file=sys.stderr)
        torch.cuda.synchronize()
    for _ in range(warmup):
        run()
    torch.cuda.synchronize()
    dist_barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    dist_barrier()
    h2d = wl.layers * (q_host[0].numel() + 2 * k_host[0].numel()) * 2
    d2h = wl.layers * out_host[0].numel() * 2
    return e0.elapsed_time(e1), h2d, d2h, how


def parity_slice(wl: "Workload", outs: torch.Tensor, q_dev: torch.Tensor, layer: int = 0, seq: int = 3, kvh: int = 0):
    """Error of one (sequence, KV head) slice of the timed workload's output against the CPU oracle (the checker
    role of oracle/: computed after the timed region, never inside it).  Returns max-abs and max-rel error."""
    from oracle import tq_oracle as O
    from turboquant.kernels import paged_layout
    f = wl.fmt
    seq = min(seq, wl.batch - 1)
    n_pages = int(wl.pages[seq])
    L = int(wl.lens[seq])
    g = wl.hq // wl.hkv
    pages = wl.caches[layer][wl.block_tables[seq, :n_pages].long(), kvh].cpu()
    u = paged_layout.unpack_pages(pages, f.k_bits, f.v_bits, f.use_qjl)
    kf = {"idx": u["k_idx"].reshape(-1, 16, 1, 128).numpy(), "norm": u["k_norm"].float().reshape(-1, 16, 1).numpy()}
    if f.use_qjl:
        kf["signs"] = u["k_signs"].reshape(-1, 16, 1, 128).numpy()
        kf["rnorm"] = u["k_rnorm"].float().reshape(-1, 16, 1).numpy()
    vf = {"idx": u["v_idx"].reshape(-1, 16, 1, 128).numpy(), "norm": u["v_norm"].float().reshape(-1, 16, 1).numpy()}
    qs = q_dev[layer, seq:seq + 1, kvh * g:(kvh + 1) * g].float().cpu().numpy()
    ref = O.paged_decode(qs, qs, kf, vf, np.arange(n_pages)[None], np.array([L]), wl.books.kc.cpu().numpy(),
                         wl.books.vc.cpu().numpy(), 1 / math.sqrt(128), math.sqrt(math.pi / 2) / 128, 16)[0]
    got = outs[layer, seq, kvh * g:(kvh + 1) * g].float().cpu().numpy()
    d = np.abs(got - ref)
    return {"slice": f"layer {layer}, sequence {seq} ({L} tokens), KV head {kvh}, {g} query heads", "max_abs": float(d.max()),
            "max_rel": float((d / np.maximum(np.abs(ref), 1e-6))[np.abs(ref) > 1e-3].max()) if (np.abs(ref) > 1e-3).any() else 0.0,
            "max_abs_minus_1e-2_ref": float((d - 1e-2 * np.abs(ref)).max()), "max_ref": float(np.abs(ref).max()),
            "bar": "max(|diff| - 1e-2 |ref|) <= 2e-3"}


def time_small_compress(wl: "Workload", reps: int = 50) -> float:
    """us per launch of the decode step's own compression: one new token per sequence (batch x KV heads items)."""
    from turboquant.kernels.paged import compress_and_scatter
    dev = wl.device
    k = torch.randn(wl.batch, wl.hkv, 128, device=dev, dtype=torch.float16)
    v = torch.randn(wl.batch, wl.hkv, 128, device=dev, dtype=torch.float16)
    last = (wl.lens - 1).long()
    slots = (wl.block_tables.cpu()[torch.arange(wl.batch), (last // 16)].long() * 16 + last % 16).to(dev)
    for _ in range(3):
        compress_and_scatter(k, v, wl.caches[0], slots, wl.books, wl.block_size)
    torch.cuda.synchronize()
    # captured in a CUDA graph like the e2e step, so that the figure is the kernel, not Python launch overhead
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            compress_and_scatter(k, v, wl.caches[0], slots, wl.books, wl.block_size)
    graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


TC = False     # time the opt-in tensor-memory rotation kernel in time_bulk_compress


def time_bulk_compress(fmt_name: str, tokens: int, hkv: int, device, reps: int = 3):
    """GB/s of compress-and-scatter for `tokens` new tokens x hkv KV heads of fp16 K/V into a paged cache
    (bytes = fp16 K + V read, packed pages written)."""
    from turboquant.kernels.paged import CacheFormat, Codebooks, allocate_cache, compress_and_scatter
    fmt = CacheFormat.named(fmt_name)
    books = Codebooks(fmt, device)
    nb = tokens // 16
    cache = allocate_cache(nb, 16, hkv, fmt, device)
    g = torch.Generator(device=device).manual_seed(5)
    K = torch.randn(tokens, hkv, 128, generator=g, device=device, dtype=torch.float16)
    V = torch.randn(tokens, hkv, 128, generator=g, device=device, dtype=torch.float16)
    K[..., OUTLIER_CHANNELS] *= 10
    V[..., OUTLIER_CHANNELS] *= 10
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(6)).to(device)
    slots = (perm.repeat_interleave(16) * 16 + torch.arange(tokens, device=device) % 16)
    compress_and_scatter(K, V, cache, slots, books, 16, tcgen05=TC)
    ms = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        compress_and_scatter(K, V, cache, slots, books, 16, tcgen05=TC)
        e1.record()
        e1.synchronize()
        ms.append(e0.elapsed_time(e1))
    nbytes = tokens * hkv * (2 * 128 * 2 + fmt.page_bytes / 16)
    del K, V, cache
    return nbytes / (min(ms) / 1e3) / 1e9, min(ms) * 1e3


def _graph_time_us(fn, reps: int = 10) -> float:
    """Device time of fn() in microseconds: `reps` calls captured in one CUDA graph, CUDA events around the replay
    (so that no Python or launch overhead sits between the kernels), best of three replays after a warm-up."""
    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(reps):
                fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(4):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        e1.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / reps)
    return best


def time_packed_attention(device, bits: int = 3, BH: int = 64, Sk: int = 32768):
    """The contiguous packed_attention call (one query per K/V stream, reference byte layouts) on random packed
    fields: us per call (partial + merge kernels) and GB/s of packed bytes read."""
    from turboquant.core import make_codebook
    from turboquant.kernels import packed_attention as PA
    g = torch.Generator(device=device).manual_seed(1)
    c, _ = make_codebook(128, bits)
    c = c.to(device)
    k_idx = torch.randint(0, 256, (BH, Sk, 16 * bits), dtype=torch.uint8, device=device, generator=g)
    k_sg = torch.randint(0, 256, (BH, Sk, 16), dtype=torch.uint8, device=device, generator=g)
    v_idx = torch.randint(0, 256, (BH, Sk, 16 * bits), dtype=torch.uint8, device=device, generator=g)
    k_rn = (torch.rand(BH, Sk, device=device, generator=g) * 3).half()
    k_n = (torch.rand(BH, Sk, device=device, generator=g) * 4 + 8).half()
    v_n = (torch.rand(BH, Sk, device=device, generator=g) * 4 + 8).half()
    Q = (torch.randn(BH, 128, device=device, generator=g) / math.sqrt(128)).half()
    Qp = (torch.randn(BH, 128, device=device, generator=g) / math.sqrt(128)).half()
    cs = math.sqrt(math.pi / 2) / math.sqrt(128)
    us = _graph_time_us(lambda: PA.packed_attention(Q, Qp, k_idx, k_sg, k_rn, k_n, v_idx, v_n, c, cs))
    nbytes = BH * Sk * (32 * bits + 16 + 6)
    return us, nbytes / us / 1e3


def time_contiguous_compress(device, bits: int = 3, n: int = 1 << 20):
    """compress_k / compress_v of n fp16 rows into the reference's contiguous packed arrays, rotation included:
    (us, GB/s) each, bytes = rows read + packed fields written."""
    from turboquant.core import make_codebook, make_wht_matrix
    from turboquant.kernels import packed_compress
    g = torch.Generator(device=device).manual_seed(2)
    x = torch.randn(n, 128, device=device, generator=g).half()
    x[:, OUTLIER_CHANNELS] *= 10
    c, b = make_codebook(128, bits)
    c, b, H = c.to(device), b.to(device), make_wht_matrix(128).to(device)
    us_k = _graph_time_us(lambda: packed_compress.compress_k_permuted(x, H, None, c, b), reps=4)
    us_v = _graph_time_us(lambda: packed_compress.compress_v(x, H, c, b), reps=4)
    bk, bv = n * (256 + 16 * bits + 16 + 4), n * (256 + 16 * bits + 2)
    return (us_k, bk / us_k / 1e3), (us_v, bv / us_v / 1e3)


def measure_contiguous_api(device, peak: float) -> dict:
    """Rows for the contiguous (non-paged) API of the reference's packed kernels."""
    res = {}
    us, gbs = time_packed_attention(device)
    res["packed_attention"] = {"workload": "contiguous packed_attention, 3-bit + QJL, BH 64 x 32768 tokens (247 MB packed)",
                               "us": us, "GBps": gbs, "frac_of_peak": gbs / peak}
    (us_k, gk), (us_v, gv) = time_contiguous_compress(device)
    res["compress_k_contiguous"] = {"workload": "compress_k, 3-bit + QJL, 1 048 576 fp16 rows, rotation in the kernel",
                                    "us": us_k, "GBps": gk, "frac_of_peak": gk / peak}
    res["compress_v_contiguous"] = {"workload": "compress_v, 3-bit, 1 048 576 fp16 rows, rotation in the kernel",
                                    "us": us_v, "GBps": gv, "frac_of_peak": gv / peak}
    gbs, us = time_bulk_compress("turbo3", 1 << 18, 8, device)
    res["compress_paged_256K_tokens"] = {"workload": "turbo3 compress-and-scatter of 262 144 new tokens x 8 KV heads (fp16 K/V)"
                                                     + (", tcgen05 rotation kernel" if TC else ""),
                                         "us": us, "GBps": gbs, "frac_of_peak": gbs / peak}
    return res


def measure_other_workloads(device, peak: float, steps: int, warmup: int) -> dict:
    """The other single-GPU workloads, two layers each, measured in the same run (device-resident inputs, CUDA
    events, one CUDA graph per step): us/layer, GB/s of packed bytes, fraction of the measured peak."""
    res = {}
    for name in ("cfg4", "cfg4s", "cfg5"):
        wl = Workload(name, 0, 1, device, 2)
        wl.build_caches()
        torch.cuda.synchronize()
        ms, skip, _ = time_device_steps(wl, steps, warmup, lambda: None)
        sec_layer = ms / 1e3 / (steps * wl.layers)
        gbs = wl.tok_heads_total * wl.bytes_per_tok_head / sec_layer / 1e9
        comp = wl.compress_ms[-1]
        row = {"workload": wl.spec["desc"], "layers": wl.layers, "us_per_layer": sec_layer * 1e6, "GBps": gbs,
               "frac_of_peak": gbs / peak, "pct_of_8TBps": 100 * gbs / 8000.0,
               "tokens": int(wl.lens.sum()), "compress_GBps": wl.compress_bytes / (comp / 1e3) / 1e9}
        if skip is not None:
            row["sparse_v"] = skip
        res[name] = row
        del wl
        torch.cuda.empty_cache()
    gbs, us = time_bulk_compress("turbo2", 1 << 20, 8, device)
    res["cfg5_compress_1M_tokens"] = {"workload": "turbo2 compress-and-scatter of 1 048 576 new tokens x 8 KV heads (fp16 K/V)",
                                      "us": us, "GBps": gbs, "frac_of_peak": gbs / peak, "pct_of_8TBps": 100 * gbs / 8000.0}
    res.update(measure_contiguous_api(device, peak))
    return res



def cpu_oracle_sample(fmt_name: str, budget_s: float, threads: int):
    """Time the CPU oracle (numpy restatement of the reference's path) on a bounded sample of the workload:
    whole (sequence, KV-head group) items of 8192 tokens x 8 query heads, compress + decode, as many as fit the
    budget.  Returns (GB/s of packed bytes decoded, items, seconds, compress vectors/s)."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import tq_oracle as O
    from turboquant.kernels.paged import CacheFormat
    # One BLAS thread per Python worker: `threads` workers each running an all-core BLAS pool oversubscribe
    # the host several times over (the same code measured 10x slower that way).
    try:
        from threadpoolctl import threadpool_limits
        blas_guard = threadpool_limits(limits=1)
    except Exception:                               # threadpoolctl missing: the pools stay as the environment set them
        blas_guard = None
    fmt = CacheFormat.named(fmt_name)
    L, G = 8192, 8
    kc, kb = O.make_codebook(128, fmt.k_bits)
    vc, vb = O.make_codebook(128, fmt.v_bits)
    H = O.make_wht_matrix(128)

    def make_item(seed):
        rng = np.random.default_rng(seed)
        K = rng.standard_normal((L, 128), dtype=np.float32)
        V = rng.standard_normal((L, 128), dtype=np.float32)
        K[:, OUTLIER_CHANNELS] *= 10
        V[:, OUTLIER_CHANNELS] *= 10
        q = rng.standard_normal((1, G, 128), dtype=np.float32)
        return K, V, q

    def compress_item(item):
        K, V, q = item
        ck = O.polarquant_compress(K, kc, kb, fmt.k_bits, fmt.use_qjl, H)
        cv = O.polarquant_compress(V, vc, vb, fmt.v_bits, False, H)
        kf = {"idx": ck["indices"].reshape(L // 16, 16, 1, 128), "norm": ck["norms"].reshape(L // 16, 16, 1)}
        if fmt.use_qjl:
            kf["signs"] = (ck["signs"] > 0).reshape(L // 16, 16, 1, 128)
            kf["rnorm"] = ck["rot_residual_norm"].reshape(L // 16, 16, 1)
        vf = {"idx": cv["indices"].reshape(L // 16, 16, 1, 128), "norm": cv["norms"].reshape(L // 16, 16, 1)}
        return kf, vf, q

    def decode_item(c):
        kf, vf, q = c
        bt = np.arange(L // 16)[None]
        return O.paged_decode(q @ H, q @ H, kf, vf, bt, np.array([L]), kc, vc, 1 / math.sqrt(128),
                              math.sqrt(math.pi / 2) / 128, 16)

    items = [make_item(i) for i in range(threads)]
    with ThreadPoolExecutor(max_workers=threads) as pool:
        t0 = time.perf_counter()
        comp = list(pool.map(compress_item, items))
        t_comp = time.perf_counter() - t0
        n_dec, t_dec = 0, 0.0
        while t_dec < budget_s:
            t0 = time.perf_counter()
            list(pool.map(decode_item, comp))
            t_dec += time.perf_counter() - t0
            n_dec += len(comp)
    bytes_dec = n_dec * L * fmt.page_bytes / 16
    if blas_guard is not None:
        blas_guard.restore_original_limits()
    return bytes_dec / t_dec / 1e9, n_dec, t_dec, 2 * L * threads / t_comp


def config_dict(workload: str, layers: int, gpus: int) -> dict:
    """The workload description both arms print (identical for the same command-line arguments)."""
    w = WORKLOADS[workload]
    return {"workload": f"{workload}: {w['desc']}", "format": w["fmt"], "layers": layers, "block_size": 16,
            "parallelism": f"kv-head sharding x{gpus}",
            "l2": "each layer has its own cache (>= 3.9x the 126 MB L2 per rank at N=1); no explicit flush",
            "tolerance": "|diff| <= 2e-3 + 1e-2 |ref| vs fp32 oracle (tests/test_gpu_decode.py)"}


def traffic_from_profile(workload: str, world: int):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary of this exact shape
    (a line `traffic_bytes_per_launch: N` in profiles/decode_partial_turbo3_cfg3.md); None for other shapes."""
    if workload != "cfg3" or world != 1:
        return None
    import re
    try:
        with open(os.path.join(ROOT, "profiles", "decode_partial_turbo3_cfg3.md")) as fh:
            m = re.search(r"traffic_bytes_per_launch:\s*(\d+)", fh.read())
        return int(m.group(1)) if m else None
    except OSError:
        return None


def load_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def run_reference_arm(args, rank: int):
    """The reference's CPU path for the same workload, restated in oracle/ (numpy), on all host threads."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    w = WORKLOADS[args.workload]
    vals = []
    for i in range(args.warmup + args.steps):
        gbs, n, secs, vps = cpu_oracle_sample(w["fmt"], budget_s=2.0, threads=threads)
        if i >= args.warmup:
            vals.append((gbs, n, secs, vps))
    gbs = statistics.mean(v[0] for v in vals)
    sample = (f"host cores, no GPU; per step a bounded sample of the workload: {vals[0][1]} (sequence, KV-head group) "
              f"items of 8192 tokens x 8 query heads, {w['fmt']} decode over unpacked oracle fields, {threads} "
              f"Python threads with one BLAS thread each")
    line = {"impl": "reference", "metric": "tq_decode_attn_hbm_GBps", "value": gbs, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * statistics.mean(v[2] for v in vals), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            # the same workload as the GPU arm (same config dict); what one CPU step covers is in cpu_baseline.sample
            "config": config_dict(args.workload, args.layers or w["layers"], args.gpus),
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample,
                             "compress_vectors_per_s": statistics.mean(v[3] for v in vals)},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (smaller profiling runs)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-others", action="store_true", help="skip the other workloads' rows (single GPU only)")
    ap.add_argument("--compress-kernel", default="default", choices=["default", "tcgen05"],
                    help="rotation kernel of the bulk compress rows: mma.sync (default) or the opt-in tcgen05 / tensor-memory one")
    ap.add_argument("--micro", action="store_true",
                    help="only the contiguous-API rows (packed_attention, compress_k, compress_v): one JSON line, for small profiling runs")
    ap.add_argument("--decode-kernel", default="default", choices=["default", "tcgen05"],
                    help="tcgen05: time the opt-in tensor-memory variant in the device-resident leg (value / roofline)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "b200" and not args.layers:
        args.warmup = 3

    if args.compress_kernel == "tcgen05":
        global TC
        TC = True
    if args.decode_kernel == "tcgen05":
        global DECODE_FLAGS
        from turboquant.kernels import _native
        DECODE_FLAGS = _native.IO_TCGEN05
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if args.micro:
        peak, peak_src = load_peak()
        print(json.dumps({"micro": measure_contiguous_api(dev, peak), "peak_GBps": peak, "peak_source": peak_src}))
        return
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

        def barrier():
            dist.barrier()
    else:
        def barrier():
            pass

    wl = Workload(args.workload, rank, world, dev, args.layers or None)
    wl.build_caches()
    torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    ms, skip, outs = time_device_steps(wl, args.steps, args.warmup, barrier)
    clocks = sampler.stop()
    e2e_ms = h2d = d2h = None
    e2e_how = ""
    if not args.no_e2e:
        e2e_ms, h2d, d2h, e2e_how = time_e2e_steps(wl, args.steps, args.warmup, barrier)

    gather_us = None
    if use_dist:
        import torch.distributed as dist
        t = torch.tensor([ms, e2e_ms or 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)          # slowest rank defines the step
        ms, e2e_max = t.tolist()
        e2e_ms = e2e_max if e2e_ms is not None else None
        # optional single-rank result: gather the per-head outputs of one layer (not part of the timed value)
        parts = [torch.empty_like(outs[0]) for _ in range(world)]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.all_gather(parts, outs[0].contiguous())
        e0.record()
        dist.all_gather(parts, outs[0].contiguous())
        e1.record()
        torch.cuda.synchronize()
        gather_us = e0.elapsed_time(e1) * 1e3

    if rank == 0:
        peak, peak_src = load_peak()
        layers = wl.layers
        bytes_layer_total = wl.tok_heads_total * wl.bytes_per_tok_head          # algorithmic packed bytes, all ranks
        bytes_layer_rank = wl.tok_heads_rank * wl.bytes_per_tok_head
        sec_per_layer = ms / 1e3 / (args.steps * layers)
        value = bytes_layer_total / sec_per_layer / 1e9
        achieved_rank = bytes_layer_rank / sec_per_layer / 1e9
        comp = wl.compress_ms[min(3, len(wl.compress_ms) - 1):] or wl.compress_ms
        comp_gbs = wl.compress_bytes / (statistics.mean(comp) / 1e3) / 1e9
        line = {
            "metric": "tq_decode_attn_hbm_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": config_dict(args.workload, layers, world),
            "us_per_layer": sec_per_layer * 1e6,
            "tokens_per_s": wl.batch / (sec_per_layer * layers),
            "pct_of_8TBps_per_gpu": 100 * achieved_rank / 8000.0,
            "compress": {"GBps_per_gpu": comp_gbs, "us_per_layer": statistics.mean(comp) * 1e3,
                         "bytes_per_layer_per_gpu": wl.compress_bytes, "frac_of_peak": comp_gbs / peak,
                         "pct_of_8TBps": 100 * comp_gbs / 8000.0,
                         "how": "CUDA events around compress_and_scatter of each layer's fp16 K+V (fresh inputs)"},
            "roofline": {"bound": "hbm", "achieved": achieved_rank, "peak": peak, "unit": "GB/s",
                         "frac": achieved_rank / peak,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this exact shape, from the
                         # committed ncu summary; other shapes were not captured
                         "traffic": traffic_from_profile(args.workload, world),
                         "peak_source": peak_src,
                         "kernel": "decode_partial_kernel (+ merge) per layer per GPU",
                         "algorithmic_bytes_per_launch": bytes_layer_rank},
            "clocks": clocks,
            "gpu_launches": args.steps * layers * 2,
        }
        if skip is not None:
            line["sparse_v"] = skip
        if e2e_ms is not None:
            e2e_sec_layer = e2e_ms / 1e3 / (args.steps * layers)
            line["e2e"] = {"value": bytes_layer_total / e2e_sec_layer / 1e9, "unit": "GB/s",
                           "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
                           "us_per_layer": e2e_sec_layer * 1e6,
                           "what": "pinned-host q + new-token K/V -> H2D, compress+scatter, rotate q, decode, "
                                   "de-rotate, D2H of the output, every layer; copies double-buffered on their own "
                                   "streams; launched as " + e2e_how}
        if gather_us is not None:
            line["output_all_gather_us"] = gather_us
        line["parity"] = parity_slice(wl, outs, time_device_steps.last_queries)
        line["compress"]["decode_step_launch_us"] = time_small_compress(wl)
        line["compress"]["decode_step_launch_what"] = (f"one new token per sequence: {wl.batch} x {wl.hkv} items per launch "
                                                       "(the compression inside the e2e step)")
        if world == 1 and not args.no_others and not args.layers:
            del outs
            wl.caches.clear()
            torch.cuda.empty_cache()
            line["other_workloads"] = measure_other_workloads(dev, peak, max(2, min(args.steps, 3)), 3)
        if not args.no_cpu_baseline and world == 1:
            threads = os.cpu_count() or 1
            gbs, n, secs, vps = cpu_oracle_sample(wl.spec["fmt"], budget_s=10.0, threads=threads)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": f"{n} (sequence, KV-head group) items of 8192 tokens x 8 query heads "
                                              f"decoded by the numpy oracle in {secs:.1f} s",
                                    "compress_vectors_per_s": vps}
        print(json.dumps(line))
    if use_dist:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
