"""Paged-cache entry points: compress-and-scatter and split-K decode attention.

These are the two calls a serving engine makes per layer and step.  They stand
where the reference has `turbo4_fp8_compress_and_scatter`
(turboquant/integration/vllm_backend.py:179-230) and the decode launch of
`TurboQuantFP4Impl.forward` (turboquant/integration/tq_fp4_backend.py:604-641),
with TurboQuant's own packed format (indices, norms, QJL signs) as the cache
content instead of FP8/FP4 values.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from turboquant.core.codebook import make_codebook
from turboquant.kernels import _native
from turboquant.kernels.paged_layout import PAGE_TOKENS, PageLayout


@dataclass(frozen=True)
class CacheFormat:
    """turbo2 = (2, 2, True), turbo3 = (3, 3, True), turbo4 = (4, 4, False); K and V widths may differ."""

    k_bits: int = 3
    v_bits: int = 3
    use_qjl: bool = True

    @staticmethod
    def named(name: str) -> "CacheFormat":
        table = {"turbo2": CacheFormat(2, 2, True), "turbo3": CacheFormat(3, 3, True),
                 "turbo4": CacheFormat(4, 4, False)}
        return table[name]

    @property
    def layout(self) -> PageLayout:
        return PageLayout(self.k_bits, self.v_bits, self.use_qjl)

    @property
    def page_bytes(self) -> int:
        return self.layout.page_bytes

    @property
    def bytes_per_token(self) -> float:
        return self.page_bytes / PAGE_TOKENS

    def cache_shape(self, num_blocks: int, block_size: int, num_kv_heads: int) -> tuple[int, int, int]:
        if block_size % PAGE_TOKENS:
            raise ValueError("block_size must be a multiple of 16")
        return (num_blocks, num_kv_heads, block_size // PAGE_TOKENS * self.page_bytes)


class Codebooks:
    """Device copies of the K and V codebooks for a format (Lloyd-Max for N(0, 1/128) by default)."""

    def __init__(self, fmt: CacheFormat, device, k_codebook=None, v_codebook=None):
        self.fmt = fmt
        dev = torch.device(device)
        kc, kb = k_codebook if k_codebook is not None else make_codebook(128, fmt.k_bits)
        if v_codebook is not None:
            vc, vb = v_codebook
        elif fmt.v_bits == fmt.k_bits:
            vc, vb = kc, kb          # one tensor for both: the decode kernel then keeps a single lookup table
        else:
            vc, vb = make_codebook(128, fmt.v_bits)
        f = lambda t: t.to(device=dev, dtype=torch.float32).contiguous()
        self.kc, self.kb = f(kc), f(kb)
        self.vc, self.vb = (self.kc, self.kb) if vc is kc else (f(vc), f(vb))


def allocate_cache(num_blocks: int, block_size: int, num_kv_heads: int, fmt: CacheFormat, device) -> torch.Tensor:
    return torch.zeros(fmt.cache_shape(num_blocks, block_size, num_kv_heads), dtype=torch.uint8, device=device)


def compress_and_scatter(key: torch.Tensor, value: torch.Tensor, cache: torch.Tensor, slot_mapping: torch.Tensor,
                         books: Codebooks, block_size: int, prerotated: bool = False, tcgen05: bool = False) -> None:
    """Compress key/value [T, Hkv, 128] and write them at `slot_mapping` (int64 [T]) into the paged cache.

    Slot s lands in block s // block_size at offset s % block_size; negative
    slots are clamped to 0 like the reference's scatter does.
    """
    fmt = books.fmt
    if slot_mapping.dtype != torch.int64:
        slot_mapping = slot_mapping.to(torch.int64)
    if tcgen05:
        # opt-in variant: rotation of fp16 / bf16 rows as a tcgen05 product (large launches only; otherwise ignored)
        from turboquant.kernels import _native
        _native._compress_paged_impl(key, value, cache, slot_mapping.contiguous(), books.kc, books.kb, books.vc, books.vb,
                                     block_size, fmt.k_bits, fmt.v_bits, fmt.use_qjl, prerotated, tcgen05=True)
        return
    torch.ops.tq_b200.compress_paged(key, value, cache, slot_mapping.contiguous(), books.kc, books.kb, books.vc,
                                     books.vb, block_size, fmt.k_bits, fmt.v_bits, fmt.use_qjl, prerotated)


def paged_decode_attention(q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
                           books: Codebooks, block_size: int, sm_scale: Optional[float] = None,
                           corr_scale: Optional[float] = None, sparse_thresh: float = 0.0,
                           q_proj: Optional[torch.Tensor] = None, rotate_q: bool = False,
                           derotate_out: bool = False, chunk_pages: int = 0,
                           out: Optional[torch.Tensor] = None, skip_stats: Optional[torch.Tensor] = None,
                           max_seq_len: int = 0, static_scratch: bool = False, tcgen05: bool = False) -> torch.Tensor:
    """One decode step over the packed paged cache.

    q [num_seqs, Hq, 128] fp16/bf16.  With rotate_q the query is first taken to
    rotated space (q' = q H); otherwise it must already be there.  q_proj is
    S q' for the QJL term (None when S = I).  The result is in rotated space
    unless derotate_out.  sm_scale defaults to 1/sqrt(128), corr_scale to
    sqrt(pi/2)/128.  sparse_thresh > 0 turns on the Sparse-V page skip.
    skip_stats: optional uint32[2] device tensor accumulating (pages visited, pages skipped).
    max_seq_len: the longest sequence of the step when the host knows it (a serving engine does); the launch is
    then sized for it rather than for the width of block_tables.  static_scratch: keep the split-K partials in
    the library's fixed 16 MiB device array instead of a torch workspace (no allocation; larger problems raise).
    tcgen05: run the tensor-memory variant of the kernel (2- and 3-bit codebooks without Sparse-V; others ignore it).
    """
    fmt = books.fmt
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(128)
    if corr_scale is None:
        corr_scale = math.sqrt(math.pi / 2) / 128
    q = q.contiguous()
    # Both rotations run inside the decode kernels (query rotated while its fragments are loaded, output
    # de-rotated where it is normalised); only a separate q_proj forces the query rotation to be its own pass.
    flags = _native.IO_DEROTATE_OUT if derotate_out else 0
    if tcgen05:
        flags |= _native.IO_TCGEN05
    if rotate_q and q_proj is None:
        flags |= _native.IO_ROTATE_Q
        q_in = q
    else:
        q_in = _native.wht_rows(q) if rotate_q else q
    if block_tables.dtype != torch.int32:
        block_tables = block_tables.to(torch.int32)
    if seq_lens.dtype != torch.int32:
        seq_lens = seq_lens.to(torch.int32)
    if out is None and skip_stats is None and not static_scratch:
        return torch.ops.tq_b200.decode_paged(q_in, q_proj, cache, block_tables, seq_lens.contiguous(), books.kc,
                                              books.vc, float(sm_scale), float(corr_scale), float(sparse_thresh),
                                              block_size, fmt.k_bits, fmt.v_bits, fmt.use_qjl, int(chunk_pages), flags,
                                              int(max_seq_len))
    res = out if out is not None else torch.empty_like(q_in)
    _native._decode_paged_impl(res, q_in, q_proj, cache, block_tables, seq_lens.contiguous(), books.kc, books.vc,
                               sm_scale, corr_scale, sparse_thresh, block_size, fmt.k_bits, fmt.v_bits,
                               fmt.use_qjl, int(chunk_pages), skip_stats=skip_stats, io_flags=flags,
                               max_seq_len=int(max_seq_len), static_scratch=static_scratch)
    return res
