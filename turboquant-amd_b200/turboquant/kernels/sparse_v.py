"""Paged GQA decode with the Sparse-V rule (turboquant/kernels/sparse_v.py of the reference).

The reference ships only two Triton kernels and a benchmark; the launch is
written out by hand at its call site.  Here the same positional arguments
(minus the strides, which the wrapper reads from the tensors) form two
functions: `tq_v12_sparse_v` (skip on) and `tq_v11_dense` (skip off).  The
format is the reference's "turbo3" of this file: 3-bit MSE-only indices plus
an fp16 norm per token, K and V sharing one codebook, softmax scale applied to
q, result in the space q lives in.

The cache argument is in this build's page layout
(uint8 [num_blocks, Hkv, block_size/16 * page_bytes], see paged_layout.py); a
cache in the reference's [num_blocks, 2, block_size, Hkv, slot] layout can be
converted once with `repack_reference_cache`.

Skip rule: a 16-token V page is skipped when no query head of the GQA group
gives any of its tokens a softmax weight above the threshold relative to the
running maximum; the weights still enter the denominator.  The reference
masks per position inside a fetched tile, which saves no memory traffic; per
page is the granularity at which HBM bytes are actually avoided, and it skips
a subset of what the reference skips, so the result is at least as close to
the dense one.
"""
from __future__ import annotations

import torch

from turboquant.kernels import _native
from turboquant.kernels import paged_layout

D = 128
DQ3 = D * 3 // 8  # 48 packed index bytes per token in the reference slot
CD = 32
SPARSE_V_THRESHOLD = 1e-6


def repack_reference_cache(tq_cache: torch.Tensor, block_size: int, bits: int = 3) -> torch.Tensor:
    """[num_blocks, 2, block_size, Hkv, slot >= 50] (reference layout) -> this build's paged cache.

    Slot bytes 0..47 are the little-endian 3-bit index stream, bytes 48..49 the
    fp16 norm (turboquant/kernels/sparse_v.py:57-60,76-80).  Pure torch, meant
    for one-off conversion and tests.
    """
    from turboquant.kernels.packed_compress import unpack_indices
    nb, two, bs, hkv, slot = tq_cache.shape
    assert two == 2 and bs == block_size and slot >= 16 * bits + 2
    nidx = 16 * bits
    fields = {}
    for name, kv in (("k", 0), ("v", 1)):
        part = tq_cache[:, kv]
        idx = unpack_indices(part[..., :nidx].reshape(-1, nidx), bits, D).reshape(nb, bs, hkv, D)
        norm = part[..., nidx:nidx + 2].contiguous().view(torch.float16).reshape(nb, bs, hkv)
        fields[f"{name}_idx"] = idx.to(torch.uint8)
        fields[f"{name}_norm"] = norm
    return paged_layout.pack_cache(fields, block_size, bits, bits, False)


def _launch(out, q, tq_cache, centroids, block_tables, seq_lens, scale, sparse_thresh):
    n = centroids.numel()
    if n not in (4, 8, 16):
        raise ValueError("centroids must have 4, 8 or 16 entries")
    bits = n.bit_length() - 1
    dev = _native._require_cuda(out, q, tq_cache, block_tables, seq_lens)
    cb = _native._f32(centroids, dev)
    row = paged_layout.page_bytes(bits, bits, False)
    if tq_cache.dim() != 3 or tq_cache.shape[2] % row:
        raise ValueError("tq_cache must be [num_blocks, Hkv, block_size/16 * page_bytes]; "
                         "convert a reference-layout cache with repack_reference_cache")
    block_size = tq_cache.shape[2] // row * 16
    bt = block_tables if block_tables.dtype == torch.int32 else block_tables.to(torch.int32)
    sl = seq_lens if seq_lens.dtype == torch.int32 else seq_lens.to(torch.int32)
    _native._decode_paged_impl(out, q.contiguous(), None, tq_cache, bt, sl.contiguous(), cb, cb, float(scale), 0.0,
                               float(sparse_thresh), block_size, bits, bits, False, 0)
    return out


def tq_v12_sparse_v(out, q, tq_cache, centroids, block_tables, seq_lens, scale, *,
                    sparse_thresh: float = SPARSE_V_THRESHOLD):
    """out[s, h] = softmax(scale * q[s, h] . K) V over the sequence's pages, skipping negligible V pages."""
    return _launch(out, q, tq_cache, centroids, block_tables, seq_lens, scale, sparse_thresh)


def tq_v11_dense(out, q, tq_cache, centroids, block_tables, seq_lens, scale):
    """The same attention with every V page read (the dense baseline of the reference's benchmark)."""
    return _launch(out, q, tq_cache, centroids, block_tables, seq_lens, scale, 0.0)
