"""Packed split-K decode attention on contiguous [BH, Sk, ...] data
(turboquant/kernels/packed_attention.py of the reference).

`packed_attention` keeps the reference's signature and returns fp16 [BH, D] in
rotated space.  The partial and merge kernels are CUDA (libtq_b200); the
tuning keywords of the reference are accepted, `num_splits` is honoured and
the Triton-specific ones (block_sk, num_warps, num_stages) are ignored.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from turboquant.kernels import _native
from turboquant.kernels.packed_compress import unpack_1bit, unpack_2bit  # noqa: F401  (same re-export as the reference)


def _get_config(BH: int, Sk: int):
    """(block_sk, num_splits, num_warps, num_stages) the kernel will use for a problem size.

    The reference looks these up in a table tuned on MI355X; here the split
    count comes from the library's B200 heuristic and the other three are
    fixed properties of the CUDA kernel (128-token tiles, 4 warps, no
    software pipelining stages).
    """
    return 128, _native.lib().tq_packed_attention_auto_splits(BH, Sk), 4, 1


def attention_unpacked_ref(Q, Q_proj, K_mse_rot, signs_float, k_r_norm, V_mse_rot, corr_scale):
    """fp32 truth on unpacked tensors: softmax(Q K_mse^T + Q_proj (signs * rnorm * corr)^T) V_mse."""
    logits = torch.einsum("bd,bsd->bs", Q, K_mse_rot)
    k_qjl = signs_float * (k_r_norm * corr_scale).unsqueeze(-1)
    logits = logits + torch.einsum("bd,bsd->bs", Q_proj, k_qjl)
    return torch.einsum("bs,bsd->bd", F.softmax(logits, dim=-1), V_mse_rot)


def packed_attention(Q, Q_proj, k_idx_packed, k_signs_packed, k_r_norm, k_norm,
                     v_idx_packed, v_norm, centroids, corr_scale,
                     num_splits=None, block_sk=None, num_warps=None, num_stages=None):
    """Q, Q_proj fp16 [BH, 128]; packed K/V as produced by compress_k_permuted / compress_v,
    reshaped to [BH, Sk, ...]; centroids fp32 [4 | 8 | 16]; returns fp16 [BH, 128]."""
    dev = _native._require_cuda(Q, Q_proj, k_idx_packed, k_signs_packed, k_r_norm, k_norm, v_idx_packed, v_norm)
    BH, D = Q.shape
    if D != 128:
        raise ValueError("only head_dim 128 is supported")
    Sk = k_r_norm.shape[1]
    n = centroids.numel()
    if n not in (4, 8, 16):
        raise ValueError("centroids must have 4, 8 or 16 entries")
    bits = n.bit_length() - 1
    if tuple(k_idx_packed.shape) != (BH, Sk, 16 * bits) or tuple(v_idx_packed.shape) != (BH, Sk, 16 * bits):
        raise ValueError(f"index tensors must be [BH, Sk, {16 * bits}] for {n} centroids")
    if tuple(k_signs_packed.shape) != (BH, Sk, 16):
        raise ValueError("k_signs_packed must be [BH, Sk, 16]")
    half = lambda t: t.to(torch.float16).contiguous()
    Qh, Qph = half(Q), half(Q_proj)
    kidx, ksg, vidx = k_idx_packed.contiguous(), k_signs_packed.contiguous(), v_idx_packed.contiguous()
    krn, kn, vn = half(k_r_norm), half(k_norm), half(v_norm)
    cb = _native._f32(centroids, dev)
    L = _native.lib()
    splits = int(num_splits) if num_splits else L.tq_packed_attention_auto_splits(BH, Sk)
    splits = max(1, min(splits, Sk))
    need = L.tq_packed_attention_workspace_bytes(BH, splits)
    ws = _native.workspace(dev, need, tag="packed_attention")
    out = torch.empty(BH, D, dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        rc = L.tq_packed_attention(
            _native._ptr(Qh), _native._ptr(Qph), _native._ptr(kidx), _native._ptr(ksg), _native._ptr(krn),
            _native._ptr(kn), _native._ptr(vidx), _native._ptr(vn), _native._ptr(cb), float(corr_scale),
            BH, Sk, bits, splits, _native._ptr(ws), ws.numel(), _native._ptr(out), _native._stream(dev))
    _native._check(rc, "tq_packed_attention")
    return out
