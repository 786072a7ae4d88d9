"""Packed K/V compression, contiguous output (turboquant/kernels/packed_compress.py of the reference).

Same functions, argument order and return tuples; the work is one CUDA kernel
per call (rotation, bucketize, residual signs, packing and, for
compress_k_permuted, the stride-4 sign order, all fused; no scratch buffer).
Differences from the reference that are deliberate:
  * arithmetic follows turboquant.core.polarquant_compress in fp32 (norm of
    the rotated vector, true division, ties go to the lower centroid), not the
    fp16-dot variant of the Triton kernel;
  * `centroids.numel()` selects the bit width (4, 8 or 16 centroids -> 2, 3,
    4 bits per index); the reference kernel is 2-bit only;
  * PiT must be None or the Walsh-Hadamard matrix of make_wht_matrix(128);
    PiST must be None or the identity (signs are taken of the rotated
    residual itself, S = I, as in turboquant.core).
"""
from __future__ import annotations

import ctypes

import torch

from turboquant.kernels import _native


def unpack_2bit(packed: torch.Tensor, D: int) -> torch.Tensor:
    """[N, D/4] uint8 -> [N, D] int8, four indices per byte, low bits first."""
    p = packed.to(torch.int32)
    parts = [(p >> s) & 3 for s in (0, 2, 4, 6)]
    return torch.stack(parts, dim=-1).reshape(packed.shape[0], D).to(torch.int8)


def unpack_4bit(packed: torch.Tensor, D: int) -> torch.Tensor:
    """[N, D/2] uint8 -> [N, D] int8, low nibble first."""
    p = packed.to(torch.int32)
    return torch.stack([p & 15, (p >> 4) & 15], dim=-1).reshape(packed.shape[0], D).to(torch.int8)


def unpack_3bit(packed: torch.Tensor, D: int) -> torch.Tensor:
    """[N, 3D/8] uint8 little-endian bit stream (dim d at bit 3d) -> [N, D] int8."""
    p = torch.cat([packed.to(torch.int32), torch.zeros_like(packed[:, :1], dtype=torch.int32)], dim=1)
    bit = torch.arange(D, device=packed.device) * 3
    lo, sh = bit >> 3, bit & 7
    return (((p[:, lo] | (p[:, lo + 1] << 8)) >> sh) & 7).to(torch.int8)


def unpack_indices(packed: torch.Tensor, bits: int, D: int = 128) -> torch.Tensor:
    return {2: unpack_2bit, 3: unpack_3bit, 4: unpack_4bit}[bits](packed, D)


def unpack_1bit(packed: torch.Tensor, D: int) -> torch.Tensor:
    """[N, D/8] uint8 -> [N, D] int8 of 0/1, byte j bit b = dim 8j+b."""
    shifts = torch.arange(8, device=packed.device)
    return ((packed.to(torch.int32).unsqueeze(-1) >> shifts) & 1).reshape(packed.shape[0], D).to(torch.int8)


def permute_signs_for_chunked(signs_packed: torch.Tensor, D: int = 128) -> torch.Tensor:
    """Sequential sign bytes -> stride-4 order: output bit 32 c + i holds dim c + 4 i.

    Kept for callers that hold sequentially packed signs; compress_k_permuted
    writes this order directly from the kernel.
    """
    shape = signs_packed.shape
    flat = signs_packed.reshape(-1, D // 8)
    bits = unpack_1bit(flat, D)
    perm = torch.cat([bits[:, c::4] for c in range(4)], dim=1).to(torch.int32)
    weights = (1 << torch.arange(8, device=flat.device, dtype=torch.int32))
    return (perm.reshape(-1, D // 8, 8) * weights).sum(-1).to(torch.uint8).reshape(shape)


def _bits_of(centroids: torch.Tensor) -> int:
    n = centroids.numel()
    if n not in (4, 8, 16):
        raise ValueError(f"centroids must have 4, 8 or 16 entries, got {n}")
    return n.bit_length() - 1


def _check_rotation(PiT, PiST) -> bool:
    """True when the kernel must rotate (PiT is the WHT matrix), False when K is already rotated."""
    if PiST is not None:
        eye = torch.eye(128, device=PiST.device, dtype=PiST.dtype)
        if tuple(PiST.shape) != (128, 128) or not torch.equal(PiST, eye):
            raise ValueError("PiST must be None or the identity: signs are taken of the rotated residual (S = I)")
    if PiT is None:
        return False
    _native.check_is_wht(PiT, 128)
    return True


def _compress_k(K, PiT, PiST, centroids, boundaries, permute: bool):
    dev = _native._require_cuda(K)
    if K.dim() != 2 or K.shape[1] != 128:
        raise ValueError("K must be [N, 128]")
    rotate = _check_rotation(PiT, PiST)
    bits = _bits_of(centroids)
    if K.dtype not in _native._DTYPES:
        K = K.float()
    K = K.contiguous()
    N = K.shape[0]
    c, b = _native._f32(centroids, dev), _native._f32(boundaries, dev)
    k_idx = torch.empty(N, 16 * bits, dtype=torch.uint8, device=dev)
    k_signs = torch.empty(N, 16, dtype=torch.uint8, device=dev)
    k_rnorm = torch.empty(N, dtype=torch.float16, device=dev)
    k_norm = torch.empty(N, dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        rc = _native.lib().tq_compress_k(
            _native._ptr(K), _native._DTYPES[K.dtype], N, _native._ptr(c), _native._ptr(b), bits, int(not rotate),
            int(permute), _native._ptr(k_idx), _native._ptr(k_signs), _native._ptr(k_rnorm), _native._ptr(k_norm),
            _native._stream(dev))
    _native._check(rc, "tq_compress_k")
    return k_idx, k_signs, k_rnorm, k_norm


def compress_k(K, PiT, PiST, centroids, boundaries):
    """-> (k_idx uint8 [N, 16*bits], k_signs uint8 [N, 16] sequential, k_rnorm fp16 [N], k_norm fp16 [N])."""
    return _compress_k(K, PiT, PiST, centroids, boundaries, permute=False)


def compress_k_permuted(K, PiT, PiST, centroids, boundaries):
    """compress_k with the signs in the stride-4 order packed_attention reads."""
    return _compress_k(K, PiT, PiST, centroids, boundaries, permute=True)


def compress_v(V, PiT, centroids, boundaries):
    """-> (v_idx uint8 [N, 16*bits], v_norm fp16 [N])."""
    dev = _native._require_cuda(V)
    if V.dim() != 2 or V.shape[1] != 128:
        raise ValueError("V must be [N, 128]")
    rotate = _check_rotation(PiT, None)
    bits = _bits_of(centroids)
    if V.dtype not in _native._DTYPES:
        V = V.float()
    V = V.contiguous()
    N = V.shape[0]
    b = _native._f32(boundaries, dev)
    v_idx = torch.empty(N, 16 * bits, dtype=torch.uint8, device=dev)
    v_norm = torch.empty(N, dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        rc = _native.lib().tq_compress_v(
            _native._ptr(V), _native._DTYPES[V.dtype], N, _native._ptr(b), bits, int(not rotate),
            _native._ptr(v_idx), _native._ptr(v_norm), _native._stream(dev))
    _native._check(rc, "tq_compress_v")
    return v_idx, v_norm
