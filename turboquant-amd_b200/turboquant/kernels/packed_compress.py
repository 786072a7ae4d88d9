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
  * the fused kernel applies the Walsh-Hadamard rotation of
    make_wht_matrix(128) and takes the signs of the rotated residual itself
    (S = I, as in turboquant.core): PiT None / that matrix and PiST None / the
    identity select it.  Any other orthogonal PiT (the reference's own demo,
    packed_compress.py:247-275, passes a QR-orthogonal Pi) and any PiST
    (Pi S^T with a Gaussian S there) take a composed path: the rotation and the
    projection of the residual are plain matrix products (torch.matmul), the
    quantisation in between runs on the same kernels.  That path is there for
    call compatibility, it is not a tuned one.
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


def _remembered(matrix: torch.Tensor, tag: str, test) -> bool:
    """test(matrix), evaluated once per tensor object and content version."""
    key = "_tq_" + tag
    hit = getattr(matrix, key, None)
    if hit is not None and hit[0] == matrix._version:
        return hit[1]
    verdict = bool(test(matrix))
    setattr(matrix, key, (matrix._version, verdict))
    return verdict


def _is_wht(matrix: torch.Tensor) -> bool:
    from turboquant.core.rotation import make_wht_matrix
    return _remembered(matrix, "is_wht", lambda m: tuple(m.shape) == (128, 128) and torch.allclose(
        m.detach().float().cpu(), make_wht_matrix(128), atol=1e-6, rtol=0))


def _is_identity(matrix: torch.Tensor) -> bool:
    return _remembered(matrix, "is_eye", lambda m: tuple(m.shape) == (128, 128) and torch.equal(
        m.detach().float().cpu(), torch.eye(128)))


def _is_orthogonal(matrix: torch.Tensor) -> bool:
    def test(m):
        mf = m.detach().float().cpu()
        return tuple(mf.shape) == (128, 128) and (mf @ mf.T - torch.eye(128)).abs().max().item() < 1e-3
    return _remembered(matrix, "is_orth", test)


def _check_rotation(PiT, PiST) -> bool:
    """True when the fused kernel must rotate (PiT is the WHT matrix), False when the input is already rotated.
    Only for the fused path: PiT None / WHT, PiST None / identity."""
    if PiST is not None and not _is_identity(PiST):
        raise ValueError("PiST must be None or the identity on the fused path")
    if PiT is None:
        return False
    _native.check_is_wht(PiT, 128)
    return True


def _fused_ok(PiT, PiST) -> bool:
    return (PiT is None or _is_wht(PiT)) and (PiST is None or _is_identity(PiST))


def _rotate_general(X: torch.Tensor, PiT: torch.Tensor) -> torch.Tensor:
    """X @ PiT in fp32 for an orthogonal PiT that is not the WHT matrix (packed_compress.py:65-66 of the reference,
    where the product is taken of the normalised rows; for an orthogonal matrix the norm is the same either side)."""
    if not _is_orthogonal(PiT):
        raise ValueError("PiT must be an orthogonal 128 x 128 matrix (the norm is taken after the rotation)")
    return X.float() @ PiT.to(device=X.device, dtype=torch.float32)


def _pack_sign_bytes(positive: torch.Tensor) -> torch.Tensor:
    """[N, 128] bool -> [N, 16] uint8, byte j bit b = dim 8 j + b."""
    w = (1 << torch.arange(8, device=positive.device, dtype=torch.int32))
    return (positive.reshape(-1, 16, 8).to(torch.int32) * w).sum(-1).to(torch.uint8)


def _compress_k_general(K, PiT, PiST, centroids, boundaries, permute: bool):
    """compress_k for an orthogonal PiT other than the WHT matrix and / or a PiST other than the identity
    (packed_compress.py:65-76 of the reference): rotate by a matrix product, quantise with the fused kernel on the
    rotated rows, and, when PiST is given, take the signs of (rotated residual) @ PiST."""
    from turboquant.core.quantizer import PolarQuantConfig, polarquant_compress
    K_rot = K.float() if PiT is None else (_rotate_general(K, PiT) if not _is_wht(PiT) else None)
    if K_rot is None:                     # WHT rotation, general PiST: rotate with the fast transform
        K_rot = _native.wht_rows(K.float().contiguous())
    K_rot = K_rot.contiguous()
    k_idx, k_signs, k_rnorm, k_norm = _compress_k(K_rot, None, None, centroids, boundaries, permute=False)
    if PiST is not None and not _is_identity(PiST):
        bits = _bits_of(centroids)
        r = polarquant_compress(K_rot, centroids, boundaries, PolarQuantConfig(bits=bits, use_qjl=False), None)
        proj = (K_rot - r["k_mse_rot"]) @ PiST.to(device=K.device, dtype=torch.float32)
        k_signs = _pack_sign_bytes(proj >= 0)
    if permute:
        k_signs = permute_signs_for_chunked(k_signs)
    return k_idx, k_signs, k_rnorm, k_norm


def _compress_k(K, PiT, PiST, centroids, boundaries, permute: bool):
    dev = _native._require_cuda(K)
    if K.dim() != 2 or K.shape[1] != 128:
        raise ValueError("K must be [N, 128]")
    if not _fused_ok(PiT, PiST):
        return _compress_k_general(K, PiT, PiST, centroids, boundaries, permute)
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
    if PiT is not None and not _is_wht(PiT):      # an orthogonal matrix other than the WHT: rotate by a matrix product
        return compress_v(_rotate_general(V, PiT).contiguous(), None, centroids, boundaries)
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
