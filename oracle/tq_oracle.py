"""CPU oracle for the two TurboQuant hot paths (TEST INFRASTRUCTURE, not product).

This file restates, in plain numpy (fp32 arithmetic, integer bit work), the
reference's algorithm for
  * KV compression (rotation, norm, Lloyd-Max bucketize, QJL signs, packing),
  * asymmetric packed decode attention (contiguous and paged + GQA + Sparse-V).
Every function cites the reference file:line it follows (paths are relative
to the reference project root).

Only tests, the smoke check and the CPU-baseline legs of the benchmark may
import this module, and only as the checker or as the timed CPU baseline.
The product package never imports it.

Parity status: pinned.  `tests/golden/` holds outputs of the reference's own
Python code (turboquant.core.*, turboquant.kernels.packed_* helpers) for
seeded inputs, produced by `tests/golden/make_golden.py`; `tests/test_oracle.py`
checks every function here against those vectors.  The paged + GQA + Sparse-V
composition has no runnable reference test (the reference only ever ran it as
Triton on a GPU); for that piece the oracle composes the pinned parts
(block-table walk, 3-bit stream decode, estimator, skip rule) and is checked
against the dense pinned formula.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np

F32 = np.float32

# ---------------------------------------------------------------------------
# Codebook and rotation construction
# ---------------------------------------------------------------------------


def solve_codebook(d: int, bits: int):
    """Lloyd-Max centroids/boundaries for N(0, 1/d), 100 iterations on +-6 sigma.

    Follows turboquant/core/codebook.py:17-54.  The reference integrates the
    Gaussian pdf numerically (scipy quad); the two integrals have closed forms,
        int x pdf = sigma^2 (pdf(a) - pdf(b)),   int pdf = Phi(b) - Phi(a),
    which are used here so the oracle has no scipy dependency.  The golden
    vectors pin the result to the reference's numeric integration.
    """
    n_levels = 2 ** bits
    sigma = 1.0 / math.sqrt(d)

    def pdf(x):
        return (1.0 / math.sqrt(2 * math.pi * sigma ** 2)) * math.exp(-x * x / (2 * sigma ** 2))

    def mass(a, b):
        # difference of erf values (not of cdf values): keeps mirrored cells exactly mirrored
        r = sigma * math.sqrt(2.0)
        return 0.5 * (math.erf(b / r) - math.erf(a / r))

    lo, hi = -6 * sigma, 6 * sigma
    boundaries = [lo + (hi - lo) * i / n_levels for i in range(1, n_levels)]
    centroids = [0.0] * n_levels
    for _ in range(100):
        edges = [lo] + boundaries + [hi]
        for i in range(n_levels):
            a, b = edges[i], edges[i + 1]
            num = sigma * sigma * (pdf(a) - pdf(b))
            den = mass(a, b)
            centroids[i] = num / max(den, 1e-30)
        # The start grid lo + (hi - lo) i / n is mirrored only up to rounding.  The reference's
        # symmetric quadrature nodes return exactly mirrored centroids (its middle boundary is
        # exactly 0.0 in the golden vectors); averaging the two mirror images reproduces that.
        centroids = [(centroids[i] - centroids[n_levels - 1 - i]) / 2 for i in range(n_levels)]
        boundaries = [(centroids[i] + centroids[i + 1]) / 2 for i in range(n_levels - 1)]
    return centroids, boundaries


def make_codebook(d: int = 128, bits: int = 3):
    """fp32 arrays of the codebook (turboquant/core/codebook.py:57-79)."""
    c, b = solve_codebook(d, bits)
    return np.asarray(c, dtype=F32), np.asarray(b, dtype=F32)


def make_wht_matrix(d: int) -> np.ndarray:
    """Normalised Sylvester Walsh-Hadamard matrix, fp32.

    turboquant/core/rotation.py:28-44: start from [[1]], double by
    [[H,H],[H,-H]] and divide by sqrt(2) (a Python float, applied in fp32)
    at each level.
    """
    H = np.array([[1.0]], dtype=F32)
    while H.shape[0] < d:
        H = (np.block([[H, H], [H, -H]]).astype(F32) / F32(math.sqrt(2))).astype(F32)
    return H[:d, :d]


# ---------------------------------------------------------------------------
# PolarQuant compression (the CPU path of the reference)
# ---------------------------------------------------------------------------


def polarquant_compress(x, centroids, boundaries, bits: int, use_qjl: bool = True,
                        rotation_matrix: Optional[np.ndarray] = None) -> dict:
    """turboquant/core/quantizer.py:111-183, fp32 throughout.

    x [N, D] (or [B, H, D]).  Returns the same dict keys as the reference:
    indices (int64), norms, k_mse_rot, and with use_qjl signs (+-1 fp32) and
    rot_residual_norm.
    """
    x = np.asarray(x)
    orig_shape = x.shape
    if x.ndim == 3:
        x = x.reshape(-1, x.shape[-1])
    x = x.astype(F32)
    centroids = np.asarray(centroids, dtype=F32)
    boundaries = np.asarray(boundaries, dtype=F32)
    # :142-145  rotation (skipped when the input is already rotated)
    if rotation_matrix is not None:
        x_rot = (x @ rotation_matrix.astype(F32)).astype(F32)
    else:
        x_rot = x
    # :148-149  norm of the ROTATED vector, true division by (norm + 1e-8)
    norms = np.sqrt(np.sum(x_rot * x_rot, axis=-1, dtype=F32)).astype(F32)
    x_n = (x_rot / (norms[:, None] + F32(1e-8))).astype(F32)
    # :152-153  searchsorted(right=False): idx = #{j : b_j < u}; ties go down
    idx = np.searchsorted(boundaries, x_n.reshape(-1), side="left").astype(np.int64)
    idx = np.clip(idx, 0, 2 ** bits - 1).reshape(x_n.shape)
    # :156-157
    recon = centroids[idx]
    k_mse_rot = (recon * norms[:, None]).astype(F32)
    out = {"indices": idx, "norms": norms, "k_mse_rot": k_mse_rot}
    if use_qjl:
        # :167-172  residual in rotated space, signs with 0 -> +1
        resid = ((x_n - recon) * norms[:, None]).astype(F32)
        rnorm = np.sqrt(np.sum(resid * resid, axis=-1, dtype=F32)).astype(F32)
        signs = np.where(resid < 0, F32(-1.0), F32(1.0)).astype(F32)
        out["signs"] = signs
        out["rot_residual_norm"] = rnorm
    if len(orig_shape) == 3:
        for k in ("indices", "k_mse_rot", "signs"):
            if k in out:
                out[k] = out[k].reshape(orig_shape)
    return out


# ---------------------------------------------------------------------------
# Packed formats (contiguous API)
# ---------------------------------------------------------------------------


def pack_2bit(idx: np.ndarray) -> np.ndarray:
    """4 indices per byte, LSB first (turboquant/kernels/packed_compress.py:80-90)."""
    i = idx.astype(np.uint8).reshape(idx.shape[0], -1, 4)
    return (i[..., 0] | (i[..., 1] << 2) | (i[..., 2] << 4) | (i[..., 3] << 6)).astype(np.uint8)


def unpack_2bit(packed: np.ndarray, D: int) -> np.ndarray:
    """turboquant/kernels/packed_compress.py:145-148."""
    p = packed.astype(np.int32)
    return np.stack([p & 3, (p >> 2) & 3, (p >> 4) & 3, (p >> 6) & 3], axis=-1).reshape(packed.shape[0], D).astype(np.int8)


def pack_4bit(idx: np.ndarray) -> np.ndarray:
    """Low nibble = even index, high nibble = odd (turboquant/integration/tq_fp4_backend.py:148-151)."""
    i = idx.astype(np.uint8)
    return (i[:, 0::2] | (i[:, 1::2] << 4)).astype(np.uint8)


def unpack_4bit(packed: np.ndarray, D: int) -> np.ndarray:
    p = packed.astype(np.int32)
    return np.stack([p & 15, (p >> 4) & 15], axis=-1).reshape(packed.shape[0], D).astype(np.int8)


def pack_3bit(idx: np.ndarray) -> np.ndarray:
    """Little-endian bit stream, dim d at bit 3d (48 bytes for D=128).

    The reference has only the decoder (turboquant/kernels/sparse_v.py:57-60,
    94-95: ((B[3d>>3] | B[(3d>>3)+1] << 8) >> (3d & 7)) & 7); this packer is
    its inverse.
    """
    N, D = idx.shape
    bits = ((idx.astype(np.uint8)[:, :, None] >> np.arange(3, dtype=np.uint8)) & 1).reshape(N, D * 3)
    return np.packbits(bits, axis=1, bitorder="little")


def unpack_3bit(packed: np.ndarray, D: int) -> np.ndarray:
    """turboquant/kernels/sparse_v.py:57-60,94-95."""
    p = packed.astype(np.int32)
    p = np.concatenate([p, np.zeros((p.shape[0], 1), np.int32)], axis=1)
    d = np.arange(D)
    bp = d * 3
    bi, bo = bp >> 3, bp & 7
    return (((p[:, bi] | (p[:, bi + 1] << 8)) >> bo) & 7).astype(np.int8)


def pack_indices(idx: np.ndarray, bits: int) -> np.ndarray:
    return {2: pack_2bit, 3: pack_3bit, 4: pack_4bit}[bits](idx)


def unpack_indices(packed: np.ndarray, bits: int, D: int = 128) -> np.ndarray:
    return {2: unpack_2bit, 3: unpack_3bit, 4: unpack_4bit}[bits](packed, D)


def pack_1bit(sign_bits: np.ndarray) -> np.ndarray:
    """Byte j bit b = sign bit of dim 8j+b (turboquant/kernels/packed_compress.py:92-106)."""
    return np.packbits(sign_bits.astype(np.uint8), axis=1, bitorder="little")


def unpack_1bit(packed: np.ndarray, D: int) -> np.ndarray:
    """turboquant/kernels/packed_compress.py:150-154."""
    return np.unpackbits(packed.astype(np.uint8), axis=1, bitorder="little")[:, :D].astype(np.int8)


def permute_signs_for_chunked(signs_packed: np.ndarray, D: int = 128) -> np.ndarray:
    """Sequential -> stride-4 order: output bit 32c+i <- dim c+4i.

    turboquant/kernels/packed_compress.py:180-216.
    """
    shape = signs_packed.shape
    flat = signs_packed.reshape(-1, D // 8)
    bits = unpack_1bit(flat, D)
    perm = np.concatenate([bits[:, c::4] for c in range(4)], axis=1)
    return pack_1bit(perm).reshape(shape)


def compress_k_packed(K, centroids, boundaries, bits: int, rotation_matrix=None, permuted: bool = True,
                      sign_projection=None):
    """Packed K in the contiguous format of compress_k / compress_k_permuted.

    Return order of turboquant/kernels/packed_compress.py:177 (k_idx, k_signs,
    k_rnorm, k_norm), arithmetic of turboquant/core/quantizer.py:111-183,
    norms rounded to fp16 as at packed_compress.py:63,73.  sign_projection
    (PiST of packed_compress.py:75-77): the signs are those of
    (rotated residual) @ sign_projection instead of the rotated residual's own.
    """
    r = polarquant_compress(K, centroids, boundaries, bits, True, rotation_matrix)
    k_idx = pack_indices(r["indices"], bits)
    if sign_projection is None:
        positive = r["signs"] > 0
    else:
        x = np.asarray(K, dtype=F32).reshape(-1, np.asarray(K).shape[-1])
        x_rot = x if rotation_matrix is None else (x @ rotation_matrix.astype(F32)).astype(F32)
        x_n = (x_rot / (r["norms"][:, None] + F32(1e-8))).astype(F32)
        resid = ((x_n - np.asarray(centroids, dtype=F32)[r["indices"]]) * r["norms"][:, None]).astype(F32)
        positive = (resid @ np.asarray(sign_projection, dtype=F32)) >= 0
    k_signs = pack_1bit(positive)
    if permuted:
        k_signs = permute_signs_for_chunked(k_signs)
    return k_idx, k_signs, r["rot_residual_norm"].astype(np.float16), r["norms"].astype(np.float16)


def compress_v_packed(V, centroids, boundaries, bits: int, rotation_matrix=None):
    """(v_idx, v_norm) as turboquant/kernels/packed_compress.py:226-240."""
    r = polarquant_compress(V, centroids, boundaries, bits, False, rotation_matrix)
    return pack_indices(r["indices"], bits), r["norms"].astype(np.float16)


# ---------------------------------------------------------------------------
# Attention
# ---------------------------------------------------------------------------


def attention_unpacked_ref(Q, Q_proj, K_mse_rot, signs_float, k_r_norm, V_mse_rot, corr_scale):
    """fp32 truth of the asymmetric estimator (turboquant/kernels/packed_attention.py:273-284).

    Q, Q_proj [BH, D]; K_mse_rot, signs_float, V_mse_rot [BH, Sk, D]; k_r_norm [BH, Sk].
    """
    Q = Q.astype(F32)
    Q_proj = Q_proj.astype(F32)
    score_mse = np.einsum("bd,bsd->bs", Q, K_mse_rot.astype(F32)).astype(F32)
    K_qjl = (signs_float.astype(F32) * k_r_norm.astype(F32)[..., None] * F32(corr_scale)).astype(F32)
    score_qjl = np.einsum("bd,bsd->bs", Q_proj, K_qjl).astype(F32)
    scores = score_mse + score_qjl
    scores = scores - scores.max(axis=-1, keepdims=True)
    e = np.exp(scores).astype(F32)
    attn = e / e.sum(axis=-1, keepdims=True)
    return np.einsum("bs,bsd->bd", attn, V_mse_rot.astype(F32)).astype(F32)


def packed_attention(Q, Q_proj, k_idx_packed, k_signs_perm, k_r_norm, k_norm,
                     v_idx_packed, v_norm, centroids, corr_scale, bits: int = 2):
    """Oracle of packed_attention (turboquant/kernels/packed_attention.py:290-344).

    Unpacks exactly as the reference's self-check does (:383-390) and applies
    attention_unpacked_ref.  Signs arrive in the permuted (stride-4) order and
    are put back in dimension order first.  Returns fp32 [BH, D].
    """
    BH, D = Q.shape
    Sk = k_r_norm.shape[1]
    centroids = np.asarray(centroids, dtype=F32)
    kidx = unpack_indices(k_idx_packed.reshape(BH * Sk, -1), bits, D).reshape(BH, Sk, D)
    vidx = unpack_indices(v_idx_packed.reshape(BH * Sk, -1), bits, D).reshape(BH, Sk, D)
    pb = unpack_1bit(k_signs_perm.reshape(BH * Sk, -1), D)  # permuted bit 32c+i <- dim c+4i
    sb = np.empty_like(pb)
    for c in range(4):
        sb[:, c::4] = pb[:, c * (D // 4):(c + 1) * (D // 4)]
    sb = sb.reshape(BH, Sk, D)
    K_mse = centroids[kidx.astype(np.int64)] * k_norm.astype(F32)[..., None]
    V_mse = centroids[vidx.astype(np.int64)] * v_norm.astype(F32)[..., None]
    signs = sb.astype(F32) * 2 - 1
    # The reference kernel rounds Q_proj*corr_scale to the query dtype (:318);
    # the truth it is compared against does not, and neither does this oracle.
    return attention_unpacked_ref(Q, Q_proj, K_mse, signs, k_r_norm.astype(F32), V_mse, corr_scale)


def paged_decode(q_rot, q_proj, k_fields: dict, v_fields: dict, block_tables, seq_lens,
                 k_centroids, v_centroids, sm_scale: float, corr_scale: float,
                 block_size: int, sparse_thresh: Optional[float] = None, return_stats: bool = False):
    """Paged + GQA decode attention over LOGICAL cache fields.

    q_rot, q_proj: [num_seqs, Hq, D] (already in rotated space; q_proj = S q_rot).
    k_fields: {"idx": int [num_blocks, block_size, Hkv, D], "norm": f16/f32
               [num_blocks, block_size, Hkv], and when QJL is on "signs" (0/1)
               [num_blocks, block_size, Hkv, D] and "rnorm"}.
    v_fields: {"idx", "norm"}.

    Structure: block-table walk and kv_h = h // (Hq/Hkv) of
    turboquant/kernels/fp4_paged_attention.py:62-106 (the same mapping as
    turboquant/kernels/sparse_v.py:48); estimator of
    turboquant/kernels/packed_attention.py:273-284; softmax scale applied to
    the logits as sparse_v.py:51.  With sparse_thresh set, the skip rule of
    sparse_v.py:108-123,149 is applied one block (page) at a time with the
    running maximum: a position's V term is dropped when the group maximum of
    exp(s - m_running) is <= thresh, while its p still enters the denominator.
    """
    ns, Hq, D = q_rot.shape
    Hkv = k_fields["idx"].shape[2]
    G = Hq // Hkv
    kc = np.asarray(k_centroids, dtype=F32)
    vc = np.asarray(v_centroids, dtype=F32)
    use_qjl = "signs" in k_fields
    out = np.zeros((ns, Hq, D), dtype=F32)
    skipped = 0
    total = 0
    for s in range(ns):
        L = int(seq_lens[s])
        if L == 0:
            continue
        nblk = (L + block_size - 1) // block_size
        blks = np.asarray(block_tables[s, :nblk]).astype(np.int64)
        for kh in range(Hkv):
            kidx = k_fields["idx"][blks, :, kh].reshape(nblk * block_size, D)[:L].astype(np.int64)
            kn = np.asarray(k_fields["norm"][blks, :, kh]).reshape(-1)[:L].astype(F32)
            vidx = v_fields["idx"][blks, :, kh].reshape(nblk * block_size, D)[:L].astype(np.int64)
            vn = np.asarray(v_fields["norm"][blks, :, kh]).reshape(-1)[:L].astype(F32)
            K = kc[kidx] * kn[:, None]
            V = vc[vidx] * vn[:, None]
            qs = q_rot[s, kh * G:(kh + 1) * G].astype(F32)            # [G, D]
            scores = qs @ K.T
            if use_qjl:
                sg = k_fields["signs"][blks, :, kh].reshape(nblk * block_size, D)[:L].astype(F32) * 2 - 1
                krn = np.asarray(k_fields["rnorm"][blks, :, kh]).reshape(-1)[:L].astype(F32)
                qp = q_proj[s, kh * G:(kh + 1) * G].astype(F32)
                scores = scores + (qp @ (sg * krn[:, None] * F32(corr_scale)).T)
            scores = (scores * F32(sm_scale)).astype(F32)           # [G, L]
            if sparse_thresh is None:
                m = scores.max(axis=1, keepdims=True)
                p = np.exp(scores - m).astype(F32)
                out[s, kh * G:(kh + 1) * G] = (p @ V) / p.sum(axis=1, keepdims=True)
            else:
                m_run = np.full((G,), -np.inf, dtype=F32)
                l_run = np.zeros((G,), dtype=F32)
                acc = np.zeros((G, D), dtype=F32)
                for b in range(nblk):
                    lo, hi = b * block_size, min((b + 1) * block_size, L)
                    sc = scores[:, lo:hi]
                    m_new = np.maximum(m_run, sc.max(axis=1))
                    p = np.exp(sc - m_new[:, None]).astype(F32)
                    alpha = np.exp(m_run - m_new).astype(F32)
                    acc *= alpha[:, None]
                    keep = p.max(axis=0) > F32(sparse_thresh)     # group max per position
                    total += hi - lo
                    skipped += int((~keep).sum())
                    acc += (p * keep[None, :]) @ V[lo:hi]
                    l_run = l_run * alpha + p.sum(axis=1)
                    m_run = m_new
                out[s, kh * G:(kh + 1) * G] = acc / l_run[:, None]
    if return_stats:
        return out, {"positions": total, "skipped": skipped}
    return out


# ---------------------------------------------------------------------------
# The CPU round trip the reference can run itself (turbo3 + QJL, 128-dim heads, seed 0)
# ---------------------------------------------------------------------------


def roundtrip_config1(K, V, q, bits: int = 3):
    """K, V fp32 [N, D], q [1, D]; turbo-`bits` with QJL; returns fp32 [1, D] in original space.

    Rotation + polarquant_compress (turboquant/core/quantizer.py:111-183), the
    asymmetric score of turboquant/kernels/packed_attention.py:273-284 with
    S = I (signs are taken of the rotated residual itself, quantizer.py:169-172)
    and corr_scale = sqrt(pi/2)/D (turboquant/kernels/attention.py:246),
    softmax scale 1/sqrt(D), MSE-V weighted sum, de-rotation out @ H
    (turboquant/integration/vllm_backend.py:158-176).
    """
    D = K.shape[1]
    H = make_wht_matrix(D)
    c, b = make_codebook(D, bits)
    ck = polarquant_compress(K, c, b, bits, True, H)
    cv = polarquant_compress(V, c, b, bits, False, H)
    q_rot = (q.astype(F32) @ H).astype(F32)
    cs = math.sqrt(math.pi / 2) / D
    sm = 1.0 / math.sqrt(D)
    out_rot = attention_unpacked_ref(
        q_rot * F32(sm), q_rot * F32(sm), ck["k_mse_rot"][None], ck["signs"][None],
        ck["rot_residual_norm"][None], cv["k_mse_rot"][None], cs)
    return (out_rot @ H).astype(F32)
