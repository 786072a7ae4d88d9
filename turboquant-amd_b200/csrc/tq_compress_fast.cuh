// Paged KV compression, fast path: tensor-core WHT + table-driven bucketize on the FMA pipe.
//
// Included by tq_compress.cu after the generic pieces (PagedParams, place_item, compress_items_generic).
//
// The generic path spends most of its issue slots in the half-rate integer/compare pipe (binary-search
// bucketize, select chains, shift-or packing) and in seven butterfly stages.  This path computes the same
// indices, signs and norms with far fewer, full-rate instructions:
//
//  * rotation (fp16 / bf16 inputs): the 128-point WHT is split by index bits.  Four bits are a 16-point transform
//    done by one m16n8k16 MMA against a constant +-1 matrix (the inputs go in exactly as loaded, the products
//    +-x are exact, accumulation is fp32), the other three are butterfly stages in registers; a lane group's
//    layout stays the one of the generic path (lane j of 4 owns dims 32 j .. 32 j + 31), so there is no shuffle.
//    The norm comes from MMAs too (diagonal of X X^T) and is known before the rotation.
//  * element arithmetic two at a time: sm_100 f32x2 instructions (fma / mul / add / sub on register pairs) do
//    the butterflies, the exactly rounded quotient u = x / (n + 1e-8) and the residual energy for two adjacent
//    dims per instruction.
//  * bucketize: u in [-1, 1] is mapped to one of 129 cells of width 1/64; no cell holds more than one
//    boundary (checked when the table is built; Lloyd-Max boundaries for 128 dims are >= 0.022 apart).  The
//    cell's table entry gives lo = #{boundaries below the cell}, and NB = -b * 2^126 for the boundary b inside
//    the cell (-inf when there is none), so  t = sat(u * 2^126 + NB)  is exactly [u > b]  (ties stay down,
//    as searchsorted(right=False)), and idx = lo + t.  The entry also carries c[lo] and c[lo+1], so the
//    centroid is c[lo] (1 - t) + c[lo+1] t: two FMAs whose result is exactly one of the two.
//  * packing: the four indices of a chunk of adjacent dims are combined by three FMAs into one float (one index
//    per nibble, exact below 2^24) and converted once; residual signs are shifted in with funnel shifts.
//  * rows are staged through shared memory with cp.async one group of items ahead of their use.
//
// On an already rotated input the indices, signs and norms are those of the generic path bit for bit, except
// where u or the residual falls in the subnormal range (|.| < 2^-126).  With the rotation done here, the
// rotated values themselves differ from a butterfly or a matrix product in the last bits, as any two
// summation orders do.  A codebook with two boundaries inside one cell makes the whole grid take the generic
// path; fp32 inputs and already rotated inputs take the table-driven quantizer without the tensor-core part.
#pragma once

namespace tq {
namespace {

// Compile-time tunables.  The tensor-core loop needs ~128 registers to stay clear of spills (a spilled build at 80
// registers and 24 warps per SM measured 1.3-1.6x slower than this one at 16 warps per SM).  One CTA of 16 warps
// per SM builds the tables once for all of them: 4 % faster than two CTAs of 8 warps.
#ifndef TQ_CMP_MINBLOCKS
#define TQ_CMP_MINBLOCKS 1
#endif
#ifndef TQ_CMP_WARPS
#define TQ_CMP_WARPS 16
#endif
constexpr int kCellScale = 64;   // cells per unit of u
constexpr int kCells = 2 * kCellScale + 1;
constexpr int kFastWarps = TQ_CMP_WARPS;
constexpr int kFastItemsPerCta = kFastWarps * kItemsPerWarp;
constexpr uint32_t kMagicBits = 0x4B400000u;   // 1.5 * 2^23: adding it leaves an integer in the low mantissa bits
constexpr float kMagic = 12582912.f;

__device__ __forceinline__ float big() { return __uint_as_float(0x7E800000u); }   // 2^126

__device__ __forceinline__ float fma_sat(float a, float b, float c) {
    float d;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ float4 lds128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ float2 lds64(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}

// D = A B with a zero accumulator (no register moves to clear one).
template <bool BF16>
__device__ __forceinline__ void mma_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1) {
    const float z = 0.f;
    if constexpr (BF16) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
    }
}

// ---- tables ------------------------------------------------------------------------------------------
// Each cell is stored once per lane residue so that a warp's lookups never collide on a bank:
// wide entries (16 B: NB, lo, c[lo], c[lo+1]) 8 copies, narrow entries (8 B: NB, lo) 16 copies; 128 B per cell.
constexpr int kCellStride = 128;
constexpr int kTableBytes = kCells * kCellStride;

// Scans sorted boundaries for one cell.  Returns how many boundaries fall inside the cell.
__device__ __forceinline__ int scan_cell(int cell, const float* __restrict__ b, int nb, int& lo, float& nbv) {
    const float center = static_cast<float>(cell - kCellScale) * (1.f / kCellScale);
    const float half = 0.5f / kCellScale + 1.f / 1048576.f;   // rounding of the cell index is absorbed by the margin
    const float lo_e = center - half, hi_e = center + half;
    int inside = 0;
    float bin = 0.f;
    lo = 0;
    for (int j = 0; j < nb; ++j) {
        const float bj = __ldg(b + j);
        lo += bj < lo_e ? 1 : 0;
        if (bj >= lo_e && bj <= hi_e) {
            ++inside;
            bin = bj;
        }
    }
    nbv = inside ? -(bin * big()) : __uint_as_float(0xff800000u);
    return inside;
}

template <int BITS, bool WIDE>
__device__ void build_table(unsigned char* tab, const float* __restrict__ b, const float* __restrict__ c, int* bad) {
    for (int cell = threadIdx.x; cell < kCells; cell += blockDim.x) {
        int lo;
        float nbv;
        const int inside = scan_cell(cell, b, (1 << BITS) - 1, lo, nbv);
        if (inside > 1) atomicOr(bad, 1);
        if constexpr (WIDE) {
            const float c_lo = __ldg(c + lo);
            const float c_hi = lo + 1 < (1 << BITS) ? __ldg(c + lo + 1) : c_lo;
            const float4 e = make_float4(nbv, static_cast<float>(lo), c_lo, c_hi);
#pragma unroll
            for (int r = 0; r < 8; ++r) reinterpret_cast<float4*>(tab + cell * kCellStride)[r] = e;
        } else {
            const float2 e = make_float2(nbv, static_cast<float>(lo));
#pragma unroll
            for (int r = 0; r < 16; ++r) reinterpret_cast<float2*>(tab + cell * kCellStride)[r] = e;
        }
    }
}

// ---- packed output (bit positions: turboquant/kernels/paged_layout.py) ------------------------------------
// Both parts of a page are made of 16-bit fields of four nibbles; a chunk of four adjacent dims fills one field
// (4-bit, 3-bit) or half the bits of one (2-bit).  K: field 2 w + h is half h of index word w of the lane's
// quarter sub-record.  V: field BITS gg + j is plane j of dim group 2 quarter + gg.  3-bit indices of the last
// two chunks (K) / of every fourth chunk (V) are spread over the spare top bits of the nibbles: bit b of the
// index in nibble e goes to bit 4 e + 3 of field / word b.
struct Packed {
    uint32_t word[4];    // K: the BITS index words of the lane's quarter sub-record
    uint32_t field[8];   // V: 2 * BITS fields (only the low 16 bits of each are meaningful)
    uint32_t signs;      // bit l = 1 when the residual of local dim l is >= 0
    float norm, rnorm;
};

// ---- two fp32 per instruction (sm_100 f32x2 arithmetic on 64-bit register pairs) ----------------------------
typedef unsigned long long f2;
__device__ __forceinline__ f2 f2pack(float lo, float hi) {
    f2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2unpack(f2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f2 f2dup(float v) { return f2pack(v, v); }
__device__ __forceinline__ f2 f2fma(f2 a, f2 b, f2 c) {
    f2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ f2 f2mul(f2 a, f2 b) {
    f2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f2 f2add(f2 a, f2 b) {
    f2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f2 f2sub(f2 a, f2 b) {
    f2 r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// Per-vector constants of the element loop, duplicated into both halves of a pair.
struct VecConsts {
    f2 inv, nden, inv64, n;
    uint32_t tab;
};

// One pair of adjacent dims (a = even, b = odd): returns their indices as floats; with QJL also accumulates the
// squared residuals and shifts the sign bits of the two residuals into `sacc` (1 = negative; pairs must come in
// descending order).  A residual that underflows to -0.0 is the one case that reads as negative here while the
// reference's (e >= 0) calls it positive.
// EXACT: u = y / den correctly rounded (one reciprocal multiply plus two correction FMAs), as the reference's true
// division; needed where the input is already rotated and the indices must be the reference's bit for bit.  Where the
// rotation is done here its own rounding already moves u in the last bits, so the kernels that rotate take the plain
// product y * (1 / den), at most one ulp away: a different index only for u within an ulp of a boundary (~1e-7 of
// the coordinates, inside the rotation's 1e-4 allowance).
template <bool QJL, bool EXACT = true>
__device__ __forceinline__ void quant_pair(f2 y, const VecConsts& vc, f2& rr, uint32_t& sacc, float& kfa, float& kfb) {
    const float kBig = big();
    const f2 q0 = f2mul(y, vc.inv);
    // The cell only needs the quotient to ~1e-6: take it from the first approximation so the lookup starts early.
    const f2 cellf = f2fma(y, vc.inv64, f2dup(kMagic + kCellScale));   // low mantissa bits: round(scale u) + scale
    const f2 u = EXACT ? f2fma(f2fma(q0, vc.nden, y), vc.inv, q0) : q0;   // y / den (correctly rounded when EXACT); |u| <= 1
    float ua, ub, cfa, cfb;
    f2unpack(u, ua, ub);
    f2unpack(cellf, cfa, cfb);
    const uint32_t addr_a = __float_as_uint(cfa) * static_cast<uint32_t>(kCellStride) + vc.tab;
    const uint32_t addr_b = __float_as_uint(cfb) * static_cast<uint32_t>(kCellStride) + vc.tab;
    if constexpr (QJL) {
        const float4 ea = lds128(addr_a), eb = lds128(addr_b);   // NB, lo, c[lo], c[lo+1]
        const float ta = fma_sat(ua, kBig, ea.x), tb = fma_sat(ub, kBig, eb.x);   // [u > boundary of the cell]
        const float ca = fmaf(ta, ea.w, fmaf(-ta, ea.z, ea.z));   // t is 0 or 1: exactly c[lo] or c[lo+1]
        const float cb = fmaf(tb, eb.w, fmaf(-tb, eb.z, eb.z));
        const f2 r = f2mul(f2sub(u, f2pack(ca, cb)), vc.n);
        rr = f2fma(r, r, rr);
        float ra, rb;
        f2unpack(r, ra, rb);
        // shift the two sign bits in from the right (1 = negative; the caller inverts): one funnel shift each
        sacc = __funnelshift_l(__float_as_uint(rb), sacc, 1);
        sacc = __funnelshift_l(__float_as_uint(ra), sacc, 1);
        kfa = ea.y + ta;
        kfb = eb.y + tb;
    } else {
        const float2 ea = lds64(addr_a), eb = lds64(addr_b);     // NB, lo
        kfa = ea.y + fma_sat(ua, kBig, ea.x);
        kfb = eb.y + fma_sat(ub, kBig, eb.x);
    }
}

// cv[c]: the four indices of chunk c (dims 4 c .. 4 c + 3), one per nibble, as a float.
template <int BITS, bool ISV>
__device__ __forceinline__ void assemble_indices(const float (&cv)[8], Packed& out) {
    // Adding 2^23 leaves a field's integer in the low mantissa bits; prmt 0x5410 joins two low halves.
    const float kInt = 8388608.f;
    if constexpr (ISV) {
        // V: field BITS gg + j of dim group gg (chunks 4 gg .. 4 gg + 3).
#pragma unroll
        for (int gg = 0; gg < 2; ++gg) {
            if constexpr (BITS == 4) {
#pragma unroll
                for (int j = 0; j < 4; ++j) out.field[4 * gg + j] = __float_as_uint(cv[4 * gg + j] + kInt);
            } else if constexpr (BITS == 3) {
                const uint32_t m = __float_as_uint(cv[4 * gg + 3] + kInt);   // fourth chunk: bit b of nibble e -> field b bit 4 e + 3
#pragma unroll
                for (int b = 0; b < 3; ++b)
                    out.field[3 * gg + b] = __float_as_uint(cv[4 * gg + b] + kInt) | ((m << (3 - b)) & 0x8888u);
            } else {
                out.field[2 * gg] = __float_as_uint(fmaf(cv[4 * gg + 1], 4.f, cv[4 * gg]) + kInt);
                out.field[2 * gg + 1] = __float_as_uint(fmaf(cv[4 * gg + 3], 4.f, cv[4 * gg + 2]) + kInt);
            }
        }
    } else {
        // K: 16-bit half h of index word w.
        if constexpr (BITS == 4) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                out.word[j] = prmt(__float_as_uint(cv[2 * j] + kInt), __float_as_uint(cv[2 * j + 1] + kInt), 0x5410);
        } else if constexpr (BITS == 3) {
            const uint32_t m = prmt(__float_as_uint(cv[6] + kInt), __float_as_uint(cv[7] + kInt), 0x5410);
#pragma unroll
            for (int b = 0; b < 3; ++b)
                out.word[b] = prmt(__float_as_uint(cv[2 * b] + kInt), __float_as_uint(cv[2 * b + 1] + kInt), 0x5410) |
                              ((m << (3 - b)) & 0x88888888u);
        } else {
            // word w: chunks 4 w + {0, 2} in the low half (the second shifted by 2 bits), 4 w + {1, 3} in the high half
#pragma unroll
            for (int j = 0; j < 2; ++j)
                out.word[j] = prmt(__float_as_uint(fmaf(cv[4 * j + 2], 4.f, cv[4 * j]) + kInt),
                                   __float_as_uint(fmaf(cv[4 * j + 3], 4.f, cv[4 * j + 1]) + kInt), 0x5410);
        }
    }
}

// Contiguous outputs (reference byte layouts: 2-bit four per byte LSB first, 4-bit low nibble first, 3-bit a
// little-endian bit stream): cv[c] holds the four indices of chunk c densely, idx_e at bit BITS * e, so a chunk is
// 4 * BITS bits of the lane's BITS output words.
template <int BITS>
__device__ __forceinline__ void assemble_contig(const float (&cv)[8], Packed& out) {
    const float kInt = 8388608.f;
    uint32_t u[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) u[c] = __float_as_uint(cv[c] + kInt);   // 0x4B000000 | value
    if constexpr (BITS == 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) out.word[j] = prmt(u[2 * j], u[2 * j + 1], 0x5410);
    } else if constexpr (BITS == 2) {
#pragma unroll
        for (int j = 0; j < 2; ++j)
            out.word[j] = prmt(prmt(u[4 * j], u[4 * j + 1], 0x0040), prmt(u[4 * j + 2], u[4 * j + 3], 0x0040), 0x5410);
    } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) u[c] &= 0xfffu;
        out.word[0] = u[0] | (u[1] << 12) | (u[2] << 24);
        out.word[1] = (u[2] >> 8) | (u[3] << 4) | (u[4] << 16) | (u[5] << 28);
        out.word[2] = (u[5] >> 4) | (u[6] << 8) | (u[7] << 20);
    }
}

// y: this lane's 32 rotated values as 16 pairs of adjacent dims, still to be multiplied by `scale` (2^-3.5 after
// the unnormalised WHT, else 1).  tab: shared address of this lane's copy of cell 0, minus kMagicBits * 128.
// The scale is applied to the norm only: u = (scale y) / (n + 1e-8) is computed as y / ((n + 1e-8) / scale),
// which is the same number up to the rounding the rotation itself carries; with scale = 1 nothing changes.
template <int BITS, bool QJL, bool ISV, bool CONTIG = false>
__device__ __forceinline__ void quantize_fast(f2 (&y)[16], float scale, float inv_scale, uint32_t tab, Packed& out) {
    constexpr float kStep = CONTIG ? static_cast<float>(1 << BITS) : 16.f;   // spacing of a chunk's four indices
    f2 sa = f2dup(0.f), sb = f2dup(0.f);
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        sa = f2fma(y[i], y[i], sa);
        sb = f2fma(y[i + 1], y[i + 1], sb);
    }
    float s0, s1, s2, s3;
    f2unpack(sa, s0, s1);
    f2unpack(sb, s2, s3);
    const float ny = sqrtf(group_sum((s0 + s1) + (s2 + s3)));
    // NaN or overflow somewhere in the vector: quantize a zero vector so that the table lookups stay in range
    // (the stored norm still shows the bad value).
    const bool finite = ny < __uint_as_float(0x7f800000u);
    if (!finite) {
#pragma unroll
        for (int i = 0; i < 16; ++i) y[i] = f2dup(0.f);
    }
    const float n_out = ny * scale;
    const float n = finite ? n_out : 0.f;
    const float den = (n + 1e-8f) * inv_scale;
    const float inv = __frcp_rn(den);
    VecConsts vc;
    vc.inv = f2dup(inv);
    vc.nden = f2dup(-den);
    vc.inv64 = f2dup(inv * kCellScale);
    vc.n = f2dup(n);
    vc.tab = tab;
    // Chunk c = dims 4 c .. 4 c + 3 -> one float holding its four indices, one per nibble.
    float cv[8];
    f2 rr = f2dup(0.f);
    uint32_t sg[2] = {0u, 0u};
#pragma unroll
    for (int c = 7; c >= 0; --c) {
        float k0, k1, k2, k3;
        quant_pair<QJL>(y[2 * c + 1], vc, rr, sg[c >> 2], k2, k3);
        quant_pair<QJL>(y[2 * c], vc, rr, sg[c >> 2], k0, k1);
        cv[c] = fmaf(fmaf(fmaf(k3, kStep, k2), kStep, k1), kStep, k0);
    }
    if constexpr (CONTIG) assemble_contig<BITS>(cv, out);
    else assemble_indices<BITS, ISV>(cv, out);
    if constexpr (QJL) {
        float ra, rb;
        out.signs = ~prmt(sg[0], sg[1], 0x5410);
        f2unpack(rr, ra, rb);
        out.rnorm = sqrtf(group_sum(ra + rb));
    } else {
        out.signs = 0u;
        out.rnorm = 0.f;
    }
    out.norm = n_out;
}

// ---- rotation + quantization of one fp16 / bf16 row on the tensor cores -----------------------------------------
// A lane's 64 bytes of a row are four 16-byte pieces j = 0..3 = dims 8 j .. 8 j + 7; piece j goes into an m16n8k16
// MMA exactly as loaded, as its A fragment (a0..a3 = the four words): the 8 items of the warp are rows 0..7 with
// the words whose dim bit 1 is 0, rows 8..15 the same items with dim bit 1 = 1; the 16 k-slots are dim bit 0
// (element within a word), dim bits 5,6 (lane within the group of four) and dim bit 2 (word pair).
//  * Rotation: against the constant +-1 matrix whose column n carries the same bit roles, lane (g, t) receives the
//    16-point transform over dim bits {0,2,5,6} for dim bits 5,6 = t - the 32 dims it owns - in two passes (dim bit
//    2 = nt).  The four outputs of MMA (j, nt) are the chunk of four adjacent dims 8 j + 4 nt .. + 3, as two
//    register pairs.  Dim bits {1,3,4} are three butterfly stages over the eight pairs of a pass.
//  * Norm: m16n8k8 MMAs with a word pair as A and one of its words as B accumulate <x_g, x_n> over the even
//    (rows 0..7) and the odd (rows 8..15) words; the diagonal is ||x||^2 = ||x H||^2 (H is orthonormal), so the
//    norm is known before the rotation and only half of the rotated values have to be live at a time.
struct WhtFragments {
    uint32_t b0[2], b1[2];   // B operand (16 x 8, +-1.0 in the input type) for nt = 0, 1
};

__device__ __forceinline__ WhtFragments make_wht_fragments(int lane, bool bf16) {
    const int g = lane >> 2, tig = lane & 3;
    const uint32_t one = bf16 ? 0x3F80u : 0x3C00u;
    WhtFragments f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
        const int n = g + 8 * nt;
        const uint32_t s00 = (__popc((2 * tig) & n) & 1) << 15, s01 = (__popc((2 * tig + 1) & n) & 1) << 15;
        const uint32_t s10 = (__popc((2 * tig + 8) & n) & 1) << 15, s11 = (__popc((2 * tig + 9) & n) & 1) << 15;
        f.b0[nt] = (one | s00) | ((one | s01) << 16);
        f.b1[nt] = (one | s10) | ((one | s11) << 16);
    }
    return f;
}

// D (+)= A B, m16n8k8, fp32 accumulate; ZERO starts from a zero accumulator.
template <bool ZERO>
__device__ __forceinline__ void mma_k8(bool bf16, float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    const float z = 0.f;
    if (bf16) {
        if constexpr (ZERO)
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                         : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(b0), "f"(z));
        else
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(b0));
    } else {
        if constexpr (ZERO)
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                         : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(b0), "f"(z));
        else
            asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                         : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(b0));
    }
}

__device__ __forceinline__ void mma_zero(bool bf16, float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    if (bf16) mma_16816_zero<true>(d, a0, a1, a2, a3, b0, b1);
    else mma_16816_zero<false>(d, a0, a1, a2, a3, b0, b1);
}

// row: shared address of this lane's first 16-byte piece of a staged row (piece j is 512 bytes further).
__device__ __forceinline__ void read_staged(uint32_t row, bool live, uint32_t (&w)[16]) {
    if (live) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(w[4 * j]), "=r"(w[4 * j + 1]), "=r"(w[4 * j + 2]), "=r"(w[4 * j + 3])
                         : "r"(row + 512 * j));
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = 0u;
    }
}

// after_read() is called once the staged row has been read for the last time (the caller requests the next row
// into the same buffer there).
template <int BITS, bool QJL, bool ISV, bool CONTIG = false, class AfterRead>
__device__ __forceinline__ void compress_row_mma(uint32_t row, bool live, int lane, bool bf16, const WhtFragments& hf,
                                                 uint32_t tab, Packed& out, AfterRead after_read) {
    constexpr float kStep = CONTIG ? static_cast<float>(1 << BITS) : 16.f;   // spacing of a chunk's four indices
    uint32_t w[16];
    read_staged(row, live, w);
    // ||x||^2: even words on the diagonal of rows 0..7 of da, odd words on that of rows 8..15 of db
    float da[4], db[4];
    mma_k8<true>(bf16, da, w[0], w[1], w[0]);
    mma_k8<true>(bf16, db, w[0], w[1], w[1]);
#pragma unroll
    for (int m = 1; m < 8; ++m) {
        mma_k8<false>(bf16, da, w[2 * m], w[2 * m + 1], w[2 * m]);
        mma_k8<false>(bf16, db, w[2 * m], w[2 * m + 1], w[2 * m + 1]);
    }
    const int g = lane >> 2;
    const float diag = (g & 1) ? da[1] + db[3] : da[0] + db[2];   // column g sits in lane (g, g >> 1)
    const float ss = __shfl_sync(0xffffffffu, diag, (lane & ~3) | (g >> 1));
    // NaN or overflow somewhere in the vector: quantize a zero vector so that the table lookups stay in range (the
    // stored norm still shows the bad value).
    const bool finite = ss < __uint_as_float(0x7f800000u);
    if (!finite) live = false;
    const float n_out = sqrtf(ss);                                // = ||x H / sqrt(128)||
    const float n = finite ? n_out : 0.f;
    const float den = (n + 1e-8f) * 11.313708498984761f;          // the unnormalised transform is sqrt(128) larger
    const float inv = __frcp_rn(den);
    VecConsts vc;
    vc.inv = f2dup(inv);
    vc.nden = f2dup(-den);
    vc.inv64 = f2dup(inv * kCellScale);
    vc.n = f2dup(n);
    vc.tab = tab;
    float cv[8];
    f2 rr = f2dup(0.f);
    uint32_t sg = 0u;   // bit l = 1 when the residual of local dim l is negative
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
        if (nt == 1 || !live) read_staged(row, live, w);
        if (nt == 1) after_read();
        f2 y[8];   // pair 2 j + r = dims 8 j + 4 nt + 2 r + {0, 1}
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float d[4];
            mma_zero(bf16, d, w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3], hf.b0[nt], hf.b1[nt]);
            y[2 * j] = f2pack(d[0], d[1]);
            y[2 * j + 1] = f2pack(d[2], d[3]);
        }
#pragma unroll
        for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (!(i & h)) {
                    const f2 a = y[i], b = y[i + h];
                    y[i] = f2add(a, b);
                    y[i + h] = f2sub(a, b);
                }
            }
        }
#pragma unroll
        for (int j = 3; j >= 0; --j) {
            const int c = 2 * j + nt;   // chunk of dims 4 c .. 4 c + 3
            float k0, k1, k2, k3;
            uint32_t nib = 0u;
            quant_pair<QJL, false>(y[2 * j + 1], vc, rr, nib, k2, k3);
            quant_pair<QJL, false>(y[2 * j], vc, rr, nib, k0, k1);
            cv[c] = fmaf(fmaf(fmaf(k3, kStep, k2), kStep, k1), kStep, k0);
            if constexpr (QJL) sg |= nib << (4 * c);
        }
    }
    if constexpr (CONTIG) assemble_contig<BITS>(cv, out);
    else assemble_indices<BITS, ISV>(cv, out);
    if constexpr (QJL) {
        float ra, rb;
        out.signs = ~sg;
        f2unpack(rr, ra, rb);
        out.rnorm = sqrtf(group_sum(ra + rb));
    } else {
        out.signs = 0u;
        out.rnorm = 0.f;
    }
    out.norm = n_out;
}

// ---- input staging (fp16 / bf16 rows): global -> shared with cp.async, one group of items ahead --------------
// Every lane copies and later reads back only its own 64 bytes of a row, as four 16-byte pieces; piece i of lane
// l sits at uint4 index 32 i + l of the warp's buffer, so both the copies and the reads are conflict-free.
constexpr int kStagePerWarp = 2 * 4 * 32 * 16;   // K and V rows of 8 items: 4 KB

__device__ __forceinline__ void stage_row(uint4* buf, int lane, const void* base, int64_t elem_off, bool live) {
    if (live) {
        const uint16_t* src = static_cast<const uint16_t*>(base) + elem_off;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(buf + 32 * i + lane)), "l"(src + 8 * i)
                         : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// Waits until at most one of this thread's copy groups is still in flight.
__device__ __forceinline__ void wait_staged() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// Loads this lane's 32 elements of one row and returns them as fp32 pairs, rotated when asked but not yet
// scaled by 2^-3.5.  Path for fp32 inputs and for inputs that are already rotated.
__device__ __forceinline__ void fetch_plain(const void* base, int64_t elem_off, bool live, int dtype, bool rotate,
                                            int lane, f2 (&y)[16]) {
    float x[32];
    if (live) load32(base, elem_off, dtype, x);
    else {
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = 0.f;
    }
    if (rotate) fwht128(x, lane);
#pragma unroll
    for (int i = 0; i < 16; ++i) y[i] = f2pack(x[2 * i], x[2 * i + 1]);
}

// ---- stores ------------------------------------------------------------------------------------------------
template <int BITS, bool QJL>
__device__ __forceinline__ void store_k_fast(uint8_t* page, int t, int quarter, const Packed& q) {
    constexpr int NW = BITS + (QJL ? 1 : 0);
    constexpr int RK = 16 * NW;
    const uint32_t (&w)[4] = q.word;
    uint8_t* dst = page + t * RK + quarter * (RK / 4);
    if constexpr (NW == 4) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], QJL ? q.signs : w[BITS - 1]);
    } else if constexpr (NW == 2) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
    } else {
#pragma unroll
        for (int j = 0; j < BITS; ++j) reinterpret_cast<uint32_t*>(dst)[j] = w[j];
        if constexpr (QJL) reinterpret_cast<uint32_t*>(dst)[BITS] = q.signs;
    }
    if (quarter == 0) {
        reinterpret_cast<__half*>(page + 16 * RK)[norm_slot(t)] = __float2half_rn(q.norm);
        if constexpr (QJL) reinterpret_cast<__half*>(page + 16 * RK + 32)[norm_slot(t)] = __float2half_rn(q.rnorm);
    }
}

template <int BITS>
__device__ __forceinline__ void store_v_fast(uint8_t* vpart, int t, int quarter, const Packed& q) {
    const int pair = t >> 1, half = t & 1;
#pragma unroll
    for (int gg = 0; gg < 2; ++gg) {
        const int g = 2 * quarter + gg;
#pragma unroll
        for (int j = 0; j < BITS; ++j)
            *reinterpret_cast<uint16_t*>(vpart + ((j * 8 + pair) * 8 + g) * 4 + half * 2) =
                static_cast<uint16_t>(q.field[gg * BITS + j]);
    }
    if (quarter == 0) reinterpret_cast<__half*>(vpart + 256 * BITS)[norm_slot(t)] = __float2half_rn(q.norm);
}

// fp32 inputs and inputs that are already rotated: plain loads, shuffle WHT, the same table-driven quantizer.
// Out of line so that its registers do not weigh on the tensor-core loop.
template <int KB, int VB, bool QJL>
__device__ __noinline__ void compress_items_plain(const void* key, const void* value, int64_t ks_t, int64_t ks_h,
                                                  int64_t vs_t, int64_t vs_h, int dtype, bool rotate, ItemPlace w, int lane,
                                                  uint32_t ktab, uint32_t vtab) {
    constexpr int KPART = k_part_bytes(KB, QJL ? 1 : 0);
    const int quarter = lane & 3;
    const float scale = rotate ? kWhtScale : 1.f, inv_scale = rotate ? 11.313708498984761f : 1.f;
    f2 x[16];
    Packed q;
    fetch_plain(key, w.tok * ks_t + w.head * ks_h + 32 * quarter, w.live, dtype, rotate, lane, x);
    quantize_fast<KB, QJL, false>(x, scale, inv_scale, ktab, q);
    if (w.live) store_k_fast<KB, QJL>(w.page, w.t, quarter, q);
    fetch_plain(value, w.tok * vs_t + w.head * vs_h + 32 * quarter, w.live, dtype, rotate, lane, x);
    quantize_fast<VB, false, true>(x, scale, inv_scale, vtab, q);
    if (w.live) store_v_fast<VB>(w.page + KPART, w.t, quarter, q);
}

// ---- kernel -----------------------------------------------------------------------------------------------
// Persistent CTAs of 16 warps, one per SM: the two tables are built once per CTA, then the CTA strides over groups of 128
// (token, head) items, 8 per warp, first the key then the value of each item.
template <int KB, int VB, bool QJL>
__global__ void __launch_bounds__(kFastWarps * 32, TQ_CMP_MINBLOCKS) compress_paged_fast_kernel(const PagedParams p, int64_t n_groups) {
    constexpr int PAGE = page_bytes(KB, VB, QJL ? 1 : 0);
    constexpr int KPART = k_part_bytes(KB, QJL ? 1 : 0);
    extern __shared__ __align__(128) unsigned char tables[];
    __shared__ float csm[1 << KB];
    __shared__ int bad;
    if (threadIdx.x == 0) bad = 0;
    if (threadIdx.x < (1 << KB)) csm[threadIdx.x] = p.kc[threadIdx.x];
    __syncthreads();
    build_table<KB, QJL>(tables, p.kb, p.kc, &bad);
    build_table<VB, false>(tables + kTableBytes, p.vb, nullptr, &bad);
    __syncthreads();
    const bool generic = bad != 0;
    const int lane = threadIdx.x & 31, quarter = lane & 3, warp = threadIdx.x >> 5;
    constexpr uint32_t kBias = kMagicBits * static_cast<uint32_t>(kCellStride);   // modulo 2^32
    const uint32_t ktab = smem_u32(tables) + (QJL ? (lane & 7) * 16 : (lane & 15) * 8) - kBias;
    const uint32_t vtab = smem_u32(tables + kTableBytes) + (lane & 15) * 8 - kBias;
    const bool rotate = p.rotate != 0;
    const int64_t item0 = warp * kItemsPerWarp + (lane >> 2);   // + group * 64
    if (generic) {
        const PagedParams pc = p;   // the out-of-line call takes an address: keep the kernel parameters themselves in the constant bank
        for (int64_t grp = blockIdx.x; grp < n_groups; grp += gridDim.x)
            compress_items_generic<KB, VB, QJL>(pc, grp * kFastItemsPerCta + item0, lane, csm);
        return;
    }
    Packed q;
    if (rotate && p.in_dtype != TQ_DTYPE_F32) {
        // Tensor-core rotation.  Rows are staged through shared memory one group ahead: the key rows of the next
        // group are requested as soon as this group's have been consumed by the MMAs, the value rows likewise,
        // so every copy has a whole group's arithmetic to hide behind.
        const bool bf16 = p.in_dtype == TQ_DTYPE_BF16;
        uint4* kbuf = reinterpret_cast<uint4*>(tables + 2 * kTableBytes + warp * kStagePerWarp);
        uint4* vbuf = kbuf + 128;
        const uint32_t krow = smem_u32(kbuf + lane), vrow = smem_u32(vbuf + lane);
        const WhtFragments hf = make_wht_fragments(lane, bf16);
        // Only the identity (token, head) of the next group's item is carried across the loop body; where the
        // current item goes in the cache is looked up when its turn comes.
        int64_t grp = blockIdx.x;
        ItemId id = identify_item(p, grp * kFastItemsPerCta + item0);
        stage_row(kbuf, lane, p.key, id.tok * p.ks_t + id.head * p.ks_h + 32 * quarter, id.live);
        stage_row(vbuf, lane, p.value, id.tok * p.vs_t + id.head * p.vs_h + 32 * quarter, id.live);
        while (grp < n_groups) {
            const ItemPlace w = place_item<PAGE>(p, id, quarter);
            grp += gridDim.x;
            id.live = false;
            if (grp < n_groups) id = identify_item(p, grp * kFastItemsPerCta + item0);
            wait_staged();
            compress_row_mma<KB, QJL, false>(krow, w.live, lane, bf16, hf, ktab, q, [&] {
                stage_row(kbuf, lane, p.key, id.tok * p.ks_t + id.head * p.ks_h + 32 * quarter, id.live);
            });
            if (w.live) store_k_fast<KB, QJL>(w.page, w.t, quarter, q);
            wait_staged();
            compress_row_mma<VB, false, true>(vrow, w.live, lane, bf16, hf, vtab, q, [&] {
                stage_row(vbuf, lane, p.value, id.tok * p.vs_t + id.head * p.vs_h + 32 * quarter, id.live);
            });
            if (w.live) store_v_fast<VB>(w.page + KPART, w.t, quarter, q);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        for (int64_t grp = blockIdx.x; grp < n_groups; grp += gridDim.x)
            compress_items_plain<KB, VB, QJL>(p.key, p.value, p.ks_t, p.ks_h, p.vs_t, p.vs_h, p.in_dtype, rotate,
                                              place_item<PAGE>(p, grp * kFastItemsPerCta + item0, quarter), lane, ktab, vtab);
    }
}

// Small launches (the new tokens of one decode step): no tables to build, one group of 32 items per CTA.
template <int KB, int VB, bool QJL>
__global__ void __launch_bounds__(kWarpsPerCta * 32) compress_paged_small_kernel(const PagedParams p) {
    __shared__ float csm[1 << KB];
    if (threadIdx.x < (1 << KB)) csm[threadIdx.x] = p.kc[threadIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t item = (static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5)) * kItemsPerWarp + (lane >> 2);
    compress_items_generic<KB, VB, QJL>(p, item, lane, csm);
}

constexpr int64_t kSmallLaunchItems = 16384;   // below this the table set-up and the 512-thread CTAs of the fast kernel cost more than they save

template <int KB, int VB, bool QJL>
int launch_paged_tc(const PagedParams& p, cudaStream_t st);   // tq_compress_tc.cuh

template <int KB, int VB, bool QJL>
int launch_paged_fast(const PagedParams& p, cudaStream_t st) {
    if (p.n_items <= kSmallLaunchItems) {
        const unsigned grid = static_cast<unsigned>((p.n_items + kItemsPerCta - 1) / kItemsPerCta);
        compress_paged_small_kernel<KB, VB, QJL><<<grid, kWarpsPerCta * 32, 0, st>>>(p);
        return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
    }
    // on request: fp16 / bf16 rows that still need the rotation go to the tensor-memory kernel (rotation as one
    // 128 x 128 x 128 product per 128 rows, one thread per vector afterwards)
    if (p.rotate && p.in_dtype != TQ_DTYPE_F32 && p.use_tcgen05) return launch_paged_tc<KB, VB, QJL>(p, st);
    const int64_t n_groups = (p.n_items + kFastItemsPerCta - 1) / kFastItemsPerCta;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return TQ_ERR_LAUNCH;
    static int sm_count[64] = {0};
    if (dev >= 0 && dev < 64 && sm_count[dev]) sms = sm_count[dev];
    else {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return TQ_ERR_LAUNCH;
        if (dev >= 0 && dev < 64) sm_count[dev] = sms;
    }
    const int64_t resident = static_cast<int64_t>(sms) * TQ_CMP_MINBLOCKS;
    const unsigned grid = static_cast<unsigned>(n_groups < resident ? n_groups : resident);
    constexpr int kSmem = 2 * kTableBytes + kFastWarps * kStagePerWarp;
    static bool configured[64] = {false};
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        if (cudaFuncSetAttribute(compress_paged_fast_kernel<KB, VB, QJL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSmem) != cudaSuccess)
            return TQ_ERR_LAUNCH;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    compress_paged_fast_kernel<KB, VB, QJL><<<grid, kFastWarps * 32, kSmem, st>>>(p, n_groups);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

}  // namespace
}  // namespace tq
