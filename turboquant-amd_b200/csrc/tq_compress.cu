// KV compression for sm_100a: fast WHT, norm, Lloyd-Max bucketize, QJL signs, bit-packing.
//
// Four lanes compress one 128-value vector: lane j of a group holds the 32 dims 32 j .. 32 j + 31
// in registers, a warp works on 8 vectors at a time (first the keys of 8 (token, head) items, then
// their values).  The 128-point Walsh-Hadamard transform is five butterfly stages inside the lane
// and two warp-shuffle stages across the four lanes, so only 2 of 7 stages pay for a shuffle, and
// every per-vector scalar (norm, square root, reciprocal) is amortised over 32 elements per lane.
// A lane's 32 dims are exactly one quarter of a K record of the paged cache, so the packed words
// are assembled in registers and written with one 16-byte store; no cross-lane reduction is needed.
//
// Everything after the rotation follows polarquant_compress of the reference
// (turboquant/core/quantizer.py:141-173) operation by operation in fp32:
//   n = sqrt(sum r^2);  u = r / (n + 1e-8);  idx = #{j : b_j < u};
//   e = (u - c[idx]) * n;  rn = sqrt(sum e^2);  sign = (e >= 0).
// The division is done as a correctly rounded reciprocal followed by one Newton-style correction
// of each quotient (q0 = r * inv; q = q0 + (r - q0 * den) * inv), which returns the IEEE quotient.
// Outputs go either into the paged cache (layout of turboquant/kernels/paged_layout.py) or into
// the contiguous arrays of compress_k / compress_v (turboquant/kernels/packed_compress.py:157-240).
#include "tq_common.cuh"

namespace tq {
namespace {

constexpr int kWarpsPerCta = 4;
constexpr int kItemsPerWarp = 8;
constexpr int kItemsPerCta = kWarpsPerCta * kItemsPerWarp;

// ---- loads: 32 consecutive elements of one row as fp32 ---------------------------------------
__device__ __forceinline__ void load32(const void* base, int64_t elem_off, int dtype, float (&x)[32]) {
    if (dtype == TQ_DTYPE_F32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem_off);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 v = __ldg(p + i);
            x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
        }
    } else {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + elem_off);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 v = __ldg(p + i);
            const uint32_t r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (dtype == TQ_DTYPE_F16) {
                    const float2 t = unpack_half2(r[k]);
                    x[8 * i + 2 * k] = t.x;
                    x[8 * i + 2 * k + 1] = t.y;
                } else {
                    x[8 * i + 2 * k] = __uint_as_float(r[k] << 16);
                    x[8 * i + 2 * k + 1] = __uint_as_float(r[k] & 0xffff0000u);
                }
            }
        }
    }
}

__device__ __forceinline__ float group_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}

// ---- bucketize: idx = number of boundaries strictly below u (searchsorted, right=False) -----------
// Branch-free binary search over boundaries held in registers; every index is a compile-time constant.
template <int BITS>
struct Boundaries {
    float b[(1 << BITS) - 1];
    __device__ __forceinline__ void load(const float* __restrict__ g) {
#pragma unroll
        for (int i = 0; i < (1 << BITS) - 1; ++i) b[i] = __ldg(g + i);
    }
    __device__ __forceinline__ int bucket(float u) const {
        if constexpr (BITS == 2) {
            const bool p1 = u > b[1];
            const bool p0 = u > (p1 ? b[2] : b[0]);
            return (p1 ? 2 : 0) + (p0 ? 1 : 0);
        } else if constexpr (BITS == 3) {
            const bool p2 = u > b[3];
            const bool p1 = u > (p2 ? b[5] : b[1]);
            const float hi = p2 ? b[6] : b[2], lo = p2 ? b[4] : b[0];
            const bool p0 = u > (p1 ? hi : lo);
            return (p2 ? 4 : 0) + (p1 ? 2 : 0) + (p0 ? 1 : 0);
        } else {
            const bool p3 = u > b[7];
            const bool p2 = u > (p3 ? b[11] : b[3]);
            const float h1 = p3 ? b[13] : b[5], l1 = p3 ? b[9] : b[1];
            const bool p1 = u > (p2 ? h1 : l1);
            const float c3 = p3 ? b[14] : b[6], c2 = p3 ? b[12] : b[4], c1 = p3 ? b[10] : b[2], c0 = p3 ? b[8] : b[0];
            const float hh = p2 ? c3 : c1, ll = p2 ? c2 : c0;
            const bool p0 = u > (p1 ? hh : ll);
            return (p3 ? 8 : 0) + (p2 ? 4 : 0) + (p1 ? 2 : 0) + (p0 ? 1 : 0);
        }
    }
};

// Result of compressing one quarter (32 dims) of a vector; norm and rnorm are whole-vector values.
struct Quarter {
    uint32_t idx[32];
    uint32_t signs;   // bit l = 1 when the residual of local dim l is >= 0
    float norm, rnorm;
};

// x: this lane's 32 values.  csm: centroids in shared memory (read only when QJL).
template <int BITS, bool QJL>
__device__ __forceinline__ void quantize_quarter(float (&x)[32], bool rotate, int lane, const Boundaries<BITS>& bd,
                                                 const float* csm, Quarter& q) {
    if (rotate) {
        fwht128(x, lane);
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] *= kWhtScale;
    }
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        s0 = fmaf(x[i], x[i], s0);
        s1 = fmaf(x[i + 1], x[i + 1], s1);
        s2 = fmaf(x[i + 2], x[i + 2], s2);
        s3 = fmaf(x[i + 3], x[i + 3], s3);
    }
    const float n = sqrtf(group_sum((s0 + s1) + (s2 + s3)));
    const float den = n + 1e-8f;
    const float inv = __frcp_rn(den);
    float r0 = 0.f, r1 = 0.f;
    uint32_t sb = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const float q0 = x[i] * inv;
        const float u = fmaf(fmaf(-q0, den, x[i]), inv, q0);   // = x / den, correctly rounded
        const int k = bd.bucket(u);
        q.idx[i] = static_cast<uint32_t>(k);
        if constexpr (QJL) {
            const float r = (u - csm[k]) * n;
            if (i & 1) r1 = fmaf(r, r, r1);
            else r0 = fmaf(r, r, r0);
            sb |= (r >= 0.f ? 1u : 0u) << i;   // -0.0 and +0.0 both count as +
        }
    }
    q.signs = sb;
    q.norm = n;
    q.rnorm = QJL ? sqrtf(group_sum(r0 + r1)) : 0.f;
}

// ---- paged stores (bit positions: turboquant/kernels/paged_layout.py) ------------------------------
// K: a lane's 32 dims are one quarter sub-record: BITS index words (+ the sign word).
template <int BITS>
__device__ __forceinline__ void pack_k_quarter(const uint32_t (&idx)[32], uint32_t (&w)[BITS]) {
#pragma unroll
    for (int j = 0; j < BITS; ++j) w[j] = 0;
#pragma unroll
    for (int l = 0; l < 32; ++l) {
        const int c = l >> 2, e = l & 3;
        if constexpr (BITS == 4) {
            w[c >> 1] |= idx[l] << ((c & 1) * 16 + 4 * e);
        } else if constexpr (BITS == 3) {
            if (c < 6) {
                w[c >> 1] |= idx[l] << ((c & 1) * 16 + 4 * e);
            } else {
#pragma unroll
                for (int b = 0; b < 3; ++b) w[b] |= ((idx[l] >> b) & 1u) << ((c - 6) * 16 + 4 * e + 3);
            }
        } else {
            w[c >> 2] |= idx[l] << ((c & 1) * 16 + 4 * e + ((c >> 1) & 1) * 2);
        }
    }
}

template <int BITS, bool QJL>
__device__ __forceinline__ void store_k_paged(uint8_t* page, int t, int quarter, const Quarter& q) {
    constexpr int NW = BITS + (QJL ? 1 : 0);
    constexpr int RK = 16 * NW;
    uint32_t w[BITS];
    pack_k_quarter<BITS>(q.idx, w);
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

// V: a lane's 32 dims are two dim groups g = 2 * quarter + {0, 1}; each gets BITS 16-bit fields.
template <int BITS>
__device__ __forceinline__ void store_v_paged(uint8_t* vpart, int t, int quarter, const Quarter& q) {
    const int pair = t >> 1, half = t & 1;
#pragma unroll
    for (int gg = 0; gg < 2; ++gg) {
        uint32_t f[BITS];
#pragma unroll
        for (int j = 0; j < BITS; ++j) f[j] = 0;
#pragma unroll
        for (int m = 0; m < 16; ++m) {
            const uint32_t i = q.idx[16 * gg + m];
            const int u = m >> 2, e = m & 3;
            if constexpr (BITS == 4) {
                f[u] |= i << (4 * e);
            } else if constexpr (BITS == 3) {
                if (u < 3) {
                    f[u] |= i << (4 * e);
                } else {
#pragma unroll
                    for (int b = 0; b < 3; ++b) f[b] |= ((i >> b) & 1u) << (4 * e + 3);
                }
            } else {
                f[u >> 1] |= i << (4 * e + (u & 1) * 2);
            }
        }
        const int g = 2 * quarter + gg;
#pragma unroll
        for (int j = 0; j < BITS; ++j)
            *reinterpret_cast<uint16_t*>(vpart + ((j * 8 + pair) * 8 + g) * 4 + half * 2) = static_cast<uint16_t>(f[j]);
    }
    if (quarter == 0) reinterpret_cast<__half*>(vpart + 256 * BITS)[norm_slot(t)] = __float2half_rn(q.norm);
}

struct PagedParams {
    const void* key;
    const void* value;
    uint8_t* cache;
    const int64_t* slot_mapping;
    const float* kc;
    const float* kb;
    const float* vb;
    int32_t* status;
    int64_t ks_t, ks_h, vs_t, vs_h;
    int64_t num_slots;
    int64_t n_items;   // n_tokens * n_kv_heads
    int Hkv, block_size, in_dtype, rotate;
    int use_tcgen05;       // TQ_COMPRESS_TCGEN05 was given
};

// Where one (token, head) item goes in the paged cache; live = false when the item is past the end or its
// slot is out of range (then nothing is stored; a bad slot also raises the status bit).
struct ItemPlace {
    int64_t tok;
    int head, t;
    uint8_t* page;
    bool live;
};

// Which token and KV head an item is; live = false past the end.
struct ItemId {
    int64_t tok;
    int head;
    bool live;
};

__device__ __forceinline__ ItemId identify_item(const PagedParams& p, int64_t item) {
    ItemId id;
    id.tok = 0; id.head = 0;
    id.live = item < p.n_items;
    if (id.live) {
        if (p.n_items <= 0x7fffffff) {   // uniform over the grid: 32-bit division is several times cheaper
            const uint32_t tk = static_cast<uint32_t>(item) / static_cast<uint32_t>(p.Hkv);
            id.tok = tk;
            id.head = static_cast<int>(static_cast<uint32_t>(item) - tk * static_cast<uint32_t>(p.Hkv));
        } else {
            id.tok = item / p.Hkv;
            id.head = static_cast<int>(item - id.tok * p.Hkv);
        }
    }
    return id;
}

template <int PAGE>
__device__ __forceinline__ ItemPlace place_item(const PagedParams& p, const ItemId& id, int quarter) {
    ItemPlace w;
    w.tok = id.tok; w.head = id.head; w.t = 0; w.page = nullptr;
    w.live = id.live;
    if (w.live) {
        int64_t slot = p.slot_mapping[w.tok];
        if (slot < 0) slot = 0;   // the reference clamps padding slots to 0
        if (slot >= p.num_slots) {
            if (quarter == 0 && p.status) atomicOr(p.status, TQ_STATUS_BAD_SLOT);
            w.live = false;
        } else {
            int64_t blk;
            if (p.num_slots <= 0x7fffffff) blk = static_cast<uint32_t>(slot) / static_cast<uint32_t>(p.block_size);
            else blk = slot / p.block_size;
            const int off = static_cast<int>(slot - blk * p.block_size);
            const int spb = p.block_size / kPageTokens;
            w.page = p.cache + ((blk * p.Hkv + w.head) * spb + off / kPageTokens) * PAGE;
            w.t = off % kPageTokens;
        }
    }
    return w;
}

template <int PAGE>
__device__ __forceinline__ ItemPlace place_item(const PagedParams& p, int64_t item, int quarter) {
    return place_item<PAGE>(p, identify_item(p, item), quarter);
}

// Generic path for one group of 8 items per warp: binary-search bucketize over arbitrary sorted boundaries.
// Lanes of items past the end still take part in the shuffles (on zeros) and store nothing.
template <int KB, int VB, bool QJL>
__device__ __noinline__ void compress_items_generic(const PagedParams& p, int64_t item, int lane, const float* csm) {
    constexpr int PAGE = page_bytes(KB, VB, QJL ? 1 : 0);
    constexpr int KPART = k_part_bytes(KB, QJL ? 1 : 0);
    const int quarter = lane & 3;
    const ItemPlace w = place_item<PAGE>(p, item, quarter);
    float x[32];
    Quarter q;
    {
        Boundaries<KB> kbd;
        kbd.load(p.kb);
        if (w.live) load32(p.key, w.tok * p.ks_t + w.head * p.ks_h + 32 * quarter, p.in_dtype, x);
        else {
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] = 0.f;
        }
        quantize_quarter<KB, QJL>(x, p.rotate != 0, lane, kbd, csm, q);
        if (w.live) store_k_paged<KB, QJL>(w.page, w.t, quarter, q);
    }
    {
        Boundaries<VB> vbd;
        vbd.load(p.vb);
        if (w.live) load32(p.value, w.tok * p.vs_t + w.head * p.vs_h + 32 * quarter, p.in_dtype, x);
        else {
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] = 0.f;
        }
        quantize_quarter<VB, false>(x, p.rotate != 0, lane, vbd, nullptr, q);
        if (w.live) store_v_paged<VB>(w.page + KPART, w.t, quarter, q);
    }
}

}  // namespace
}  // namespace tq

#include "tq_compress_fast.cuh"
#include "tq_compress_tc.cuh"

namespace tq {
namespace {

// ---- contiguous outputs ---------------------------------------------------------------------------
enum class OutMode { kPackedK, kPackedV, kUnpacked };

struct ContigParams {
    const void* x;
    const float* c;
    const float* b;
    uint8_t* idx_out;
    uint8_t* sign_out;
    __half* rnorm_h;
    __half* norm_h;
    int64_t* indices;
    float* norms;
    float* mse;
    float* signs;
    float* rnorm;
    int64_t n;
    int in_dtype, rotate, permute;
};

// Reference byte layouts: 2-bit 4 per byte LSB first, 4-bit low nibble first, 3-bit little-endian stream.
// A lane's 32 dims are 8 / 12 / 16 consecutive bytes of the row.
template <int BITS>
__device__ __forceinline__ void store_idx_contig(uint8_t* row, int quarter, const uint32_t (&idx)[32]) {
    uint32_t w[BITS];
#pragma unroll
    for (int j = 0; j < BITS; ++j) w[j] = 0;
#pragma unroll
    for (int l = 0; l < 32; ++l) {
        const int bit = l * BITS;
        w[bit >> 5] |= idx[l] << (bit & 31);
        if ((bit & 31) + BITS > 32) w[(bit >> 5) + 1] |= idx[l] >> (32 - (bit & 31));
    }
    uint32_t* dst = reinterpret_cast<uint32_t*>(row + quarter * (4 * BITS));
    if constexpr (BITS == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    else if constexpr (BITS == 2) *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
    else {
#pragma unroll
        for (int j = 0; j < BITS; ++j) dst[j] = w[j];
    }
}

// Sign bits and norms of one packed row (this lane's quarter).  signs: bit l = 1 when the residual of local dim l is >= 0.
template <bool QJL>
__device__ __forceinline__ void store_contig_tail(const ContigParams& p, int64_t row, int quarter, uint32_t signs, float norm,
                                                  float rnorm) {
    if constexpr (QJL) {
        uint8_t* srow = p.sign_out + row * 16;
        if (p.permute) {
            // stride-4 order: output bit 32 c + i <- dim c + 4 i.  This lane's dim 32 q + l has
            // c = l & 3 and i = 8 q + (l >> 2): it fills byte q of each of the four 32-bit words.
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v = 0;
#pragma unroll
                for (int k = 0; k < 8; ++k) v |= ((signs >> (4 * k + c)) & 1u) << k;
                srow[4 * c + quarter] = static_cast<uint8_t>(v);
            }
        } else {
            reinterpret_cast<uint32_t*>(srow)[quarter] = signs;   // byte j bit b <- dim 8 j + b
        }
        if (quarter == 0) p.rnorm_h[row] = __float2half_rn(rnorm);
    }
    if (quarter == 0) p.norm_h[row] = __float2half_rn(norm);
}

// One group of 8 rows per warp on the generic quantizer (binary-search bucketize over arbitrary sorted boundaries).
// Lanes of rows past the end still take part in the shuffles (on zeros) and store nothing.
template <int BITS, OutMode MODE>
__device__ __forceinline__ void compress_contig_rows(const ContigParams& p, int64_t row, int lane, const float* csm) {
    constexpr bool QJL = MODE != OutMode::kPackedV;
    const int quarter = lane & 3;
    const bool live = row < p.n;
    Boundaries<BITS> bd;
    bd.load(p.b);
    float x[32];
    Quarter q;
    if (live) load32(p.x, row * kHeadDim + 32 * quarter, p.in_dtype, x);
    else {
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = 0.f;
    }
    if constexpr (MODE == OutMode::kUnpacked) {
        const bool with_signs = p.signs != nullptr;   // uniform over the grid
        if (with_signs) quantize_quarter<BITS, true>(x, p.rotate != 0, lane, bd, csm, q);
        else quantize_quarter<BITS, false>(x, p.rotate != 0, lane, bd, csm, q);
        if (!live) return;
        const int64_t o = row * kHeadDim + 32 * quarter;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            longlong2 v;
            v.x = q.idx[i];
            v.y = q.idx[i + 1];
            *reinterpret_cast<longlong2*>(p.indices + o + i) = v;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(p.mse + o + i) = make_float4(csm[q.idx[i]] * q.norm, csm[q.idx[i + 1]] * q.norm,
                                                                   csm[q.idx[i + 2]] * q.norm, csm[q.idx[i + 3]] * q.norm);
        if (with_signs) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                float s[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) s[e] = ((q.signs >> (i + e)) & 1u) ? 1.f : -1.f;
                *reinterpret_cast<float4*>(p.signs + o + i) = make_float4(s[0], s[1], s[2], s[3]);
            }
        }
        if (quarter == 0) {
            p.norms[row] = q.norm;
            if (p.rnorm) p.rnorm[row] = q.rnorm;
        }
    } else {
        quantize_quarter<BITS, QJL>(x, p.rotate != 0, lane, bd, csm, q);
        if (!live) return;
        store_idx_contig<BITS>(p.idx_out + row * (16 * BITS), quarter, q.idx);
        store_contig_tail<QJL>(p, row, quarter, q.signs, q.norm, q.rnorm);
    }
}

template <int BITS, OutMode MODE>
__global__ void __launch_bounds__(kWarpsPerCta * 32) compress_contig_kernel(const ContigParams p) {
    __shared__ float csm[1 << BITS];
    if (threadIdx.x < (1 << BITS)) csm[threadIdx.x] = p.c ? p.c[threadIdx.x] : 0.f;
    __syncthreads();
    const int lane = threadIdx.x & 31;
    compress_contig_rows<BITS, MODE>(
        p, (static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5)) * kItemsPerWarp + (lane >> 2), lane, csm);
}

// ---- packed contiguous outputs on the table-driven quantizer ------------------------------------------------------
// Persistent CTAs of 16 warps, one per SM, as the paged kernel: the table is built once per CTA, which then strides over
// groups of 128 rows, 8 per warp.  fp16 / bf16 rows that still need the rotation are staged through two buffers per
// warp, two groups ahead, and rotated on the tensor cores; fp32 and already rotated rows take plain loads.
template <int BITS, bool QJL>
__device__ __forceinline__ void store_contig_fast(const ContigParams& p, int64_t row, int quarter, const Packed& q) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(p.idx_out + row * (16 * BITS) + quarter * (4 * BITS));
    if constexpr (BITS == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(q.word[0], q.word[1], q.word[2], q.word[3]);
    else if constexpr (BITS == 2) *reinterpret_cast<uint2*>(dst) = make_uint2(q.word[0], q.word[1]);
    else {
#pragma unroll
        for (int j = 0; j < BITS; ++j) dst[j] = q.word[j];
    }
    store_contig_tail<QJL>(p, row, quarter, q.signs, q.norm, q.rnorm);
}

template <int BITS, bool QJL>
__global__ void __launch_bounds__(kFastWarps * 32, 1) compress_contig_fast_kernel(const ContigParams p, int64_t n_groups) {
    extern __shared__ __align__(128) unsigned char tables[];
    __shared__ float csm[1 << BITS];
    __shared__ int bad;
    if (threadIdx.x == 0) bad = 0;
    if (threadIdx.x < (1 << BITS)) csm[threadIdx.x] = p.c ? p.c[threadIdx.x] : 0.f;
    __syncthreads();
    build_table<BITS, QJL>(tables, p.b, p.c, &bad);
    __syncthreads();
    const int lane = threadIdx.x & 31, quarter = lane & 3, warp = threadIdx.x >> 5;
    const int64_t row0 = warp * kItemsPerWarp + (lane >> 2);   // + group * 128
    if (bad != 0) {   // two boundaries inside one cell: the generic quantizer
        const ContigParams pc = p;
        for (int64_t grp = blockIdx.x; grp < n_groups; grp += gridDim.x)
            compress_contig_rows<BITS, QJL ? OutMode::kPackedK : OutMode::kPackedV>(pc, grp * kFastItemsPerCta + row0, lane, csm);
        return;
    }
    constexpr uint32_t kBias = kMagicBits * static_cast<uint32_t>(kCellStride);   // modulo 2^32
    const uint32_t tab = smem_u32(tables) + (QJL ? (lane & 7) * 16 : (lane & 15) * 8) - kBias;
    Packed q;
    if (p.rotate && p.in_dtype != TQ_DTYPE_F32) {
        const bool bf16 = p.in_dtype == TQ_DTYPE_BF16;
        uint4* buf = reinterpret_cast<uint4*>(tables + kTableBytes + warp * kStagePerWarp);   // two buffers of 128 uint4
        const WhtFragments hf = make_wht_fragments(lane, bf16);
        int64_t grp = blockIdx.x;
        const int64_t step = gridDim.x;
        {
            const int64_t r0 = grp * kFastItemsPerCta + row0, r1 = (grp + step) * kFastItemsPerCta + row0;
            stage_row(buf, lane, p.x, r0 * kHeadDim + 32 * quarter, r0 < p.n);
            stage_row(buf + 128, lane, p.x, r1 * kHeadDim + 32 * quarter, grp + step < n_groups && r1 < p.n);
        }
        int cur = 0;
        for (; grp < n_groups; grp += step, cur ^= 1) {
            const int64_t row = grp * kFastItemsPerCta + row0;
            const int64_t nxt = (grp + 2 * step) * kFastItemsPerCta + row0;
            const bool nxt_live = grp + 2 * step < n_groups && nxt < p.n;
            uint4* b = buf + 128 * cur;
            wait_staged();
            compress_row_mma<BITS, QJL, false, true>(smem_u32(b + lane), row < p.n, lane, bf16, hf, tab, q, [&] {
                stage_row(b, lane, p.x, nxt * kHeadDim + 32 * quarter, nxt_live);
            });
            if (row < p.n) store_contig_fast<BITS, QJL>(p, row, quarter, q);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        const bool rotate = p.rotate != 0;
        const float scale = rotate ? kWhtScale : 1.f, inv_scale = rotate ? 11.313708498984761f : 1.f;
        for (int64_t grp = blockIdx.x; grp < n_groups; grp += gridDim.x) {
            const int64_t row = grp * kFastItemsPerCta + row0;
            f2 y[16];
            fetch_plain(p.x, row * kHeadDim + 32 * quarter, row < p.n, p.in_dtype, rotate, lane, y);
            quantize_fast<BITS, QJL, false, true>(y, scale, inv_scale, tab, q);
            if (row < p.n) store_contig_fast<BITS, QJL>(p, row, quarter, q);
        }
    }
}

template <int BITS, bool QJL>
int launch_contig_fast(const ContigParams& p, cudaStream_t st) {
    const int64_t n_groups = (p.n + kFastItemsPerCta - 1) / kFastItemsPerCta;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return TQ_ERR_LAUNCH;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return TQ_ERR_LAUNCH;
    const unsigned grid = static_cast<unsigned>(n_groups < sms ? n_groups : sms);
    constexpr int kSmem = kTableBytes + kFastWarps * kStagePerWarp;
    static bool configured[64] = {false};
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        if (cudaFuncSetAttribute(compress_contig_fast_kernel<BITS, QJL>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) !=
            cudaSuccess)
            return TQ_ERR_LAUNCH;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    compress_contig_fast_kernel<BITS, QJL><<<grid, kFastWarps * 32, kSmem, st>>>(p, n_groups);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

template <int KB, int VB>
int launch_paged(const PagedParams& p, bool qjl, cudaStream_t st) {
    return qjl ? launch_paged_fast<KB, VB, true>(p, st) : launch_paged_fast<KB, VB, false>(p, st);
}

template <int KB>
int launch_paged_v(const PagedParams& p, int vb, bool qjl, cudaStream_t st) {
    switch (vb) {
        case 2: return launch_paged<KB, 2>(p, qjl, st);
        case 3: return launch_paged<KB, 3>(p, qjl, st);
        case 4: return launch_paged<KB, 4>(p, qjl, st);
    }
    return TQ_ERR_UNSUPPORTED;
}

template <OutMode MODE>
int launch_contig(const ContigParams& p, int bits, cudaStream_t st) {
    if constexpr (MODE != OutMode::kUnpacked) {
        // large packed launches: the persistent table-driven kernel.  Measured on fp16 rows with the rotation: 16384
        // rows 5.9 us (binary-search kernel) against 6.8 us, 32768 rows about 11 us either way, 65536 rows 22 against
        // 15 us: below about two groups of 128 rows per SM the persistent kernel mostly builds its table.
        if (p.n > 2 * kSmallLaunchItems) {
            constexpr bool QJL = MODE == OutMode::kPackedK;
            switch (bits) {
                case 2: return launch_contig_fast<2, QJL>(p, st);
                case 3: return launch_contig_fast<3, QJL>(p, st);
                case 4: return launch_contig_fast<4, QJL>(p, st);
                default: return TQ_ERR_UNSUPPORTED;
            }
        }
    }
    const unsigned grid = static_cast<unsigned>((p.n + kItemsPerCta - 1) / kItemsPerCta);
    switch (bits) {
        case 2: compress_contig_kernel<2, MODE><<<grid, kWarpsPerCta * 32, 0, st>>>(p); break;
        case 3: compress_contig_kernel<3, MODE><<<grid, kWarpsPerCta * 32, 0, st>>>(p); break;
        case 4: compress_contig_kernel<4, MODE><<<grid, kWarpsPerCta * 32, 0, st>>>(p); break;
        default: return TQ_ERR_UNSUPPORTED;
    }
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

bool dtype_ok(int d) { return d == TQ_DTYPE_F16 || d == TQ_DTYPE_BF16 || d == TQ_DTYPE_F32; }
int elem_bytes(int d) { return d == TQ_DTYPE_F32 ? 4 : 2; }

}  // namespace
}  // namespace tq
using namespace tq;

extern "C" int tq_version(void) { return (0 << 16) | 1; }

extern "C" int tq_page_bytes(int k_bits, int v_bits, int use_qjl) {
    if (k_bits < 2 || k_bits > 4 || v_bits < 2 || v_bits > 4) return TQ_ERR_UNSUPPORTED;
    return page_bytes(k_bits, v_bits, use_qjl ? 1 : 0);
}

extern "C" int tq_compress_paged(const void* key, const void* value, int in_dtype, int64_t k_stride_token,
                                 int64_t k_stride_head, int64_t v_stride_token, int64_t v_stride_head, void* cache,
                                 int64_t num_blocks, int block_size, const int64_t* slot_mapping,
                                 const float* k_centroids, const float* k_boundaries, const float* v_centroids,
                                 const float* v_boundaries, int n_tokens, int n_kv_heads, int k_bits, int v_bits,
                                 int use_qjl, int prerotated, int32_t* status, tq_stream_t stream) {
    (void)v_centroids;  // V stores indices and a norm only; its centroids are not needed to compress
    if (n_tokens == 0) return TQ_OK;
    if (!key || !value || !cache || !slot_mapping || !k_centroids || !k_boundaries || !v_boundaries) return TQ_ERR_ARG;
    if (n_tokens < 0 || n_kv_heads <= 0 || num_blocks <= 0) return TQ_ERR_ARG;
    if (!dtype_ok(in_dtype)) return TQ_ERR_UNSUPPORTED;
    if (block_size <= 0 || block_size % kPageTokens) return TQ_ERR_UNSUPPORTED;
    if (k_bits < 2 || k_bits > 4 || v_bits < 2 || v_bits > 4) return TQ_ERR_UNSUPPORTED;
    const int align_elems = 16 / elem_bytes(in_dtype);  // lanes read rows with 16-byte vector loads
    if (k_stride_token % align_elems || k_stride_head % align_elems || v_stride_token % align_elems ||
        v_stride_head % align_elems)
        return TQ_ERR_ARG;
    const uintptr_t amask = 15;
    if ((reinterpret_cast<uintptr_t>(key) & amask) || (reinterpret_cast<uintptr_t>(value) & amask) ||
        (reinterpret_cast<uintptr_t>(cache) & 15))
        return TQ_ERR_ARG;
    PagedParams p;
    p.key = key;
    p.value = value;
    p.cache = static_cast<uint8_t*>(cache);
    p.slot_mapping = slot_mapping;
    p.kc = k_centroids;
    p.kb = k_boundaries;
    p.vb = v_boundaries;
    p.status = status;
    p.ks_t = k_stride_token;
    p.ks_h = k_stride_head;
    p.vs_t = v_stride_token;
    p.vs_h = v_stride_head;
    p.num_slots = num_blocks * block_size;
    p.n_items = static_cast<int64_t>(n_tokens) * n_kv_heads;
    p.Hkv = n_kv_heads;
    p.block_size = block_size;
    p.in_dtype = in_dtype;
    p.rotate = (prerotated & 1) ? 0 : 1;
    p.use_tcgen05 = (prerotated & TQ_COMPRESS_TCGEN05) ? 1 : 0;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (k_bits) {
        case 2: return launch_paged_v<2>(p, v_bits, use_qjl != 0, st);
        case 3: return launch_paged_v<3>(p, v_bits, use_qjl != 0, st);
        case 4: return launch_paged_v<4>(p, v_bits, use_qjl != 0, st);
    }
    return TQ_ERR_UNSUPPORTED;
}

extern "C" int tq_compress_k(const void* K, int in_dtype, int64_t n, const float* centroids, const float* boundaries,
                             int bits, int prerotated, int permute_signs, uint8_t* k_idx, uint8_t* k_signs,
                             void* k_rnorm, void* k_norm, tq_stream_t stream) {
    if (n == 0) return TQ_OK;
    if (!K || !centroids || !boundaries || !k_idx || !k_signs || !k_rnorm || !k_norm || n < 0) return TQ_ERR_ARG;
    if (!dtype_ok(in_dtype)) return TQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(K) | reinterpret_cast<uintptr_t>(k_signs)) & 15) return TQ_ERR_ARG;
    ContigParams p = {};
    p.x = K; p.c = centroids; p.b = boundaries; p.idx_out = k_idx; p.sign_out = k_signs;
    p.rnorm_h = static_cast<__half*>(k_rnorm); p.norm_h = static_cast<__half*>(k_norm);
    p.n = n; p.in_dtype = in_dtype; p.rotate = prerotated ? 0 : 1; p.permute = permute_signs;
    return launch_contig<OutMode::kPackedK>(p, bits, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int tq_compress_v(const void* V, int in_dtype, int64_t n, const float* boundaries, int bits, int prerotated,
                             uint8_t* v_idx, void* v_norm, tq_stream_t stream) {
    if (n == 0) return TQ_OK;
    if (!V || !boundaries || !v_idx || !v_norm || n < 0) return TQ_ERR_ARG;
    if (!dtype_ok(in_dtype)) return TQ_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(V) & 15) return TQ_ERR_ARG;
    ContigParams p = {};
    p.x = V; p.b = boundaries; p.idx_out = v_idx; p.norm_h = static_cast<__half*>(v_norm);
    p.n = n; p.in_dtype = in_dtype; p.rotate = prerotated ? 0 : 1;
    return launch_contig<OutMode::kPackedV>(p, bits, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int tq_polarquant_compress(const void* x, int in_dtype, int64_t n, const float* centroids,
                                      const float* boundaries, int bits, int use_qjl, int prerotated, int64_t* indices,
                                      float* norms, float* k_mse_rot, float* signs, float* rnorm, tq_stream_t stream) {
    if (n == 0) return TQ_OK;
    if (!x || !centroids || !boundaries || !indices || !norms || !k_mse_rot || n < 0) return TQ_ERR_ARG;
    if (use_qjl && (!signs || !rnorm)) return TQ_ERR_ARG;
    if (!dtype_ok(in_dtype)) return TQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(k_mse_rot) | reinterpret_cast<uintptr_t>(signs)) & 15)
        return TQ_ERR_ARG;
    ContigParams p = {};
    p.x = x; p.c = centroids; p.b = boundaries; p.indices = indices; p.norms = norms; p.mse = k_mse_rot;
    p.signs = use_qjl ? signs : nullptr; p.rnorm = use_qjl ? rnorm : nullptr;
    p.n = n; p.in_dtype = in_dtype; p.rotate = prerotated ? 0 : 1;
    return launch_contig<OutMode::kUnpacked>(p, bits, reinterpret_cast<cudaStream_t>(stream));
}
