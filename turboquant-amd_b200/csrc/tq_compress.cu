// KV compression for sm_100a: fast WHT, norm, Lloyd-Max bucketize, QJL signs, bit-packing.
//
// One warp compresses one 128-value vector; lane l holds dims 4l..4l+3.  The
// 128-point Walsh-Hadamard transform is two in-register butterfly stages and
// five warp-shuffle stages.  Everything after the rotation follows
// polarquant_compress of the reference (turboquant/core/quantizer.py:141-173)
// operation by operation in fp32:
//   n = sqrt(sum r^2);  u = r / (n + 1e-8);  idx = #{j : b_j < u};
//   e = (u - c[idx]) * n;  rn = sqrt(sum e^2);  sign = (e >= 0).
// The packed fields are then written either into the paged cache (layout of
// turboquant/kernels/paged_layout.py) or into the contiguous arrays of
// compress_k / compress_v (turboquant/kernels/packed_compress.py:157-240).
#include "tq_common.cuh"

namespace tq {
namespace {

constexpr int kWarpsPerCta = 4;

// ---- 128-point WHT across a warp (unnormalised) -------------------------------------
__device__ __forceinline__ void fwht128(float (&x)[4], int lane) {
    float a = x[0] + x[1], b = x[0] - x[1], c = x[2] + x[3], d = x[2] - x[3];
    x[0] = a + c; x[1] = b + d; x[2] = a - c; x[3] = b - d;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const float sgn = (lane & m) ? -1.f : 1.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, x[e], m);
            x[e] = fmaf(sgn, x[e], other);
        }
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int BITS>
struct Boundaries {
    float b[(1 << BITS) - 1];
    __device__ __forceinline__ void load(const float* __restrict__ g) {
#pragma unroll
        for (int i = 0; i < (1 << BITS) - 1; ++i) b[i] = __ldg(g + i);
    }
    // searchsorted(right=False): number of boundaries strictly below u; ties go down.
    __device__ __forceinline__ int bucket(float u) const {
        int idx = 0;
#pragma unroll
        for (int i = 0; i < (1 << BITS) - 1; ++i) idx += (u > b[i]) ? 1 : 0;
        return idx;
    }
};

struct Quantized {
    int idx[4];
    uint32_t sign4;   // bit e = 1 when the residual of element e is >= 0
    float norm, rnorm;
    float u[4];       // normalised rotated coordinates (kept for the unpacked output mode)
};

// x: 4 raw values of this lane.  csm: centroids in shared memory (only read when QJL).
template <int BITS, bool QJL>
__device__ __forceinline__ void quantize_vec(float (&x)[4], bool rotate, int lane, const Boundaries<BITS>& bd,
                                             const float* csm, Quantized& q) {
    if (rotate) {
        fwht128(x, lane);
#pragma unroll
        for (int e = 0; e < 4; ++e) x[e] *= kWhtScale;
    }
    float ss = x[0] * x[0];
    ss = fmaf(x[1], x[1], ss);
    ss = fmaf(x[2], x[2], ss);
    ss = fmaf(x[3], x[3], ss);
    ss = warp_sum(ss);
    const float n = sqrtf(ss);
    const float den = n + 1e-8f;
    float rs = 0.f;
    uint32_t sb = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float u = __fdiv_rn(x[e], den);
        const int i = bd.bucket(u);
        q.idx[e] = i;
        q.u[e] = u;
        if constexpr (QJL) {
            const float r = (u - csm[i]) * n;
            rs = fmaf(r, r, rs);
            sb |= (r >= 0.f ? 1u : 0u) << e;   // -0.0 and +0.0 both count as +
        }
    }
    q.sign4 = sb;
    q.norm = n;
    if constexpr (QJL) q.rnorm = sqrtf(warp_sum(rs));
    else q.rnorm = 0.f;
}

__device__ __forceinline__ uint32_t nibbles4(const int (&i)[4]) {
    return static_cast<uint32_t>(i[0]) | (static_cast<uint32_t>(i[1]) << 4) | (static_cast<uint32_t>(i[2]) << 8) |
           (static_cast<uint32_t>(i[3]) << 12);
}

// Bit b of each of the 4 indices, placed at the top bit of nibbles 0..3.
__device__ __forceinline__ uint32_t hole_bits(const int (&i)[4], int b) {
    uint32_t r = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) r |= ((static_cast<uint32_t>(i[e]) >> b) & 1u) << (4 * e + 3);
    return r;
}

// ---- paged stores -----------------------------------------------------------------------
// K sub-record words of this lane's dim quarter (lane = 8 * quarter + c).
template <int BITS, bool QJL>
__device__ __forceinline__ void store_k_paged(uint8_t* page, int t, int lane, const Quantized& q) {
    constexpr int NW = BITS + (QJL ? 1 : 0);
    constexpr int RK = 16 * NW;
    const int quarter = lane >> 3, c = lane & 7;
    const uint32_t gmask = 0xffu << (8 * quarter);
    uint32_t w[NW];
    const uint32_t f = nibbles4(q.idx);
#pragma unroll
    for (int j = 0; j < BITS; ++j) {
        uint32_t v = 0;
        if constexpr (BITS == 4) {
            if (j == (c >> 1)) v = f << (16 * (c & 1));
        } else if constexpr (BITS == 3) {
            if (c < 6) {
                if (j == (c >> 1)) v = f << (16 * (c & 1));
            } else {
                v = hole_bits(q.idx, j) << (16 * (c - 6));
            }
        } else {
            if (j == (c >> 2)) v = (f << (2 * ((c >> 1) & 1))) << (16 * (c & 1));
        }
        w[j] = __reduce_or_sync(gmask, v);
    }
    if constexpr (QJL) {
        w[BITS] = __reduce_or_sync(gmask, q.sign4 << (4 * c));   // bit l = sign of dim 32 * quarter + l
    }
    if (c == 0) {
        uint8_t* dst = page + t * RK + quarter * (RK / 4);
        if constexpr (NW == 4) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
        } else if constexpr (NW == 2) {
            *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
        } else {
#pragma unroll
            for (int j = 0; j < NW; ++j) reinterpret_cast<uint32_t*>(dst)[j] = w[j];
        }
    }
    if (lane == 0) {
        reinterpret_cast<__half*>(page + 16 * RK)[norm_slot(t)] = __float2half_rn(q.norm);
        if constexpr (QJL) reinterpret_cast<__half*>(page + 16 * RK + 32)[norm_slot(t)] = __float2half_rn(q.rnorm);
    }
}

// V 16-bit fields of this lane's dim group (lane = 4 * g + u).
template <int BITS>
__device__ __forceinline__ void store_v_paged(uint8_t* vpart, int t, int lane, const Quantized& q) {
    const int g = lane >> 2, u = lane & 3;
    const uint32_t gmask = 0xfu << (4 * g);
    const uint32_t f = nibbles4(q.idx);
    uint32_t mine = 0;
#pragma unroll
    for (int j = 0; j < BITS; ++j) {
        uint32_t v = 0;
        if constexpr (BITS == 4) {
            if (j == u) v = f;
        } else if constexpr (BITS == 3) {
            if (u < 3) {
                if (j == u) v = f;
            } else {
                v = hole_bits(q.idx, j);
            }
        } else {
            if (j == (u >> 1)) v = f << (2 * (u & 1));
        }
        const uint32_t r = __reduce_or_sync(gmask, v);
        if (j == u) mine = r;
    }
    if (u < BITS) {
        const int pair = t >> 1;
        uint8_t* dst = vpart + ((u * 8 + pair) * 8 + g) * 4 + (t & 1) * 2;
        *reinterpret_cast<uint16_t*>(dst) = static_cast<uint16_t>(mine);
    }
    if (lane == 0) reinterpret_cast<__half*>(vpart + 256 * BITS)[norm_slot(t)] = __float2half_rn(q.norm);
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
};

template <int KB, int VB, bool QJL>
__global__ void __launch_bounds__(kWarpsPerCta * 32) compress_paged_kernel(const PagedParams p) {
    constexpr int PAGE = page_bytes(KB, VB, QJL ? 1 : 0);
    constexpr int KPART = k_part_bytes(KB, QJL ? 1 : 0);
    __shared__ float csm[1 << KB];
    if (threadIdx.x < (1 << KB)) csm[threadIdx.x] = p.kc[threadIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    if (item >= p.n_items) return;
    const int64_t tok = item / p.Hkv;
    const int head = static_cast<int>(item % p.Hkv);
    int64_t slot = p.slot_mapping[tok];
    if (slot < 0) slot = 0;   // the reference clamps padding slots to 0
    if (slot >= p.num_slots) {
        if (lane == 0 && p.status) atomicOr(p.status, TQ_STATUS_BAD_SLOT);
        return;
    }
    const int64_t blk = slot / p.block_size;
    const int off = static_cast<int>(slot % p.block_size);
    const int spb = p.block_size / kPageTokens;
    uint8_t* page = p.cache + ((blk * p.Hkv + head) * spb + off / kPageTokens) * PAGE;
    const int t = off % kPageTokens;

    Boundaries<KB> kbd;
    kbd.load(p.kb);
    float x[4];
    Quantized q;
    load4(p.key, tok * p.ks_t + head * p.ks_h + 4 * lane, p.in_dtype, x);
    quantize_vec<KB, QJL>(x, p.rotate != 0, lane, kbd, csm, q);
    store_k_paged<KB, QJL>(page, t, lane, q);

    Boundaries<VB> vbd;
    vbd.load(p.vb);
    load4(p.value, tok * p.vs_t + head * p.vs_h + 4 * lane, p.in_dtype, x);
    quantize_vec<VB, false>(x, p.rotate != 0, lane, vbd, nullptr, q);
    store_v_paged<VB>(page + KPART, t, lane, q);
}

// ---- contiguous outputs ---------------------------------------------------------------------
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

template <int BITS>
__device__ __forceinline__ void store_idx_contig(uint8_t* row, int lane, const int (&i)[4]) {
    if constexpr (BITS == 2) {
        row[lane] = static_cast<uint8_t>(i[0] | (i[1] << 2) | (i[2] << 4) | (i[3] << 6));
    } else if constexpr (BITS == 4) {
        reinterpret_cast<uint16_t*>(row)[lane] = static_cast<uint16_t>(nibbles4(i));
    } else {
        // 12 bits per lane; four lanes make 48 bits = 6 bytes of the little-endian stream.
        const uint32_t mine = i[0] | (i[1] << 3) | (i[2] << 6) | (i[3] << 9);
        const int base = lane & ~3;
        const uint32_t a = __shfl_sync(0xffffffffu, mine, base), b = __shfl_sync(0xffffffffu, mine, base + 1);
        const uint32_t c = __shfl_sync(0xffffffffu, mine, base + 2), d = __shfl_sync(0xffffffffu, mine, base + 3);
        const uint64_t v = static_cast<uint64_t>(a) | (static_cast<uint64_t>(b) << 12) | (static_cast<uint64_t>(c) << 24) |
                           (static_cast<uint64_t>(d) << 36);
        const int k = lane & 3;
        if (k < 3) reinterpret_cast<uint16_t*>(row + 6 * (lane >> 2))[k] = static_cast<uint16_t>(v >> (16 * k));
    }
}

template <int BITS, OutMode MODE>
__global__ void __launch_bounds__(kWarpsPerCta * 32) compress_contig_kernel(const ContigParams p) {
    constexpr bool QJL = MODE != OutMode::kPackedV;
    __shared__ float csm[1 << BITS];
    if (threadIdx.x < (1 << BITS)) csm[threadIdx.x] = p.c ? p.c[threadIdx.x] : 0.f;
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    if (row >= p.n) return;
    Boundaries<BITS> bd;
    bd.load(p.b);
    float x[4];
    Quantized q;
    load4(p.x, row * kHeadDim + 4 * lane, p.in_dtype, x);
    if constexpr (MODE == OutMode::kUnpacked) {
        if (p.signs) quantize_vec<BITS, true>(x, p.rotate != 0, lane, bd, csm, q);
        else quantize_vec<BITS, false>(x, p.rotate != 0, lane, bd, csm, q);
        const int64_t o = row * kHeadDim + 4 * lane;
        float m[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            p.indices[o + e] = q.idx[e];
            m[e] = csm[q.idx[e]] * q.norm;
        }
        *reinterpret_cast<float4*>(p.mse + o) = make_float4(m[0], m[1], m[2], m[3]);
        if (p.signs) {
            float s[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) s[e] = ((q.sign4 >> e) & 1u) ? 1.f : -1.f;
            *reinterpret_cast<float4*>(p.signs + o) = make_float4(s[0], s[1], s[2], s[3]);
        }
        if (lane == 0) {
            p.norms[row] = q.norm;
            if (p.rnorm) p.rnorm[row] = q.rnorm;
        }
    } else {
        quantize_vec<BITS, QJL>(x, p.rotate != 0, lane, bd, csm, q);
        store_idx_contig<BITS>(p.idx_out + row * (16 * BITS), lane, q.idx);
        if constexpr (QJL) {
            uint8_t* srow = p.sign_out + row * 16;
            if (p.permute) {
                // stride-4 order: output bit 32 c + i <- dim c + 4 i, i.e. word c collects element c of every lane
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) w[e] = __ballot_sync(0xffffffffu, (q.sign4 >> e) & 1u);
                if (lane == 0) *reinterpret_cast<uint4*>(srow) = make_uint4(w[0], w[1], w[2], w[3]);
            } else {
                // sequential: byte j bit b <- dim 8 j + b; two lanes share a byte
                const uint32_t other = __shfl_xor_sync(0xffffffffu, q.sign4, 1);
                if (!(lane & 1)) srow[lane >> 1] = static_cast<uint8_t>(q.sign4 | (other << 4));
            }
            if (lane == 0) p.rnorm_h[row] = __float2half_rn(q.rnorm);
        }
        if (lane == 0) p.norm_h[row] = __float2half_rn(q.norm);
    }
}

template <int KB, int VB>
int launch_paged(const PagedParams& p, bool qjl, cudaStream_t st) {
    const unsigned grid = static_cast<unsigned>((p.n_items + kWarpsPerCta - 1) / kWarpsPerCta);
    if (qjl) compress_paged_kernel<KB, VB, true><<<grid, kWarpsPerCta * 32, 0, st>>>(p);
    else compress_paged_kernel<KB, VB, false><<<grid, kWarpsPerCta * 32, 0, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
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
    const unsigned grid = static_cast<unsigned>((p.n + kWarpsPerCta - 1) / kWarpsPerCta);
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
    const int align_elems = 4;  // each lane loads 4 consecutive elements with one vector load
    if (k_stride_token % align_elems || k_stride_head % align_elems || v_stride_token % align_elems ||
        v_stride_head % align_elems)
        return TQ_ERR_ARG;
    const uintptr_t amask = static_cast<uintptr_t>(4 * elem_bytes(in_dtype) - 1);
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
    p.rotate = prerotated ? 0 : 1;
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
