// Paged decode attention on the 5th-generation tensor cores (tcgen05 + tensor memory) for 2- and 3-bit codebooks.
//
// Included by tq_decode.cu (DecodeParams, the split-K workspace format and the merge kernel are shared with the
// mma.sync kernel there).  One CTA works on a chunk of pages of one (sequence, KV head, group of <= 8 query heads),
// 128 tokens (8 pages) at a time:
//
//   producer warp   bulk async copies of the tile's 8 packed pages into a shared-memory ring (mbarrier complete_tx);
//   key warps 0-3   one thread per token: its 64-byte key record becomes rows of three e4m3 operand planes in
//                   tensor memory (centroid = hi + lo, two byte planes; the QJL sign plane is +-1.0).  A masked
//                   16-bit half of a packed word is four byte-table selectors, so one `prmt` against the 8-entry
//                   centroid table held in two registers yields four operand bytes (0.25 instructions per element
//                   and plane, against 1.5 for the half2 table look-ups of the mma.sync kernel);
//   MMA thread      S[128 tokens x 16] = K_planes (tensor memory) x q^T (shared memory, q = q1 + q2 in e4m3, rows
//                   0-7 and 8-15 of the B operand), `tcgen05.mma kind::f8f6f4`, fp32 accumulators in tensor memory;
//   key warps       read their token's row of S back (`tcgen05.ld`), fold norms, tile softmax (maximum over the
//                   tile through integer `redux.sync` + one shared-memory exchange), weights w = w1 + w2 in e4m3
//                   written as the B operand of the value product, per-thread denominators;
//   value warps 4-7 dequantise V the same way into two e4m3 planes in shared memory, laid out as the MN-major A
//                   operand (dims contiguous) in exactly the order the token-owning stores produce;
//   MMA thread      O_t[128 dims x 16] = V_planes^T x W  (both operands MN-major from shared memory);
//   value warps     thread = dim: O += alpha * O + beta * O_t in registers (fp32), so tensor memory never needs the
//                   running-maximum rescale.
//
// Weights are relative to the maximum of their own tile (including the token's value norm), so the e4m3 range is
// used fully in every tile however far the tile lies below the running maximum; the fp32 factors alpha / beta
// carry the difference.  Arithmetic restated from the reference as in tq_decode.cu
// (turboquant/kernels/packed_attention.py:150-196,273-284; turboquant/kernels/sparse_v.py:39-48,70-71).
//
// All mbarrier waits are bounded; a wait that gives up sets TQ_STATUS_TIMEOUT, every role leaves its loop and the
// CTA still frees its tensor memory.  Only this GPU's own memory is read; the bulk copies are the non-multicast form.
#pragma once

namespace tq {
namespace {

constexpr int kUmThreads = 320;         // warps 0-3 keys + softmax, 4-7 values + accumulate, 8 producer, 9 MMA
constexpr int kUmTilePages = 8;
constexpr int kUmTileTokens = kUmTilePages * kPageTokens;   // 128
constexpr int kUmStages = 2;            // tiles in flight in the page ring
constexpr int kUmTmemCols = 256;        // half of an SM's tensor memory: two CTAs per SM
// tensor-memory columns
constexpr int kColPlanes = 0;           // [2][96]: khi, klo, sign
constexpr int kColS = 192;              // [32]: 16 MSE + 16 QJL accumulators (single buffer, handed back by the key warps)
constexpr int kColO = 224;              // [2][16]
constexpr float kWScale = 256.f;        // weights are stored as w * 256 (e4m3 max is 448)

__host__ __device__ constexpr int um_page_stride(int page) { return page + ((112 - page % 128) + 128) % 128; }

// ---- shared memory map (bytes from the start of dynamic shared memory, 1024-aligned) ----------------------
struct UmSmem {
    static constexpr int kBars = 0;                 // 32 mbarriers
    static constexpr int kTmemSlot = 256;
    static constexpr int kTab = 272;                // 4 x 8 bytes: K hi, K lo, V hi, V lo tables (+ pad)
    static constexpr int kScal = 320;               // floats: mse_scale, qjl_scale, out_scale, m_final[8], l_final[8]
    static constexpr int kStat = 512;               // [4] x { m_tile[8], alpha[8], beta[8] floats, wmax[4][8] ints } = 4 x 224
    static constexpr int kLred = 512 + 4 * 224;     // [4 warps][8] floats
    static constexpr int kQ = 2048;                 // B operand of the MSE product, 2 KB
    static constexpr int kQP = 4096;                // B operand of the sign product, 2 KB
    static constexpr int kP = 6144;                 // [2] x 2 KB
    static constexpr int kV = 10240;                // [2] x 2 planes x 16 KB
    static constexpr int kRing = 10240 + 65536;     // [kUmStages] x 8 x page stride (two CTAs of ~104 KB fit one SM) (two CTAs of ~104 KB fit one SM)
};

enum UmBar { kFull = 0, kEmpty = 3, kKReady = 6, kSDone = 8, kSFree = 9, kPReady = 10, kVReady = 12, kPVDone = 14, kNumBars = 16 };

// ---- small wrappers -----------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // shared-memory matrix descriptor, no swizzle: start address, leading / stride byte offsets (all >> 4), version 1
    return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
// instruction descriptor of kind::f8f6f4: e4m3 x e4m3 -> f32, M x N, operand majors (0 = K-major, 1 = MN-major)
__host__ __device__ constexpr uint32_t umma_idesc(int M, int N, int a_mn, int b_mn) {
    return (1u << 4) | (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
           (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accum), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// two floats -> two e4m3 bytes (a in bits 8..15, b in bits 0..7), round to nearest, saturating
__device__ __forceinline__ uint32_t cvt_e4m3x2(float a, float b) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(byte & 0xffu)));
    return unpack_half2(h2).x;
}
__device__ __forceinline__ int redux_max(int v) {
    int r;
    asm volatile("redux.sync.max.s32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ float lg2(float x) {
    float r;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 lds_f128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_w(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts_u128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ float lds_half(uint32_t addr) {
    uint16_t h;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(addr));
    return __half2float(__ushort_as_half(h));
}

// Byte tables of one codebook: c[i] * S = hi[i] + lo[i] with both in e4m3.  Sixteen lanes (lane & 15 = candidate j) try
// S = 2^e (1 + j / 16), with 2^e the power of two that puts the largest centroid in [64, 128), and the candidate whose
// worst centroid is represented best wins (a codebook has few distinct magnitudes, so some scale puts all of them close
// to byte pairs); the winner writes the tables.  Every lane of the half-warp returns 1 / S.
template <int BITS>
__device__ __forceinline__ float build_byte_tables(const float* __restrict__ c, uint8_t* hi, uint8_t* lo, int lane) {
    float cv[1 << BITS], mx = 0.f;
#pragma unroll
    for (int i = 0; i < (1 << BITS); ++i) {
        cv[i] = __ldg(c + i);
        mx = fmaxf(mx, fabsf(cv[i]));
    }
    int e = 0;
    if (mx > 0.f && mx < __uint_as_float(0x7f800000u)) e = 133 - static_cast<int>((__float_as_uint(mx) >> 23) & 0xffu);   // 2^e * mx in [64, 128)
    e = max(-100, min(100, e));
    const int j = lane & 15;
    const float S = __uint_as_float(static_cast<uint32_t>(127 + e) << 23) * (1.f + static_cast<float>(j) * 0.0625f);
    uint32_t hb[1 << BITS], lb[1 << BITS];
    float err = 0.f;
#pragma unroll
    for (int i = 0; i < (1 << BITS); ++i) {
        const float v = cv[i] * S;
        hb[i] = cvt_e4m3x2(0.f, v) & 0xffu;
        const float h = e4m3_to_float(hb[i]);
        lb[i] = cvt_e4m3x2(0.f, v - h) & 0xffu;
        const float rep = h + e4m3_to_float(lb[i]);
        err = fmaxf(err, fabsf(v - rep) / fmaxf(fabsf(v), 1e-30f));
    }
    // argmin over the 16 candidates of this half-warp (ties: the smaller j)
    float best = err;
    int who = j;
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
        const float oe = __shfl_xor_sync(0xffffffffu, best, o);
        const int ow = __shfl_xor_sync(0xffffffffu, who, o);
        if (oe < best || (oe == best && ow < who)) { best = oe; who = ow; }
    }
    if (j == who) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            hi[i] = i < (1 << BITS) ? static_cast<uint8_t>(hb[i < (1 << BITS) ? i : 0]) : 0;
            lo[i] = i < (1 << BITS) ? static_cast<uint8_t>(lb[i < (1 << BITS) ? i : 0]) : 0;
        }
    }
    const float Sw = __uint_as_float(static_cast<uint32_t>(127 + e) << 23) * (1.f + static_cast<float>(who) * 0.0625f);
    return 1.f / Sw;
}

#ifdef TQ_UM_TRACE
// Debug build only: lane 0 of each role of CTA (0,0,0) writes the SM clock at pipeline events into the buffer passed
// as skip_stats: trace[role * 2048 + tile * 16 + event].
#define UM_TRACE(role, tile, ev)                                                                          \
    do {                                                                                                  \
        if (trace_on && lane == 0 && (tile) < 128) p.skip_stats[(role) * 2048 + (tile) * 16 + (ev)] = static_cast<uint32_t>(clock()); \
    } while (0)
#else
#define UM_TRACE(role, tile, ev) do {} while (0)
#endif

template <int KB, int VB, bool QJL>
__global__ void __launch_bounds__(kUmThreads, 2) decode_umma_kernel(const DecodeParams p) {
    static_assert(KB <= 3 && VB <= 3, "byte-table dequantisation holds at most 8 centroids");
    constexpr int NWK = KB + (QJL ? 1 : 0);
    constexpr int RK = 16 * NWK;
    constexpr int KN_OFF = 16 * RK;
    constexpr int KRN_OFF = KN_OFF + 32;
    constexpr int KPART = KN_OFF + 32 + (QJL ? 32 : 0);
    constexpr int VN_OFF = KPART + 256 * VB;
    constexpr int PAGE = KPART + 256 * VB + 32;
    constexpr int PSTRIDE = um_page_stride(PAGE);
    constexpr int STAGE = kUmTilePages * PSTRIDE;

    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + UmSmem::kBars);
    const uint32_t sbase = smem_u32(smem);
    float* scal = reinterpret_cast<float*>(smem + UmSmem::kScal);

    pdl_release_and_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunk = blockIdx.x;
    const int kvh = blockIdx.y / p.ngroups, qg = blockIdx.y % p.ngroups;
    const int seq = blockIdx.z;
#ifdef TQ_UM_TRACE
    const bool trace_on = p.skip_stats && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    UM_TRACE(4, 0, 0);
#endif
    const int L = p.seq_lens[seq];
    const bool too_long = L > p.max_pages * kPageTokens;
    const int npages = too_long ? p.max_pages : (L + kPageTokens - 1) / kPageTokens;
    const int nq = min(8, p.G - qg * 8);
    const int head0 = kvh * p.G + qg * 8;
    if (L <= 0) {
        if (chunk == 0) {
            for (int i = tid; i < nq * kHeadDim; i += kUmThreads) {
                const int64_t o = (static_cast<int64_t>(seq) * p.Hq + head0 + i / kHeadDim) * kHeadDim + i % kHeadDim;
                static_cast<uint16_t*>(p.out)[o] = 0;
            }
        }
        return;
    }
    const int p0 = chunk * p.chunk_pages;
    if (p0 >= npages) return;
    const int p1 = min(p0 + p.chunk_pages, npages);
    const int n_tiles = (p1 - p0 + kUmTilePages - 1) / kUmTilePages;
    const int nchunks = (npages + p.chunk_pages - 1) / p.chunk_pages;

    // ---- set-up: barriers, tensor memory, byte tables, query operands -----------------------------------------
    if (tid == 0) {
        for (int s = 0; s < kUmStages; ++s) {
            mbar_init(bars + kFull + s, 1);
            mbar_init(bars + kEmpty + s, 8);          // one arrival per key / value warp
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bars + kKReady + b, 4);         // key warps
            mbar_init(bars + kPReady + b, 4);
            mbar_init(bars + kVReady + b, 4);         // value warps
            mbar_init(bars + kPVDone + b, 1);
        }
        mbar_init(bars + kSDone, 1);                  // tcgen05.commit
        mbar_init(bars + kSFree, 4);                  // key warps have read the score accumulators
        mbar_init(bars + kSDone, 1);                  // tcgen05.commit
        mbar_init(bars + kSFree, 4);                  // key warps have read the score accumulators
        fence_barrier_init();
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + UmSmem::kTmemSlot), "r"(static_cast<uint32_t>(kUmTmemCols)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp == 8) {
        // lanes 0-15: key codebook, lanes 16-31: value codebook
        const float inv_s = lane < 16 ? build_byte_tables<KB>(p.kc, smem + UmSmem::kTab, smem + UmSmem::kTab + 8, lane)
                                      : build_byte_tables<VB>(p.vc, smem + UmSmem::kTab + 16, smem + UmSmem::kTab + 24, lane);
        if (lane == 0) scal[0] = inv_s;             // completed below once the query scale is known
        if (lane == 16) scal[2] = inv_s * (1.f / kWScale);
    }
    if (warp == 0) {
        // Query rows of the group (lane = (row gid, quarter tig) as in the mma.sync kernel), split q = q1 + q2 in e4m3
        // under one power-of-two scale for the whole group, written as K-major B operands: row r = q1 of head r,
        // row 8 + r = q2; byte (k / 16) * 256 + row * 16 + k % 16.
        const int gid = lane >> 2, tig = lane & 3;
        const bool valid = qg * 8 + gid < p.G;
        const int64_t row = (static_cast<int64_t>(seq) * p.Hq + head0 + gid) * kHeadDim;
        float xq[32];
        load_q32(p.q, row, tig, p.io_dtype, valid, xq);
        if (p.rotate_q) rotate_q32(xq, lane, p.io_dtype);
        auto write_operand = [&](const float (&x)[32], uint32_t dst, bool permute_for_signs) -> float {
            float mx = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fabsf(x[i]));
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            int e = 0;
            if (mx > 0.f && mx < __uint_as_float(0x7f800000u)) e = 134 - static_cast<int>((__float_as_uint(mx) >> 23) & 0xffu);
            e = max(-100, min(100, e));
            const float S = __uint_as_float(static_cast<uint32_t>(127 + e) << 23);
            uint32_t b1[8], b2[8];
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                uint32_t r1 = 0, r2 = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    // sign operand: operand byte (register w, byte i) of a quarter faces residual-sign bit 8 i + 7 - w
                    const int src = permute_for_signs ? 8 * i + 7 - w : 4 * w + i;
                    const float v = x[src] * S;
                    const uint32_t h = cvt_e4m3x2(0.f, v) & 0xffu;
                    const uint32_t l = cvt_e4m3x2(0.f, v - e4m3_to_float(h)) & 0xffu;
                    r1 |= h << (8 * i);
                    r2 |= l << (8 * i);
                }
                b1[w] = r1;
                b2[w] = r2;
            }
            const uint32_t a0 = dst + (2 * tig) * 256 + gid * 16;
            sts_u128(a0, b1[0], b1[1], b1[2], b1[3]);
            sts_u128(a0 + 256, b1[4], b1[5], b1[6], b1[7]);
            sts_u128(a0 + 128, b2[0], b2[1], b2[2], b2[3]);
            sts_u128(a0 + 128 + 256, b2[4], b2[5], b2[6], b2[7]);
            return __uint_as_float(static_cast<uint32_t>(127 - e) << 23);   // 1 / S
        };
        const float inv_sq = write_operand(xq, sbase + UmSmem::kQ, false);
        float inv_sqp = inv_sq;
        if constexpr (QJL) {
            if (p.qp) load_q32(p.qp, row, tig, p.io_dtype, valid, xq);
            inv_sqp = write_operand(xq, sbase + UmSmem::kQP, true);
        }
        if (lane == 0) {
            scal[3] = inv_sq * p.qscale;                      // times 1 / S_k below
            scal[1] = inv_sqp * p.qpscale * (1.f / 16.f);     // qpscale carries the mma.sync kernel's factor 16
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *reinterpret_cast<volatile uint32_t*>(smem + UmSmem::kTmemSlot);
    const float mse_scale = scal[0] * scal[3], qjl_scale = scal[1], out_scale = scal[2];
    UM_TRACE(4, 0, 1 + (warp & 7));

    bool timed_out = false, bad_block = false;
    const uint8_t* head_base = p.cache + (static_cast<int64_t>(kvh) << p.sub_shift) * PAGE;

    if (warp == 8) {
        // =================================== producer ===================================
        const int32_t* bt = p.block_tables + static_cast<int64_t>(seq) * p.bt_stride;
        for (int i = 0; i < n_tiles && !timed_out; ++i) {
            const int s = i % kUmStages;
            if (i >= kUmStages && !mbar_wait_bounded(bars + kEmpty + s, ((i / kUmStages) - 1) & 1)) { timed_out = true; break; }
            const int pg0 = p0 + i * kUmTilePages;
            const int live = min(kUmTilePages, p1 - pg0);
            if (lane == 0) mbar_expect_tx(bars + kFull + s, static_cast<uint32_t>(live) * PAGE);
            UM_TRACE(3, i, 0);
            __syncwarp();
            if (lane < live) {
                const int pg = pg0 + lane;
                int32_t blk = __ldg(bt + (pg >> p.sub_shift));
                if (blk < 0 || blk >= p.num_blocks) { bad_block = true; blk = 0; }
                const uint8_t* src = head_base + static_cast<int64_t>(blk) * p.block_stride + (pg & ((1 << p.sub_shift) - 1)) * PAGE;
                bulk_g2s(smem + UmSmem::kRing + s * STAGE + lane * PSTRIDE, src, PAGE, bars + kFull + s);
            }
        }
    } else if (warp == 9) {
        // =================================== MMA issue ===================================
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc(128, 16, 0, 0), idesc_pv = umma_idesc(128, 16, 1, 1);
            auto issue_s = [&](int i) {
                const int b = i & 1;
                const uint32_t planes = tbase + kColPlanes + b * 96, d = tbase + kColS;
#pragma unroll
                for (int pl = 0; pl < 2; ++pl)
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        umma_ts(d, planes + pl * 32 + ks * 8, umma_desc(sbase + UmSmem::kQ + ks * 512, 256, 128), idesc_s, (pl | ks) ? 1u : 0u);
                if constexpr (QJL) {
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        umma_ts(d + 16, planes + 64 + ks * 8, umma_desc(sbase + UmSmem::kQP + ks * 512, 256, 128), idesc_s, ks ? 1u : 0u);
                }
                umma_commit(bars + kSDone);
            };
            if (mbar_wait_bounded(bars + kKReady + 0, 0)) { tc_fence_after(); issue_s(0); } else timed_out = true;
            for (int i = 0; i < n_tiles && !timed_out; ++i) {
                const int b = i & 1;
                const uint32_t ph = (i >> 1) & 1;
                if (i + 1 < n_tiles) {
                    // the next tile's planes are ready and the key warps have read this tile's scores out of the accumulators
                    if (!mbar_wait_bounded(bars + kKReady + (b ^ 1), ((i + 1) >> 1) & 1) || !mbar_wait_bounded(bars + kSFree, i & 1)) { timed_out = true; break; }
                    tc_fence_after();
                    UM_TRACE(2, i + 1, 0);
                    issue_s(i + 1);
                    UM_TRACE(2, i + 1, 1);
                }
                if (!mbar_wait_bounded(bars + kPReady + b, ph) || !mbar_wait_bounded(bars + kVReady + b, ph)) { timed_out = true; break; }
                tc_fence_after();
                UM_TRACE(2, i, 2);
                const uint32_t d = tbase + kColO + b * 16;
#pragma unroll
                for (int pl = 0; pl < 2; ++pl)
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        umma_ss(d, umma_desc(sbase + UmSmem::kV + b * 32768 + pl * 16384 + ks * 4096, 1024, 128),
                                umma_desc(sbase + UmSmem::kP + b * 2048 + ks * 512, 128, 128), idesc_pv, (pl | ks) ? 1u : 0u);
                umma_commit(bars + kPVDone + b);
                UM_TRACE(2, i, 3);
            }
        }
    } else if (warp < 4) {
        // =================================== key warps: dequantise K, softmax ===================================
        const int pg = tid & 7, tok = tid >> 3;                       // tensor-memory lane tid = tok * 8 + pg
        const uint32_t lane_addr = tbase + (static_cast<uint32_t>(warp * 32) << 16);
        const uint32_t khi0 = *reinterpret_cast<const uint32_t*>(smem + UmSmem::kTab), khi1 = *reinterpret_cast<const uint32_t*>(smem + UmSmem::kTab + 4);
        const uint32_t klo0 = *reinterpret_cast<const uint32_t*>(smem + UmSmem::kTab + 8), klo1 = *reinterpret_cast<const uint32_t*>(smem + UmSmem::kTab + 12);
        float kn_next = 0.f, krn_next = 0.f, vn_next = 0.f;
        bool valid_next = false;
        auto dequant_k = [&](int i) -> bool {
            const int s = i % kUmStages, b = i & 1;
            if (!mbar_wait_bounded(bars + kFull + s, (i / kUmStages) & 1)) return false;
            UM_TRACE(0, i, 0);
            const uint32_t page = sbase + UmSmem::kRing + s * STAGE + pg * PSTRIDE;
            const uint32_t rec = page + tok * RK;
            uint32_t w[4 * NWK];
#pragma unroll
            for (int j = 0; j < NWK; ++j) {
                const uint4 v = lds_u128(rec + 16 * j);
                w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
            }
            kn_next = lds_half(page + KN_OFF + 2 * norm_slot(tok));
            if constexpr (QJL) krn_next = lds_half(page + KRN_OFF + 2 * norm_slot(tok));
            vn_next = lds_half(page + VN_OFF + 2 * norm_slot(tok));
            const int gpage = p0 + i * kUmTilePages + pg;
            valid_next = gpage < p1 && gpage * kPageTokens + tok < L;
            const uint32_t planes = lane_addr + kColPlanes + b * 96;
#pragma unroll
            for (int qt = 0; qt < 4; ++qt) {
                uint32_t iw[KB], mw[4];
#pragma unroll
                for (int j = 0; j < KB; ++j) iw[j] = w[qt * NWK + j];
                masked_words<KB>(iw, mw);
                uint32_t hi[8], lo[8];
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const uint32_t sel = (r & 1) ? (mw[r >> 1] >> 16) : mw[r >> 1];   // prmt reads the low four nibbles only
                    hi[r] = prmt(khi0, khi1, sel);
                    lo[r] = prmt(klo0, klo1, sel);
                }
                tmem_st8(planes + qt * 8, hi);
                tmem_st8(planes + 32 + qt * 8, lo);
                if constexpr (QJL) {
                    const uint32_t sw = w[qt * NWK + KB];
                    uint32_t sg[8];
#pragma unroll
                    for (int r = 0; r < 8; ++r) sg[r] = ((sw << r) & 0x80808080u) ^ 0xB8B8B8B8u;   // bit = 1 -> +1.0 (0x38), 0 -> -1.0 (0xB8)
                    tmem_st8(planes + 64 + qt * 8, sg);
                }
            }
            UM_TRACE(0, i, 1);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bars + kKReady + b);
                mbar_arrive(bars + kEmpty + s);
            }
            UM_TRACE(0, i, 2);
            return true;
        };

        float l_acc[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) l_acc[h] = 0.f;
        float m_run = -INFINITY;                                     // lanes 0..7 of warp 0: running maximum of head `lane`
        if (!dequant_k(0)) timed_out = true;
        for (int i = 0; i < n_tiles && !timed_out; ++i) {
            const int b = i & 1;
            const float kn = kn_next * mse_scale, krn = krn_next * qjl_scale;
            const float vn = fmaxf(vn_next, 9.094947e-13f);            // 2^-40: a zero value norm still counts in the denominator
            const bool valid = valid_next;
            if (i + 1 < n_tiles && !dequant_k(i + 1)) { timed_out = true; break; }
            UM_TRACE(0, i, 3);
            if (!mbar_wait_bounded(bars + kSDone, i & 1)) { timed_out = true; break; }
            tc_fence_after();
            UM_TRACE(0, i, 4);
            uint32_t d[16], dq[16];
            tmem_ld16(lane_addr + kColS, d);
            if constexpr (QJL) tmem_ld16(lane_addr + kColS + 16, dq);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + kSFree);
            UM_TRACE(0, i, 5);
            const float lvn = lg2(vn);
            float sc[8];
            int imax[8];
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                float s = (__uint_as_float(d[h]) + __uint_as_float(d[8 + h])) * kn;
                if constexpr (QJL) s = fmaf(__uint_as_float(dq[h]) + __uint_as_float(dq[8 + h]), krn, s);
                s += lvn;
                sc[h] = valid ? s : -INFINITY;
                imax[h] = redux_max(__float2int_rd(fminf(fmaxf(sc[h], -1.0e6f), 1.0e6f) * 1024.f) + 1);   // >= the true maximum, in 1/1024 steps
            }
            // exchange of the four warps' maxima; lanes 0..7 of warp 0 own the running maximum of head `lane`
            const uint32_t stat = sbase + UmSmem::kStat + (i & 3) * 224;
            if (lane < 8) {
                int mine = imax[0];
#pragma unroll
                for (int h = 1; h < 8; ++h) mine = lane == h ? imax[h] : mine;
                asm volatile("st.shared.u32 [%0], %1;" ::"r"(stat + 96 + (lane * 4 + warp) * 4), "r"(mine) : "memory");
            }
            UM_TRACE(0, i, 6);
            asm volatile("bar.sync 2, 128;" ::: "memory");
            UM_TRACE(0, i, 7);
            if (warp == 0 && lane < 8) {
                const uint4 wm = lds_u128(stat + 96 + lane * 16);
                const int im = max(max(static_cast<int>(wm.x), static_cast<int>(wm.y)), max(static_cast<int>(wm.z), static_cast<int>(wm.w)));
                const float m_tile = static_cast<float>(im) * (1.f / 1024.f);
                const float m_new = fmaxf(m_run, m_tile);
                const float alpha = ex2(m_run - m_new), beta = ex2(m_tile - m_new);
                m_run = m_new;
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(stat + lane * 4), "f"(m_tile) : "memory");
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(stat + 32 + lane * 4), "f"(alpha) : "memory");
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(stat + 64 + lane * 4), "f"(beta) : "memory");
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");
            UM_TRACE(0, i, 8);
            float mt[8], al[8], be[8];
            {
                const float4 a = lds_f128(stat), c = lds_f128(stat + 16), e = lds_f128(stat + 32), f = lds_f128(stat + 48),
                             g = lds_f128(stat + 64), hh = lds_f128(stat + 80);
                mt[0] = a.x; mt[1] = a.y; mt[2] = a.z; mt[3] = a.w; mt[4] = c.x; mt[5] = c.y; mt[6] = c.z; mt[7] = c.w;
                al[0] = e.x; al[1] = e.y; al[2] = e.z; al[3] = e.w; al[4] = f.x; al[5] = f.y; al[6] = f.z; al[7] = f.w;
                be[0] = g.x; be[1] = g.y; be[2] = g.z; be[3] = g.w; be[4] = hh.x; be[5] = hh.y; be[6] = hh.z; be[7] = hh.w;
            }
            const float rvn = __frcp_rn(vn);
            uint32_t b1[4], b2[4];
            float w1v[8], w2v[8];
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                const float ws = ex2(sc[h] - mt[h]) * kWScale;              // weight <= 1 (up to the 1/1024 step), times 256
                w1v[h] = __uint_as_float(__float_as_uint(ws) & 0xFFF00000u);   // 4 significant bits: exact in e4m3 when in range
                w2v[h] = __uint_as_float(__float_as_uint(ws - w1v[h]) & 0xFFF00000u);
                // the denominator sums the weight the value product really uses (w1 + w2), so a lone token comes out exactly
                l_acc[h] = fmaf(l_acc[h], al[h], (w1v[h] + w2v[h]) * (rvn * (1.f / kWScale)) * be[h]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                b1[j] = cvt_e4m3x2(w1v[2 * j + 1], w1v[2 * j]);
                b2[j] = cvt_e4m3x2(w2v[2 * j + 1], w2v[2 * j]);
            }
            // The P buffer of this parity was last read by the value product two tiles ago.  The MMA thread issued that
            // product before the score product of this tile, and tcgen05 operations of one thread complete in order:
            // seeing S(i) done (above) already says that PV(i - 2) is done.
            sts_u128(sbase + UmSmem::kP + b * 2048 + tid * 16, b1[0] | (b1[1] << 16), b1[2] | (b1[3] << 16),
                     b2[0] | (b2[1] << 16), b2[2] | (b2[3] << 16));
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + kPReady + b);
            UM_TRACE(0, i, 11);
        }
        // ---- denominators: reduce the per-thread sums over the 128 token slots --------------------------------
#pragma unroll
        for (int h = 0; h < 8; ++h) {
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) l_acc[h] += __shfl_xor_sync(0xffffffffu, l_acc[h], o);
        }
        if (lane == 0) {
            float* lred = reinterpret_cast<float*>(smem + UmSmem::kLred) + warp * 8;
#pragma unroll
            for (int h = 0; h < 8; ++h) lred[h] = l_acc[h];
        }
        if (warp == 0 && lane < 8) scal[4 + lane] = m_run;
    } else {
        // =================================== value warps: dequantise V, accumulate ===================================
        const int vt = tid - 128;                                      // also the output dim this thread accumulates
        const int vw = warp - 4;
        const int pg = lane & 7;
        const int g = (lane >> 3) + 4 * (vw & 1);
        const uint32_t lane_addr = tbase + (static_cast<uint32_t>(vw * 32) << 16);
        const uint32_t vhi0 = *reinterpret_cast<const uint32_t*>(smem + UmSmem::kTab + 16), vhi1 = *reinterpret_cast<const uint32_t*>(smem + UmSmem::kTab + 20);
        const uint32_t vlo0 = *reinterpret_cast<const uint32_t*>(smem + UmSmem::kTab + 24), vlo1 = *reinterpret_cast<const uint32_t*>(smem + UmSmem::kTab + 28);
        float oacc[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) oacc[h] = 0.f;
        auto accumulate = [&](int i) -> bool {
            const int b = i & 1;
            UM_TRACE(1, i, 4);
            if (!mbar_wait_bounded(bars + kPVDone + b, (i >> 1) & 1)) return false;
            tc_fence_after();
            UM_TRACE(1, i, 5);
            uint32_t d[16];
            tmem_ld16(lane_addr + kColO + b * 16, d);
            tmem_wait_ld();
            const uint32_t stat = sbase + UmSmem::kStat + (i & 3) * 224;
            const float4 e = lds_f128(stat + 32), f = lds_f128(stat + 48), gg = lds_f128(stat + 64), hh = lds_f128(stat + 80);
            const float al[8] = {e.x, e.y, e.z, e.w, f.x, f.y, f.z, f.w}, be[8] = {gg.x, gg.y, gg.z, gg.w, hh.x, hh.y, hh.z, hh.w};
#pragma unroll
            for (int h = 0; h < 8; ++h)
                oacc[h] = fmaf(oacc[h], al[h], (__uint_as_float(d[h]) + __uint_as_float(d[8 + h])) * be[h]);
            UM_TRACE(1, i, 6);
            return true;
        };
        for (int i = 0; i < n_tiles && !timed_out; ++i) {
            const int s = i % kUmStages, b = i & 1;
            UM_TRACE(1, i, 0);
            if (!mbar_wait_bounded(bars + kFull + s, (i / kUmStages) & 1)) { timed_out = true; break; }
            UM_TRACE(1, i, 1);
            // the V planes of this parity were last read by the value product two tiles ago: that product was waited
            // for when tile i - 2 was accumulated (previous iteration)
            const uint32_t vpart = sbase + UmSmem::kRing + s * STAGE + pg * PSTRIDE + KPART + g * 4;
            const uint32_t vdst = sbase + UmSmem::kV + b * 32768 + g * 128 + pg * 16;
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int pair = (vw >> 1) * 4 + it;
                uint32_t pw[VB], mv[4];
#pragma unroll
                for (int j = 0; j < VB; ++j) pw[j] = lds_w(vpart + (j * 8 + pair) * 32);
                masked_words<VB>(pw, mv);
                uint32_t ehi[4], elo[4], ohi[4], olo[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t se = mv[u], so = mv[u] >> 16;
                    ehi[u] = prmt(vhi0, vhi1, se);
                    elo[u] = prmt(vlo0, vlo1, se);
                    ohi[u] = prmt(vhi0, vhi1, so);
                    olo[u] = prmt(vlo0, vlo1, so);
                }
                const uint32_t da = vdst + (2 * pair) * 1024;          // token 2 pair of page pg sits at k = tok * 8 + pg
                sts_u128(da, ehi[0], ehi[1], ehi[2], ehi[3]);
                sts_u128(da + 16384, elo[0], elo[1], elo[2], elo[3]);
                sts_u128(da + 1024, ohi[0], ohi[1], ohi[2], ohi[3]);
                sts_u128(da + 1024 + 16384, olo[0], olo[1], olo[2], olo[3]);
            }
            UM_TRACE(1, i, 2);
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bars + kVReady + b);
                mbar_arrive(bars + kEmpty + s);
            }
            UM_TRACE(1, i, 3);
            if (i >= 1 && !accumulate(i - 1)) { timed_out = true; break; }
        }
        if (!timed_out && !accumulate(n_tiles - 1)) timed_out = true;

        // ---- epilogue: thread vt owns output dim vt of the group's heads ---------------------------------------
        asm volatile("bar.sync 3, 256;" ::: "memory");                 // key warps have published m and the denominators
        const float* lred = reinterpret_cast<const float*>(smem + UmSmem::kLred);
        float* sm_wht = reinterpret_cast<float*>(smem + UmSmem::kV);    // scratch for the output rotation (V planes are dead)
        for (int h = 0; h < nq; ++h) {
            const float o = oacc[h] * out_scale;
            const float l = (lred[h] + lred[8 + h]) + (lred[16 + h] + lred[24 + h]);
            if (nchunks == 1) {
                float r = o / l;
                if (p.derotate_out) r = block_wht128(r, sm_wht, vt);
                const int64_t off = (static_cast<int64_t>(seq) * p.Hq + head0 + h) * kHeadDim + vt;
                if (p.io_dtype == TQ_DTYPE_F16) static_cast<__half*>(p.out)[off] = __float2half_rn(r);
                else static_cast<__nv_bfloat16*>(p.out)[off] = __float2bfloat16_rn(r);
            } else {
                const int64_t slot = ((static_cast<int64_t>(seq) * p.Hkv * p.ngroups + blockIdx.y) * p.max_chunks + chunk) * 8 + h;
                p.ws_o[slot * kHeadDim + vt] = o;
                if (vt == 0) {
                    p.ws_ml[slot * 2] = scal[4 + h];
                    p.ws_ml[slot * 2 + 1] = l;
                }
            }
        }
    }
    if (warp < 4) asm volatile("bar.sync 3, 256;" ::: "memory");       // pairs with the value warps' epilogue barrier

    if (p.status) {
        int bits = 0;
        if (__any_sync(0xffffffffu, bad_block) || (too_long && tid == 0)) bits |= TQ_STATUS_BAD_BLOCK;
        if (__any_sync(0xffffffffu, timed_out)) bits |= TQ_STATUS_TIMEOUT;
        if (bits && lane == 0) atomicOr(p.status, bits);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(static_cast<uint32_t>(kUmTmemCols)) : "memory");
}

template <int KB, int VB, bool QJL>
int launch_umma(const DecodeParams& p, dim3 grid, cudaStream_t stream) {
    constexpr int PAGE = page_bytes(KB, VB, QJL ? 1 : 0);
    constexpr size_t smem = UmSmem::kRing + static_cast<size_t>(kUmStages) * kUmTilePages * um_page_stride(PAGE);
    static_assert(smem <= 113 * 1024, "two CTAs per SM");
    auto kern = decode_umma_kernel<KB, VB, QJL>;
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TQ_ERR_LAUNCH;
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
            return TQ_ERR_LAUNCH;
        configured[dev] = true;
    }
    return launch_chained(kern, grid, dim3(kUmThreads), smem, stream, p) == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

}  // namespace
}  // namespace tq
