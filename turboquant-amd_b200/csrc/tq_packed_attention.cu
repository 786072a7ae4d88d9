// Contiguous packed decode attention (one query row per BH, no GQA, no paging) and the
// row-wise fast Walsh-Hadamard rotation, for sm_100a.
//
// packed_attention keeps the data layout of the reference's Triton path
// (turboquant/kernels/packed_attention.py:76-227): token-major index bytes,
// sign bytes in the stride-4 order of permute_signs_for_chunked
// (turboquant/kernels/packed_compress.py:180-216) and separate fp16 norm arrays.
// With one query per K/V stream there is no group to share tensor-core tiles, so
// this kernel is CUDA-core code built around conflict-free shared-memory tables:
//  * a warp takes 8 tokens per step, lane = 4 * slot + quarter: the lane reads the quarter's index words of its
//    token (the warp's loads cover 8 whole rows) and keeps the quarter's 32 query values in registers;
//  * pair table: (c[i0], c[i1]) as two floats for every pair of indices, one copy per lane (entry stride 256 B), so a
//    64-bit load per two adjacent dims never collides on a bank; K scores and the V sum use f32x2 multiply-adds;
//  * sign table of the query: for each of a quarter's 8 sign nibbles the 16 sums of +-q' over its 4 dims, one copy
//    per lane; the QJL term is 8 look-ups per lane instead of 32 selects;
//  * every slot runs its own online softmax over the tokens it sees (no shuffles across tokens in the loop, the
//    maximum is only raised when a score exceeds it by 2^8); slots, warps and splits are merged at the end.
#include "tq_common.cuh"

namespace tq {
namespace {

// Warps per CTA: 8 (two CTAs per SM, so that one CTA's table set-up and final merge overlap the other's token loop)
// where two sets of tables fit in shared memory, 16 (one CTA per SM) for 4-bit indices.  Either way 16 warps per SM at
// up to 128 registers per thread.
template <int BITS> struct PAWarps { static constexpr int value = BITS == 4 ? 16 : 8; };
constexpr int kSignTabBytes = 8 * 16 * 128;     // [nibble position][nibble value][lane]
constexpr float kLog2e = 1.4426950408889634f;

struct PAParams {
    const __half* Q;
    const __half* Qp;
    const uint8_t* k_idx;
    const uint8_t* k_signs;
    const __half* k_rnorm;
    const __half* k_norm;
    const uint8_t* v_idx;
    const __half* v_norm;
    const float* centroids;
    float* ws_acc;   // [BH, splits, 128]
    float* ws_lse;   // [BH, splits, 2]  (max in the log2 domain, sum)
    __half* out;
    float corr_scale;
    int Sk, num_splits;
};

typedef unsigned long long pa_f2;   // two fp32 in a 64-bit register (sm_100 f32x2 arithmetic)
__device__ __forceinline__ pa_f2 pa_pack(float lo, float hi) {
    pa_f2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void pa_unpack(pa_f2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ pa_f2 pa_fma(pa_f2 a, pa_f2 b, pa_f2 c) {
    pa_f2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ pa_f2 pa_mul(pa_f2 a, pa_f2 b) {
    pa_f2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ pa_f2 pa_lds64(uint32_t addr) {
    pa_f2 v;
    asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float pa_lds32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float pa_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Byte offset, inside a lane-replicated pair table, of this lane's copy of the entry of dims (2 j, 2 j + 1) of a
// quarter: the 2 * BITS index bits at bit 2 * BITS * j of the quarter's little-endian stream, shifted to the entry
// stride 2^SHIFT, or-ed with the lane's offset inside an entry.  One shift and one logic op.
template <int BITS, int SHIFT>
__device__ __forceinline__ uint32_t pair_offset(const uint32_t (&w)[BITS], int j, uint32_t lane_off) {
    constexpr int PB = 2 * BITS;
    constexpr uint32_t kMask = ((1u << PB) - 1u) << SHIFT;
    const int o = PB * j, lo = o >> 5, sh = o & 31;
    uint32_t x;
    if (sh + PB > 32) x = __funnelshift_r(w[lo], w[lo + 1 < BITS ? lo + 1 : lo], sh - SHIFT);
    else if (sh >= SHIFT) x = w[lo] >> (sh - SHIFT);
    else x = w[lo] << (SHIFT - sh);
    return (x & kMask) | lane_off;
}

template <int BITS>
__device__ __forceinline__ void lds_words(uint32_t addr, uint32_t (&w)[BITS]) {
    if constexpr (BITS == 4) {
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr));
    } else if constexpr (BITS == 2) {
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(addr));
    } else {
#pragma unroll
        for (int i = 0; i < BITS; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[i]) : "r"(addr + 4 * i));
    }
}

constexpr int kPaStages = 2;   // ring of 16-token steps per warp: the one being worked on, the others in flight

template <int BITS>
struct PALayout {
    static constexpr int kRow = 16 * BITS;                              // index bytes per token
    static constexpr int kPairs = 1 << (2 * BITS);
    static constexpr int kPairTabBytes = kPairs * 256;                  // (c[i0], c[i1]) as two floats per lane: V
    static constexpr int kHalfTabBytes = kPairs * 128;                  // the same as half2 per lane: K operand of the MMAs
    static constexpr int kSignTabOff = kPairTabBytes + kHalfTabBytes;
    static constexpr int kStageOff = kSignTabOff + kSignTabBytes;
    static constexpr int kStageBytes = 32 * kRow + 256;                 // 16 K rows, 16 V rows, 16 sign rows
    static constexpr int kWarps = PAWarps<BITS>::value;
    static constexpr int kThreads = kWarps * 32;
    static constexpr int kStepTokens = kWarps * 16;                     // tokens one step of the whole CTA covers
    static constexpr int kSmem = kStageOff + kWarps * kPaStages * kStageBytes;
};

// A warp takes 16 tokens per step.  Lane (slot, quarter) = (lane >> 2, lane & 3) owns quarter `quarter` (32 dims) of
// tokens slot and slot + 8 of the step:
//  * K score: the lane's 16 pairs of adjacent dims of both tokens are looked up as half2 and are, as they come, the A
//    operands of 8 m16n8k16 MMAs (row = token, the 16 k-slots of MMA ks are dims 4 ks .. 4 ks + 3 of the four
//    quarters); the B operand carries the query in column 0 only, so the fp32 dot products land in the quarter-0 lanes;
//  * QJL term: per quarter, 8 look-ups in the query's sign table;
//  * V: per token 16 look-ups of (c[i0], c[i1]) as floats, f32x2 multiply-adds into the lane's 32 accumulators.
// Every slot runs its own online softmax (no exchange between tokens inside the loop).
template <int BITS>
__global__ void __launch_bounds__(PAWarps<BITS>::value * 32, 16 / PAWarps<BITS>::value) packed_attn_partial(const PAParams p, int n_items) {
    using LO = PALayout<BITS>;
    constexpr int ROW = LO::kRow;
    constexpr int kPaWarps = LO::kWarps, kThreads = LO::kThreads, kStepTokens = LO::kStepTokens;
    extern __shared__ __align__(128) unsigned char pa_smem[];
    unsigned char* pair_tab = pa_smem;
    unsigned char* half_tab = pa_smem + LO::kPairTabBytes;
    unsigned char* sign_tab = pa_smem + LO::kSignTabOff;        // [nibble position][value][lane] float
    __shared__ __align__(16) float sqp[kHeadDim];
    __shared__ float scb[1 << BITS];
    __shared__ __align__(16) float sacc[kPaWarps][kHeadDim];
    __shared__ float sml[kPaWarps][2];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slot = lane >> 2, quarter = lane & 3;
    const int per = (p.Sk + p.num_splits - 1) / p.num_splits;   // tokens per split (packed_attention.py:98-100)
    // the pair tables depend on the codebook only: built once, the CTA then strides over (row, split) items
    if (tid < (1 << BITS)) scb[tid] = p.centroids[tid];
    __syncthreads();
    for (int e = tid; e < LO::kPairs * 32; e += kThreads) {
        const int pr = e >> 5;
        const float c0 = scb[pr & ((1 << BITS) - 1)], c1 = scb[pr >> BITS];
        *reinterpret_cast<float2*>(pair_tab + e * 8) = make_float2(c0, c1);
        *reinterpret_cast<uint32_t*>(half_tab + e * 4) = pack_half2(c0, c1);
    }
    // ---- item state: which (row, split) the CTA works on, and the warp's asynchronous staging of it: per step a warp
    // copies its 16 K rows, 16 V rows and 16 sign rows in 16-byte pieces (every row is a multiple of 16 bytes, so any
    // token starts on a 16-byte boundary) ----
    const uint32_t stage0 = smem_u32(pa_smem + LO::kStageOff + warp * kPaStages * LO::kStageBytes);
    int bh = 0, split = 0, t1 = 0;
    int tok16 = 0;                                              // first token of this warp's current step
    const uint8_t *kptr = nullptr, *vptr = nullptr, *sptr = nullptr;
    const uint16_t *knp = nullptr, *krnp = nullptr, *vnp = nullptr;
    int tok_issue = 0, stage_issue = 0;
    uint16_t nrm[6] = {0, 0, 0, 0, 0, 0};                       // kn, krn, vn of token A (slot); of token B (slot + 8)
    // token row of this lane's pieces (piece c + lane of the 16 rows); 99 = the lane has no such piece
    int piece_row[(ROW + 31) / 32];
#pragma unroll
    for (int c = 0; c < ROW; c += 32) piece_row[c / 32] = c + lane < ROW ? ((c + lane) * 16) / ROW : 99;
    auto issue = [&]() {
        const uint32_t dst = stage0 + stage_issue * LO::kStageBytes + lane * 16;
#pragma unroll
        for (int c = 0; c < ROW; c += 32) {
            if (tok_issue + piece_row[c / 32] < t1 && piece_row[c / 32] < 16) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + c * 16), "l"(kptr + c * 16) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16 * ROW + c * 16), "l"(vptr + c * 16) : "memory");
            }
        }
        if (lane < 16 && tok_issue + lane < t1)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 32 * ROW), "l"(sptr) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
        kptr += kStepTokens * ROW;
        vptr += kStepTokens * ROW;
        sptr += kStepTokens * 16;
        tok_issue += kStepTokens;
        stage_issue = stage_issue + 1 == kPaStages ? 0 : stage_issue + 1;
    };
    auto load_norms = [&](int tk, uint16_t (&n)[6]) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int t = tk + slot + 8 * h;
            if (t < t1) {
                n[3 * h] = __ldg(knp + t);
                n[3 * h + 1] = __ldg(krnp + t);
                n[3 * h + 2] = __ldg(vnp + t);
            } else {
                n[3 * h] = n[3 * h + 1] = n[3 * h + 2] = 0;
            }
        }
    };
    // Starts an item: its first copies and norms are requested here, i.e. (from the second item on) before the merge of
    // the item just finished, so their latency is hidden behind it.
    auto begin_item = [&](int item) {
        bh = item / p.num_splits;
        split = item - bh * p.num_splits;
        const int t0 = min(split * per, p.Sk);
        t1 = min(t0 + per, p.Sk);
        const int64_t base = static_cast<int64_t>(bh) * p.Sk;
        tok16 = t0 + warp * 16;
        kptr = p.k_idx + (base + tok16) * ROW + lane * 16;
        vptr = p.v_idx + (base + tok16) * ROW + lane * 16;
        sptr = p.k_signs + (base + tok16) * 16 + lane * 16;
        knp = reinterpret_cast<const uint16_t*>(p.k_norm) + base;
        krnp = reinterpret_cast<const uint16_t*>(p.k_rnorm) + base;
        vnp = reinterpret_cast<const uint16_t*>(p.v_norm) + base;
        tok_issue = tok16;
        stage_issue = 0;
#pragma unroll
        for (int i = 0; i < kPaStages - 1; ++i) issue();
        load_norms(tok16, nrm);
    };
    int item = blockIdx.x;
    if (item < n_items) begin_item(item);
  while (item < n_items) {
    // B operands: the query's quarter `quarter` as loaded (pairs of adjacent dims), in column 0 (slot 0) only
    uint32_t qf[16];
    {
        const uint4* qsrc = reinterpret_cast<const uint4*>(p.Q + static_cast<int64_t>(bh) * kHeadDim + 32 * quarter);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 v = slot == 0 ? __ldg(qsrc + i) : make_uint4(0u, 0u, 0u, 0u);
            qf[4 * i] = v.x; qf[4 * i + 1] = v.y; qf[4 * i + 2] = v.z; qf[4 * i + 3] = v.w;
        }
    }
    // ---- the query's sign table ----
    if (tid < kHeadDim) sqp[tid] = __half2float(p.Qp[static_cast<int64_t>(bh) * kHeadDim + tid]) * p.corr_scale;
    __syncthreads();
    // Sign nibble g = 2 c + h of a lane's sign word (byte c = byte `quarter` of sign word c) holds, in bit kk, the
    // sign of local dim 4 (4 h + kk) + c (stride-4 order: dim 4 i + c is bit i of word c).
    for (int e = tid; e < 8 * 16 * 32; e += kThreads) {
        const int ln = e & 31, v = (e >> 5) & 15, g = e >> 9, c = g >> 1, h = g & 1, q = ln & 3;
        float acc = 0.f;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const float x = sqp[32 * q + 4 * (4 * h + kk) + c];
            acc += ((v >> kk) & 1) ? x : -x;
        }
        *reinterpret_cast<float*>(sign_tab + e * 4) = acc;
    }
    __syncthreads();
    const uint32_t lane8 = lane * 8, lane4 = lane * 4;
    // selector that gathers byte `quarter` of two sign words
    const uint32_t sel_lo = static_cast<uint32_t>(quarter) | (static_cast<uint32_t>(4 + quarter) << 4);
    const uint32_t my_words = stage0 + lane * (4 * BITS);       // this lane's K words of token A inside a stage
    const uint32_t my_signs = stage0 + 32 * ROW + slot * 16;

    float m_run = -INFINITY, l_run = 0.f;     // this slot's online softmax (log2 domain)
    pa_f2 acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = pa_pack(0.f, 0.f);

    int stage = 0;
    for (; tok16 < t1; tok16 += kStepTokens) {
        const bool valid_a = tok16 + slot < t1, valid_b = tok16 + slot + 8 < t1;
        issue();
        uint16_t nrm_n[6];
        load_norms(tok16 + kStepTokens, nrm_n);
        asm volatile("cp.async.wait_group %0;" ::"n"(kPaStages - 1) : "memory");
        __syncwarp();
        const uint32_t so = stage * LO::kStageBytes;
        uint32_t kwa[BITS], kwb[BITS];
        lds_words<BITS>(my_words + so, kwa);
        lds_words<BITS>(my_words + so + 8 * ROW, kwb);
        uint4 sga, sgb;
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(sga.x), "=r"(sga.y), "=r"(sga.z), "=r"(sga.w) : "r"(my_signs + so));
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(sgb.x), "=r"(sgb.y), "=r"(sgb.z), "=r"(sgb.w) : "r"(my_signs + so + 128));
        // ---- K scores: rows = the 16 tokens, column 0 = the query ----
        float mse[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint32_t a0 = *reinterpret_cast<const uint32_t*>(half_tab + pair_offset<BITS, 7>(kwa, 2 * ks, lane4));
            const uint32_t a1 = *reinterpret_cast<const uint32_t*>(half_tab + pair_offset<BITS, 7>(kwb, 2 * ks, lane4));
            const uint32_t a2 = *reinterpret_cast<const uint32_t*>(half_tab + pair_offset<BITS, 7>(kwa, 2 * ks + 1, lane4));
            const uint32_t a3 = *reinterpret_cast<const uint32_t*>(half_tab + pair_offset<BITS, 7>(kwb, 2 * ks + 1, lane4));
            mma_f16_16816(mse, a0, a1, a2, a3, qf[2 * ks], qf[2 * ks + 1]);
        }
        // ---- QJL term of this lane's quarter, both tokens ----
        const uint32_t swa = prmt(prmt(sga.x, sga.y, sel_lo), prmt(sga.z, sga.w, sel_lo), 0x5410);
        const uint32_t swb = prmt(prmt(sgb.x, sgb.y, sel_lo), prmt(sgb.z, sgb.w, sel_lo), 0x5410);
        float qja = 0.f, qjb = 0.f;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const uint32_t xa = 4 * g >= 7 ? (swa >> (4 * g - 7)) : (swa << (7 - 4 * g));
            const uint32_t xb = 4 * g >= 7 ? (swb >> (4 * g - 7)) : (swb << (7 - 4 * g));
            qja += *reinterpret_cast<const float*>(sign_tab + g * 2048 + ((xa & (15u << 7)) | lane4));
            qjb += *reinterpret_cast<const float*>(sign_tab + g * 2048 + ((xb & (15u << 7)) | lane4));
        }
        // the quarter-0 lane of a slot holds the whole MSE dot product (column 0 of rows slot and slot + 8)
        float pa = __half2float(__ushort_as_half(nrm[1])) * qja, pb = __half2float(__ushort_as_half(nrm[4])) * qjb;
        if (quarter == 0) {
            pa = fmaf(__half2float(__ushort_as_half(nrm[0])), mse[0], pa);
            pb = fmaf(__half2float(__ushort_as_half(nrm[3])), mse[2], pb);
        }
        pa += __shfl_xor_sync(0xffffffffu, pa, 1);
        pb += __shfl_xor_sync(0xffffffffu, pb, 1);
        pa += __shfl_xor_sync(0xffffffffu, pa, 2);
        pb += __shfl_xor_sync(0xffffffffu, pb, 2);
        const float sa = valid_a ? pa * kLog2e : -INFINITY, sb = valid_b ? pb * kLog2e : -INFINITY;
        // ---- online softmax of this slot: the maximum is raised only when a score exceeds it by 2^8 ----
        const float smax = fmaxf(sa, sb);
        if (smax > m_run + 8.f) {
            const float alpha = pa_ex2(m_run - smax);     // 0 on the first token
            const pa_f2 al2 = pa_pack(alpha, alpha);
            l_run *= alpha;
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = pa_mul(acc[j], al2);
            m_run = smax;
        }
        const float pra = valid_a ? pa_ex2(sa - m_run) : 0.f, prb = valid_b ? pa_ex2(sb - m_run) : 0.f;
        l_run += pra + prb;
        // ---- V ----
        {
            uint32_t vw[BITS];
            lds_words<BITS>(my_words + so + 16 * ROW, vw);
            const float wv = pra * __half2float(__ushort_as_half(nrm[2]));
            const pa_f2 wv2 = pa_pack(wv, wv);
#pragma unroll
            for (int j = 0; j < 16; ++j)
                acc[j] = pa_fma(wv2, *reinterpret_cast<const pa_f2*>(pair_tab + pair_offset<BITS, 8>(vw, j, lane8)), acc[j]);
        }
        {
            uint32_t vw[BITS];
            lds_words<BITS>(my_words + so + 24 * ROW, vw);
            const float wv = prb * __half2float(__ushort_as_half(nrm[5]));
            const pa_f2 wv2 = pa_pack(wv, wv);
#pragma unroll
            for (int j = 0; j < 16; ++j)
                acc[j] = pa_fma(wv2, *reinterpret_cast<const pa_f2*>(pair_tab + pair_offset<BITS, 8>(vw, j, lane8)), acc[j]);
        }
#pragma unroll
        for (int i = 0; i < 6; ++i) nrm[i] = nrm_n[i];
        stage = stage + 1 == kPaStages ? 0 : stage + 1;
        __syncwarp();   // every lane has read this stage before the next step's copy may land in it
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    const int64_t out_slot = static_cast<int64_t>(bh) * p.num_splits + split;   // of the item just finished
    item += gridDim.x;
    if (item < n_items) begin_item(item);

    // ---- merge the 8 slots of the warp, then the warps ----
    float M = m_run;
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float f = (m_run == -INFINITY) ? 0.f : pa_ex2(m_run - M);
    float L = l_run * f;
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        float x, y;
        pa_unpack(acc[j], x, y);
        x *= f;
        y *= f;
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            x += __shfl_xor_sync(0xffffffffu, x, o);
            y += __shfl_xor_sync(0xffffffffu, y, o);
        }
        if (slot == 0) *reinterpret_cast<float2*>(&sacc[warp][32 * quarter + 2 * j]) = make_float2(x, y);
    }
    if (lane == 0) {
        sml[warp][0] = M;
        sml[warp][1] = L;
    }
    __syncthreads();
    if (tid < kHeadDim) {
        float Mc = sml[0][0];
#pragma unroll
        for (int w = 1; w < kPaWarps; ++w) Mc = fmaxf(Mc, sml[w][0]);
        float o = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < kPaWarps; ++w) {
            const float fw = (sml[w][0] == -INFINITY) ? 0.f : pa_ex2(sml[w][0] - Mc);
            o = fmaf(fw, sacc[w][tid], o);
            l = fmaf(fw, sml[w][1], l);
        }
        p.ws_acc[out_slot * kHeadDim + tid] = o;
        if (tid == 0) {
            p.ws_lse[out_slot * 2] = Mc;
            p.ws_lse[out_slot * 2 + 1] = l;
        }
    }
    __syncthreads();   // the shared partials and the sign table are free for the next item
  }
}

__global__ void __launch_bounds__(kHeadDim) packed_attn_merge(const PAParams p) {
    const int bh = blockIdx.x, d = threadIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < p.num_splits; ++s) M = fmaxf(M, p.ws_lse[(static_cast<int64_t>(bh) * p.num_splits + s) * 2]);
    float o = 0.f, l = 0.f;
    for (int s = 0; s < p.num_splits; ++s) {
        const int64_t slot = static_cast<int64_t>(bh) * p.num_splits + s;
        const float m = p.ws_lse[slot * 2];
        const float w = (m == -INFINITY) ? 0.f : pa_ex2(m - M);   // empty splits carry no weight
        o = fmaf(w, p.ws_acc[slot * kHeadDim + d], o);
        l = fmaf(w, p.ws_lse[slot * 2 + 1], l);
    }
    p.out[static_cast<int64_t>(bh) * kHeadDim + d] = __float2half_rn(o / l);
}

// ---- row-wise WHT ----------------------------------------------------------------------
__global__ void __launch_bounds__(128) wht_rows_kernel(const void* in, void* out, int dtype, int64_t n, float scale) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (row >= n) return;
    float x[4];
    load4(in, row * kHeadDim + 4 * lane, dtype, x);
    float a = x[0] + x[1], b = x[0] - x[1], c = x[2] + x[3], d = x[2] - x[3];
    x[0] = a + c; x[1] = b + d; x[2] = a - c; x[3] = b - d;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const float sgn = (lane & m) ? -1.f : 1.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) x[e] = fmaf(sgn, x[e], __shfl_xor_sync(0xffffffffu, x[e], m));
    }
    const float k = kWhtScale * scale;
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] *= k;
    const int64_t o = row * kHeadDim + 4 * lane;
    if (dtype == TQ_DTYPE_F32) {
        *reinterpret_cast<float4*>(static_cast<float*>(out) + o) = make_float4(x[0], x[1], x[2], x[3]);
    } else if (dtype == TQ_DTYPE_F16) {
        *reinterpret_cast<uint2*>(static_cast<uint16_t*>(out) + o) = make_uint2(pack_half2(x[0], x[1]), pack_half2(x[2], x[3]));
    } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]), hi = __floats2bfloat162_rn(x[2], x[3]);
        *reinterpret_cast<uint2*>(static_cast<uint16_t*>(out) + o) =
            make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
}

}  // namespace
}  // namespace tq

using namespace tq;

extern "C" int tq_packed_attention_auto_splits(int BH, int Sk) {
    if (BH <= 0 || Sk <= 0) return TQ_ERR_ARG;
    // Two 256-thread CTAs per SM (one 512-thread CTA for 4-bit indices: half as many per wave, so a grid that fills
    // waves of 296 fills waves of 148 too).  Take the split count (at least 1024 tokens per split, at most 64 splits)
    // whose grid fills whole waves best; a small penalty per split keeps the merge short among near-ties.
    const double penalty = 0.002;
    const int max_splits = Sk / 1024 < 1 ? 1 : (Sk / 1024 > 64 ? 64 : Sk / 1024);
    int best = 1;
    double best_score = -1.0;
    for (int s = 1; s <= max_splits; ++s) {
        const double waves = static_cast<double>(BH) * s / 296.0;
        const double full = waves <= 1.0 ? 1.0 : static_cast<double>(static_cast<long long>(waves + 0.999999));
        const double score = waves / full - penalty * s;
        if (score > best_score) {
            best_score = score;
            best = s;
        }
    }
    return best;
}

extern "C" int64_t tq_packed_attention_workspace_bytes(int BH, int num_splits) {
    if (BH <= 0 || num_splits <= 0) return TQ_ERR_ARG;
    return static_cast<int64_t>(BH) * num_splits * (kHeadDim + 2) * static_cast<int64_t>(sizeof(float));
}

extern "C" int tq_packed_attention(const void* Q, const void* Q_proj, const uint8_t* k_idx, const uint8_t* k_signs_perm,
                                   const void* k_rnorm, const void* k_norm, const uint8_t* v_idx, const void* v_norm,
                                   const float* centroids, float corr_scale, int BH, int Sk, int bits, int num_splits,
                                   void* workspace, int64_t workspace_bytes, void* out, tq_stream_t stream) {
    if (BH == 0) return TQ_OK;
    if (!Q || !Q_proj || !k_idx || !k_signs_perm || !k_rnorm || !k_norm || !v_idx || !v_norm || !centroids || !out)
        return TQ_ERR_ARG;
    if (BH < 0 || Sk <= 0) return TQ_ERR_ARG;
    if (bits < 2 || bits > 4) return TQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(k_idx) | reinterpret_cast<uintptr_t>(k_signs_perm) | reinterpret_cast<uintptr_t>(v_idx)) & 15)
        return TQ_ERR_ARG;
    if (num_splits <= 0) num_splits = tq_packed_attention_auto_splits(BH, Sk);
    if (num_splits > Sk) num_splits = Sk;
    if (num_splits > 65535) return TQ_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < tq_packed_attention_workspace_bytes(BH, num_splits)) return TQ_ERR_WORKSPACE;
    PAParams p;
    p.Q = static_cast<const __half*>(Q);
    p.Qp = static_cast<const __half*>(Q_proj);
    p.k_idx = k_idx;
    p.k_signs = k_signs_perm;
    p.k_rnorm = static_cast<const __half*>(k_rnorm);
    p.k_norm = static_cast<const __half*>(k_norm);
    p.v_idx = v_idx;
    p.v_norm = static_cast<const __half*>(v_norm);
    p.centroids = centroids;
    p.ws_acc = static_cast<float*>(workspace);
    p.ws_lse = p.ws_acc + static_cast<int64_t>(BH) * num_splits * kHeadDim;
    p.out = static_cast<__half*>(out);
    p.corr_scale = corr_scale;
    p.Sk = Sk;
    p.num_splits = num_splits;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    static bool configured[64] = {false};
    static int sm_count[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return TQ_ERR_LAUNCH;
    if (dev < 0 || dev >= 64) return TQ_ERR_UNSUPPORTED;
    if (!configured[dev]) {
        if (cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return TQ_ERR_LAUNCH;
        if (cudaFuncSetAttribute(packed_attn_partial<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, PALayout<4>::kSmem) != cudaSuccess ||
            cudaFuncSetAttribute(packed_attn_partial<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, PALayout<3>::kSmem) != cudaSuccess ||
            cudaFuncSetAttribute(packed_attn_partial<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PALayout<2>::kSmem) != cudaSuccess)
            return TQ_ERR_LAUNCH;
        configured[dev] = true;
    }
    // persistent CTAs: as many as are resident at once, each strides over the (row, split) items
    const int64_t items64 = static_cast<int64_t>(BH) * num_splits;
    if (items64 > 2147483647) return TQ_ERR_UNSUPPORTED;
    const int n_items = static_cast<int>(items64);
    const int resident = sm_count[dev] * (bits == 4 ? 1 : 2);
    const unsigned grid = static_cast<unsigned>(n_items < resident ? n_items : resident);
    switch (bits) {
        case 2: packed_attn_partial<2><<<grid, PALayout<2>::kThreads, PALayout<2>::kSmem, st>>>(p, n_items); break;
        case 3: packed_attn_partial<3><<<grid, PALayout<3>::kThreads, PALayout<3>::kSmem, st>>>(p, n_items); break;
        case 4: packed_attn_partial<4><<<grid, PALayout<4>::kThreads, PALayout<4>::kSmem, st>>>(p, n_items); break;
    }
    if (cudaGetLastError() != cudaSuccess) return TQ_ERR_LAUNCH;
    packed_attn_merge<<<BH, kHeadDim, 0, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

extern "C" int tq_wht_rows(const void* in, void* out, int dtype, int64_t n_rows, float scale, tq_stream_t stream) {
    if (n_rows == 0) return TQ_OK;
    if (!in || !out || n_rows < 0) return TQ_ERR_ARG;
    if (dtype != TQ_DTYPE_F16 && dtype != TQ_DTYPE_BF16 && dtype != TQ_DTYPE_F32) return TQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) return TQ_ERR_ARG;
    const unsigned grid = static_cast<unsigned>((n_rows + 3) / 4);
    wht_rows_kernel<<<grid, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(in, out, dtype, n_rows, scale);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}
