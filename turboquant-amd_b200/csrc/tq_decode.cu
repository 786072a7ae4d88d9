// Asymmetric packed paged decode attention (GQA, split-K, optional Sparse-V) for sm_100a.
//
// One CTA = 4 warps works on a chunk of 16-token pages of one (sequence, kv head,
// group of <= 8 query heads).  Every warp owns every 4th page of the chunk and is
// its own producer and consumer: lane 0 streams the next packed pages from HBM
// into the warp's private shared-memory ring with bulk async copies that
// complete on mbarriers, the whole warp then
//   * turns packed indices into fp16 tensor-core fragments: a masked byte of the packed word is
//     the pair index of two neighbouring dims and addresses a lane-replicated half2 table in
//     shared memory (one byte-extract, one multiply-add, one conflict-free shared load per pair),
//   * scores 16 tokens x 8 query heads with mma.m16n8k16 (tokens on M, the GQA
//     group on N), a second MMA chain for the +-1 QJL sign term,
//   * runs the online softmax on the accumulator fragment,
//   * accumulates P V with mma (the transposed P fragment comes from one
//     movmatrix per 8 tokens; the two dims a lane owns per column are told
//     apart by the row half of the accumulator, so V is fed exactly as stored).
// Warps merge in shared memory; chunks merge in a second small kernel.
//
// Arithmetic restated from the reference: score and softmax of
// turboquant/kernels/packed_attention.py:150-196,273-284, paging and GQA head
// mapping of turboquant/kernels/sparse_v.py:39-48,70-71, skip rule of
// sparse_v.py:108-123,149.
#include "tq_common.cuh"

namespace tq {
namespace {

#ifndef TQ_DEC_WARPS
#define TQ_DEC_WARPS 4
#endif
#ifndef TQ_DEC_STAGES
#define TQ_DEC_STAGES 4
#endif
#ifndef TQ_DEC_MINBLOCKS
#define TQ_DEC_MINBLOCKS 4
#endif
#ifndef TQ_DEC_PDL
#define TQ_DEC_PDL 1
#endif
constexpr int kWarps = TQ_DEC_WARPS;
constexpr int kThreads = kWarps * 32;
constexpr int kOPad = 132;  // row stride of the merge buffer (floats)
constexpr int kStages = TQ_DEC_STAGES;  // pages in flight per warp
constexpr int kBarBytes = kWarps * 2 * kStages * 8;  // mbarriers at the start of dynamic shared memory

// Programmatic dependent launch: the partial and merge kernels of consecutive calls are launched with the
// stream-serialization attribute, so a kernel's CTAs are scheduled while the previous kernel drains.  Each kernel
// lets its successor go at once and waits for its predecessor's results before it reads or writes anything; both
// instructions do nothing in a kernel that was launched without the attribute.
__device__ __forceinline__ void pdl_release_and_wait() {
#if TQ_DEC_PDL
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
#endif
}

template <typename Kernel, typename... Args>
cudaError_t launch_chained(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
#if TQ_DEC_PDL
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
#else
    kernel<<<grid, block, smem, stream>>>(args...);
    return cudaGetLastError();
#endif
}

struct DecodeParams {
    void* out;
    const void* q;
    const void* qp;
    const uint8_t* cache;
    const int32_t* block_tables;
    const int32_t* seq_lens;
    const float* kc;
    const float* vc;
    float* ws_o;
    float* ws_ml;
    int32_t* status;
    uint32_t* skip_stats;
    int64_t bt_stride;
    int64_t num_blocks;
    float qscale;    // sm_scale * log2(e)
    float qpscale;   // sm_scale * corr_scale * log2(e) * 16
    float log2_thresh;
    int Hq, Hkv, G, ngroups;
    int sub_shift;           // log2(block_size / 16)
    int64_t block_stride;    // bytes between consecutive blocks of the cache
    int chunk_pages, max_chunks;
    int max_pages;           // pages per sequence the block table and the workspace were sized for
    int io_dtype;
    int share_tables;        // K and V use the same codebook: one pair table serves both
    int rotate_q;            // the query is in original space: rotate it (fast WHT) while loading
    int derotate_out;        // write the output in original space
    int use_tcgen05;         // TQ_IO_TCGEN05 was given
};

// ---------------------------------------------------------------------------------
// Pair lookup table in shared memory.  After masking, every byte of an index word holds the
// indices of two neighbouring dims of one token in its two nibbles; that byte addresses a table
// of half2(c[i0], c[i1]) which is replicated per lane (entry stride 128 bytes, lane l reads
// word l of an entry) so that a warp's 32 lookups never collide on a bank.  One byte-extract
// (ALU), one multiply-add for the address (FMA pipe) and one shared load replace the two table
// permutes and the interleave permute of the register-only path: the logic pipe is the
// bottleneck of this kernel, the load/store pipe is not.
// ---------------------------------------------------------------------------------
// 2-bit indices: a whole byte of a packed word (four indices = two pairs: bits 1:0 with 5:4, bits 3:2 with 7:6)
// addresses a table of two half2, so one look-up serves four elements; an entry holds 16 copies of its 8 bytes (a 64-bit
// load is served half a warp at a time, lanes l and l + 16 never meet).
template <int BITS>
__host__ __device__ constexpr int lut_entries() { return BITS == 2 ? 256 : (BITS == 3 ? 128 : 256); }
template <int BITS>
__host__ __device__ constexpr int lut_bytes() { return lut_entries<BITS>() * 128; }

// Every lane fetches one centroid (already rounded to fp16) and the entries are assembled from warp shuffles, so the
// fill does not wait on a global load per entry.
template <int BITS>
__device__ __forceinline__ void fill_pair_lut(uint32_t* tab, const float* __restrict__ c, int warp, int lane) {
    const float cv = __half2float(__float2half_rn(__ldg(c + (lane & ((1 << BITS) - 1)))));
    if constexpr (BITS == 2) {
        for (int b = warp; b < 256; b += kWarps) {
            const int i0 = (lane & 1) ? (b >> 2) & 3 : b & 3, i1 = (lane & 1) ? (b >> 6) & 3 : (b >> 4) & 3;   // word 0: pair A, word 1: pair B
            tab[b * 32 + lane] = pack_half2(__shfl_sync(0xffffffffu, cv, i0), __shfl_sync(0xffffffffu, cv, i1));
        }
        return;
    }
    for (int b = warp; b < lut_entries<BITS>(); b += kWarps) {
        const int i0 = b & 15, i1 = b >> 4;
        const float c0 = __shfl_sync(0xffffffffu, cv, i0 & ((1 << BITS) - 1)), c1 = __shfl_sync(0xffffffffu, cv, i1 & ((1 << BITS) - 1));
        if (i0 < (1 << BITS) && i1 < (1 << BITS)) tab[b * 32 + lane] = pack_half2(c0, c1);
    }
}

// Words whose bytes are pair indices; word order matches the 8 groups of 4 elements (2 bytes each).
template <int BITS>
__device__ __forceinline__ void masked_words(const uint32_t (&w)[BITS], uint32_t (&mw)[4]) {
    if constexpr (BITS == 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) mw[j] = w[j];
    } else if constexpr (BITS == 3) {
#pragma unroll
        for (int j = 0; j < 3; ++j) mw[j] = w[j] & 0x77777777u;
        mw[3] = ((w[0] >> 3) & 0x11111111u) | ((w[1] >> 2) & 0x22222222u) | ((w[2] >> 1) & 0x44444444u);
    } else {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            mw[2 * j] = w[j] & 0x33333333u;
            mw[2 * j + 1] = (w[j] >> 2) & 0x33333333u;
        }
    }
}

// half2(c[i0], c[i1]) for byte k of a masked word; lane_base = shared address of the table + 4 * lane.
__device__ __forceinline__ uint32_t lut_pair(uint32_t lane_base, uint32_t mw, int k) {
    const uint32_t x = prmt(mw, 0u, 0x4440u | static_cast<uint32_t>(k));
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(lane_base + x * 128u));
    return v;
}

// 2-bit tables: (half2 of the pair in bits 1:0 / 5:4, half2 of the pair in bits 3:2 / 7:6) for byte k of a packed
// word; lane_base = shared address of the table + 8 * (lane & 15).
__device__ __forceinline__ uint2 lut_quad(uint32_t lane_base, uint32_t w, int k) {
    const uint32_t x = prmt(w, 0u, 0x4440u | static_cast<uint32_t>(k));
    uint2 v;
    asm("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(lane_base + x * 128u));
    return v;
}

// QJL sign term on fp16 tensor cores with one logic op per pair of signs.
//
// The sign word holds bit l = 1 when the residual of local dim l is >= 0.  A register of the
// A fragment is a pair of dims (j, j + 16), i.e. bits j and j + 16.  After x = sw << k the pair
// whose bits landed on 15/31 is turned into +-1 by one and-or; the pairs on bits 14/30, 13/29
// and 12/28 are used as they are: a lone exponent bit of an fp16 number is the value 2, 2^-7 or
// 2^-11.  Those three forms give (value) * [sign >= 0] instead of +-1; since
// 2 * [s >= 0] = sigma + 1, the query operand of those slots is pre-scaled (1, 2^8, 2^12) and
// the constant sum of the query over those dims is subtracted once (accumulator start value).
// Form 0 yields -sigma, so its query operand is negated.  All query operands carry 1/16 to keep
// 2^12 * q inside fp16; the factor 16 is folded into the fp32 scale of the residual norm.
// This lane's 32 query values (dims 32 * tig .. 32 * tig + 31 of query row gid) as fp32; zeros when !valid.
__device__ __forceinline__ void load_q32(const void* q, int64_t row_off, int tig, int io_dtype, bool valid, float (&x)[32]) {
    if (!valid) {
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = 0.f;
        return;
    }
    const uint16_t* base = static_cast<const uint16_t*>(q) + row_off + tig * 32;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(base) + i);
        const uint32_t r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (io_dtype == TQ_DTYPE_F16) {
                const float2 t = unpack_half2(r[j]);
                x[8 * i + 2 * j] = t.x;
                x[8 * i + 2 * j + 1] = t.y;
            } else {
                x[8 * i + 2 * j] = __uint_as_float(r[j] << 16);
                x[8 * i + 2 * j + 1] = __uint_as_float(r[j] & 0xffff0000u);
            }
        }
    }
}

// q' = q H for the query row spread over the 4 lanes of a tig group, rounded to the io dtype exactly as
// a separate rotation pass writing fp16 / bf16 would.
__device__ __forceinline__ void rotate_q32(float (&x)[32], int lane, int io_dtype) {
    fwht128(x, lane);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const float v = x[i] * kWhtScale;
        x[i] = io_dtype == TQ_DTYPE_F16 ? __half2float(__float2half_rn(v)) : __bfloat162float(__float2bfloat16_rn(v));
    }
}

__device__ __forceinline__ void q_frag_from(const float (&x)[32], uint32_t (&f)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = pack_half2(x[2 * i], x[2 * i + 1]);
}

// Query operands of the sign term (see above): per MMA m and slot, half2 of dims (j, j + 16) times the
// coefficient of the form; `correction` returns this lane's share of the query sum over the one-sided forms.
__device__ __forceinline__ void qp_frag_signed_from(const float (&x)[32], uint32_t (&f)[16], float& correction) {
    correction = 0.f;
    const float coef[4] = {-1.f / 16.f, 1.f / 16.f, 16.f, 256.f};   // form 0..3, times the common 1/16
#pragma unroll
    for (int m = 0; m < 8; ++m) {
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
            const int form = 2 * (m & 1) + sl, k = 4 * (m >> 1), j = 15 - form - k;
            f[2 * m + sl] = pack_half2(coef[form] * x[j], coef[form] * x[j + 16]);
            if (form) correction += (x[j] + x[j + 16]) * (1.f / 16.f);
        }
    }
}

// Shared-memory loads by 32-bit shared address + compile-time offset (one add per page and access pattern instead
// of 64-bit generic pointer arithmetic per load).
template <int OFF>
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}

template <int NW, int OFF>
__device__ __forceinline__ void lds_words(uint32_t addr, uint32_t (&w)[NW]) {
    if constexpr (NW == 4) {
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr), "n"(OFF));
    } else if constexpr (NW == 2) {
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(w[0]), "=r"(w[1]) : "r"(addr), "n"(OFF));
    } else {
        w[0] = lds_u32<OFF>(addr);
        if constexpr (NW > 1) w[1] = lds_u32<OFF + 4>(addr);
        if constexpr (NW > 2) w[2] = lds_u32<OFF + 8>(addr);
        if constexpr (NW > 3) w[3] = lds_u32<OFF + 12>(addr);
        if constexpr (NW > 4) w[4] = lds_u32<OFF + 16>(addr);
        static_assert(NW <= 5, "record has at most 4 index words and a sign word");
    }
}

// Output de-rotation inside a block: 128 threads hold one value each (thread = dim); returns (v H)[dim].
// Five butterfly stages by warp shuffle, two through shared memory (buf: 128 floats).
__device__ __forceinline__ float block_wht128(float v, float* buf, int tid) {
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, v, m);
        v = (tid & m) ? o - v : v + o;
    }
#pragma unroll
    for (int m = 32; m < 128; m <<= 1) {
        buf[tid] = v;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const float o = buf[tid ^ m];
        v = (tid & m) ? o - v : v + o;
        asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    return v * kWhtScale;
}

template <int KB, int VB, bool QJL, bool SPARSE, int NSTAGE>
__global__ void __launch_bounds__(kThreads, TQ_DEC_MINBLOCKS) decode_partial_kernel(const DecodeParams p) {
    constexpr int NWK = KB + (QJL ? 1 : 0);
    constexpr int RK = 16 * NWK;
    constexpr int KN_OFF = 16 * RK;
    constexpr int KRN_OFF = KN_OFF + 32;
    constexpr int KPART = KN_OFF + 32 + (QJL ? 32 : 0);
    constexpr int VN_OFF = KPART + 256 * VB;
    constexpr int PAGE = KPART + 256 * VB + 32;

    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);                 // [kWarps][2 * NSTAGE]
    uint32_t* tabk = reinterpret_cast<uint32_t*>(smem + kBarBytes);     // pair table of the K codebook
    uint32_t* tabv = p.share_tables ? tabk : tabk + lut_bytes<KB>() / 4;
    uint8_t* ring = smem + kBarBytes + lut_bytes<KB>() + (p.share_tables ? 0 : lut_bytes<VB>());  // [kWarps][NSTAGE][PAGE]
    float* sm_o = reinterpret_cast<float*>(ring);                       // reused after the page loop
    __shared__ float sm_m[kWarps][8];
    __shared__ float sm_l[kWarps][8];
    __shared__ float sm_wht[kHeadDim];

    pdl_release_and_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int chunk = blockIdx.x;
    const int kvh = blockIdx.y / p.ngroups, qg = blockIdx.y % p.ngroups;
    const int seq = blockIdx.z;
    const int L = p.seq_lens[seq];
    // A length beyond what the block table and the workspace were sized for is cut to that size and flagged:
    // the walk never leaves the table row and a chunk index never leaves the workspace.
    const bool too_long = L > p.max_pages * kPageTokens;
    const int npages = too_long ? p.max_pages : (L + kPageTokens - 1) / kPageTokens;
    const int g_in_group = qg * 8 + gid;                // query index inside the GQA group
    const int nq = min(8, p.G - qg * 8);                // live query heads in this CTA
    const int head0 = kvh * p.G + qg * 8;

    if (L <= 0) {
        if (chunk == 0) {  // zeros for empty sequences
            for (int i = threadIdx.x; i < nq * kHeadDim; i += kThreads) {
                const int64_t o = (static_cast<int64_t>(seq) * p.Hq + head0 + i / kHeadDim) * kHeadDim + i % kHeadDim;
                static_cast<uint16_t*>(p.out)[o] = 0;
            }
        }
        return;
    }
    const int p0 = chunk * p.chunk_pages;
    if (p0 >= npages) return;
    const int p1 = min(p0 + p.chunk_pages, npages);
    const int n_my = (p0 + warp < p1) ? (p1 - p0 - warp + kWarps - 1) / kWarps : 0;

    uint64_t* mybar = bars + warp * 2 * NSTAGE;        // [0..NSTAGE) K (or whole page), [NSTAGE..) V
    uint8_t* myring = ring + warp * NSTAGE * PAGE;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < 2 * NSTAGE; ++s) mbar_init(mybar + s, 1);
        fence_barrier_init();
    }
    __syncwarp();

    // ---- block-table window: lane l holds the entry of this warp's page jbase + l ---
    const int32_t* bt = p.block_tables + static_cast<int64_t>(seq) * p.bt_stride;
    int jbase = 0;
    int32_t btreg = 0;
    bool bad_block = false;
    auto load_bt = [&](int jb) {
        jbase = jb;
        const int j = jb + lane;
        int32_t b = 0;
        if (j < n_my) {
            b = __ldg(bt + ((p0 + warp + kWarps * j) >> p.sub_shift));
            if (b < 0 || b >= p.num_blocks) {
                bad_block = true;
                b = 0;
            }
        }
        btreg = b;
    };
    const uint8_t* head_base = p.cache + (static_cast<int64_t>(kvh) << p.sub_shift) * PAGE;
    auto page_src = [&](int j) -> const uint8_t* {
        const int32_t blk = __shfl_sync(0xffffffffu, btreg, j - jbase);
        const int pg = p0 + warp + kWarps * j;
        const int sub = pg & ((1 << p.sub_shift) - 1);
        return head_base + static_cast<int64_t>(blk) * p.block_stride + sub * PAGE;
    };
    // Dense mode: one copy of the whole page.  Sparse mode: K part now, V part on demand.
    // whole = K and V parts in one copy (always in dense mode; in sparse mode when the V part is expected to be needed)
    auto issue_k = [&](int j, bool whole = true) {
        const uint8_t* src = page_src(j);
        const int s = j % NSTAGE;
        if (lane == 0) {
            const uint32_t bytes = (SPARSE && !whole) ? KPART : PAGE;
            mbar_expect_tx(mybar + s, bytes);
            bulk_g2s(myring + s * PAGE, src, bytes, mybar + s);
        }
    };
    auto issue_v = [&](int j) {
        const uint8_t* src = page_src(j);
        const int s = j % NSTAGE;
        if (lane == 0) {
            mbar_expect_tx(mybar + NSTAGE + s, PAGE - KPART);
            bulk_g2s(myring + s * PAGE + KPART, src + KPART, PAGE - KPART, mybar + NSTAGE + s);
        }
    };

    // The first pages are requested before anything else is set up: their HBM latency hides behind the
    // table fill and the query fragments.
    if (n_my > 0) load_bt(0);
#pragma unroll
    for (int j = 0; j < NSTAGE; ++j)
        if (j < n_my) issue_k(j);

    // ---- query fragments (their loads are in flight together with the first pages and the table fill) -----
    uint32_t qf[16], qpf[QJL ? 16 : 1];
    float sq_init0 = 0.f, sq_init1 = 0.f;   // minus the query sums of the one-sided sign forms
    {
        const bool valid = g_in_group < p.G;
        const int64_t row = (static_cast<int64_t>(seq) * p.Hq + head0 + gid) * kHeadDim;
        float xq[32];
        load_q32(p.q, row, tig, p.io_dtype, valid, xq);
        if (p.rotate_q) rotate_q32(xq, lane, p.io_dtype);
        q_frag_from(xq, qf);
        if constexpr (QJL) {
            if (p.qp) load_q32(p.qp, row, tig, p.io_dtype, valid, xq);   // S q' given separately
            float corr;
            qp_frag_signed_from(xq, qpf, corr);
            corr += __shfl_xor_sync(0xffffffffu, corr, 1);
            corr += __shfl_xor_sync(0xffffffffu, corr, 2);      // total over the 128 dims of query gid
            sq_init0 = -__shfl_sync(0xffffffffu, corr, 8 * tig);       // query 2 * tig lives on lanes 8 * tig ..
            sq_init1 = -__shfl_sync(0xffffffffu, corr, 8 * tig + 4);   // query 2 * tig + 1
        }
    }

    // ---- per-CTA constants: pair tables of the codebooks ----------------------------------------------
    fill_pair_lut<KB>(tabk, p.kc, warp, lane);
    if (!p.share_tables) fill_pair_lut<VB>(tabv, p.vc, warp, lane);
    __syncthreads();
    const uint32_t klut = smem_u32(tabk) + (KB == 2 ? 8 * (lane & 15) : 4 * lane);
    const uint32_t vlut = smem_u32(tabv) + (VB == 2 ? 8 * (lane & 15) : 4 * lane);
    // this lane's three access patterns inside a ring stage: its two K records, the norm slots, the V words
    const uint32_t ring_k = smem_u32(myring) + lane * (NWK * 4);
    const uint32_t ring_n = smem_u32(myring) + gid * 4;
    const uint32_t ring_v = smem_u32(myring) + (tig * 8 + gid) * 4;
    // ---- online-softmax state ---------------------------------------------------------
    float m0 = -INFINITY, m1 = -INFINITY;   // running max for queries 2*tig, 2*tig+1 (log2 domain)
    float l0 = 0.f, l1 = 0.f;               // this lane's share of the denominators
    float oacc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int r = 0; r < 4; ++r) oacc[i][r] = 0.f;
    bool timed_out = false;
    uint32_t v_skipped = 0;
    uint32_t v_parity = 0;                  // bit s: phase of the V barrier of stage s (sparse mode)
    int j_stop = n_my;
    uint32_t v_with_k = (1u << NSTAGE) - 1u;  // sparse mode, bit s: the page in stage s brought its V part along (the first pages do)

    auto wait_v = [&](int j) -> bool {
        const int s = j % NSTAGE;
        const bool ok = mbar_wait_bounded(mybar + NSTAGE + s, (v_parity >> s) & 1u);
        v_parity ^= 1u << s;
        return ok;
    };
    // O += P V for page j (already resident in its ring stage); weights are relative to the running maximum.
    auto accumulate_v = [&](int j, float w0, float w1, float w2, float w3, int valid_tokens) {
        const uint32_t stage = (j % NSTAGE) * PAGE;
        const bool va = gid < valid_tokens, vb = gid + 8 < valid_tokens;
        const float2 vn = unpack_half2(lds_u32<VN_OFF>(ring_n + stage));
        const uint32_t vaddr = ring_v + stage;
        const uint32_t pr0 = pack_half2(va ? w0 * vn.x : 0.f, va ? w1 * vn.x : 0.f);
        const uint32_t pr1 = pack_half2(vb ? w2 * vn.y : 0.f, vb ? w3 * vn.y : 0.f);
        const uint32_t t[2] = {movmatrix_trans(pr0), movmatrix_trans(pr1)};
#pragma unroll
        for (int o = 0; o < 2; ++o) {
            const uint32_t vo = vaddr + o * 128;
            const uint32_t pa0 = t[o] & 0xffffu, pa1 = t[o] << 16, pa2 = t[o] >> 16, pa3 = t[o] & 0xffff0000u;
            uint32_t pw[VB];
#pragma unroll
            for (int i = 0; i < VB; ++i)
                pw[i] = i == 0 ? lds_u32<KPART>(vo) : (i == 1 ? lds_u32<KPART + 256>(vo) : (i == 2 ? lds_u32<KPART + 512>(vo) : lds_u32<KPART + 768>(vo)));
            if constexpr (VB == 2) {
                // byte k of packed word jw: the pairs of group u = 2 jw (first half2) and u = 2 jw + 1 (second)
#pragma unroll
                for (int jw = 0; jw < 2; ++jw) {
                    const uint2 a0 = lut_quad(vlut, pw[jw], 0), a1 = lut_quad(vlut, pw[jw], 1);
                    const uint2 b0 = lut_quad(vlut, pw[jw], 2), b1 = lut_quad(vlut, pw[jw], 3);
                    mma_f16_16816(oacc[4 * jw], pa0, pa1, pa2, pa3, a0.x, b0.x);
                    mma_f16_16816(oacc[4 * jw + 1], pa0, pa1, pa2, pa3, a1.x, b1.x);
                    mma_f16_16816(oacc[4 * jw + 2], pa0, pa1, pa2, pa3, a0.y, b0.y);
                    mma_f16_16816(oacc[4 * jw + 3], pa0, pa1, pa2, pa3, a1.y, b1.y);
                }
            } else {
                uint32_t mv[4];
                masked_words<VB>(pw, mv);   // bytes 0,1: token a (dims 4u..4u+3), bytes 2,3: token b
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t a0 = lut_pair(vlut, mv[u], 0), a1 = lut_pair(vlut, mv[u], 1);
                    const uint32_t b0 = lut_pair(vlut, mv[u], 2), b1 = lut_pair(vlut, mv[u], 3);
                    mma_f16_16816(oacc[2 * u], pa0, pa1, pa2, pa3, a0, b0);
                    mma_f16_16816(oacc[2 * u + 1], pa0, pa1, pa2, pa3, a1, b1);
                }
            }
        }
    };

    for (int j = 0; j < n_my; ++j) {
        if constexpr (SPARSE) {
            if ((v_with_k >> (j % NSTAGE)) & 1u) {
#define TQ_PAGE_HAVE_V 1
#include "tq_decode_page.inc"
#undef TQ_PAGE_HAVE_V
            } else {
#define TQ_PAGE_HAVE_V 0
#include "tq_decode_page.inc"
#undef TQ_PAGE_HAVE_V
            }
        } else {
#define TQ_PAGE_HAVE_V 1
#include "tq_decode_page.inc"
#undef TQ_PAGE_HAVE_V
        }
    }
    if (timed_out) {
        // Give copies that were already issued a bounded chance to land before the ring is reused.
        for (int j = j_stop + 1; j < min(n_my, j_stop + NSTAGE); ++j)
            (void)mbar_wait_bounded(mybar + j % NSTAGE, (j / NSTAGE) & 1);
    }

    if (p.status) {
        int bits = 0;
        if (__any_sync(0xffffffffu, bad_block) || too_long) bits |= TQ_STATUS_BAD_BLOCK;
        if (__any_sync(0xffffffffu, timed_out)) bits |= TQ_STATUS_TIMEOUT;
        if (bits && lane == 0) atomicOr(p.status, bits);
    }
    if constexpr (SPARSE) {
        if (p.skip_stats && lane == 0) {
            atomicAdd(p.skip_stats, static_cast<uint32_t>(j_stop));   // pages this warp visited
            atomicAdd(p.skip_stats + 1, v_skipped);
        }
    }

    // ---- merge the 4 warps --------------------------------------------------------------
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }
    __syncthreads();  // every warp is done with its ring; it becomes the merge buffer
    if (gid == 0) {
        sm_m[warp][2 * tig] = m0;
        sm_m[warp][2 * tig + 1] = m1;
        sm_l[warp][2 * tig] = l0;
        sm_l[warp][2 * tig + 1] = l1;
    }
    {
        float* row = sm_o + (warp * 8 + gid) * kOPad;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int dim = 16 * (2 * tig + (r & 1)) + 2 * nt + (r >> 1);
                row[dim + (dim >> 5)] = oacc[nt][r];
            }
    }
    __syncthreads();
    const int dim = threadIdx.x;
    const int col = dim + (dim >> 5);
    const int nchunks = (npages + p.chunk_pages - 1) / p.chunk_pages;
    for (int g = 0; g < (dim < kHeadDim ? nq : 0); ++g) {
        float M = sm_m[0][g];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) M = fmaxf(M, sm_m[w][g]);
        float o = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float sc = ex2(sm_m[w][g] - M);
            o = fmaf(sc, sm_o[(w * 8 + g) * kOPad + col], o);
            l = fmaf(sc, sm_l[w][g], l);
        }
        if (nchunks == 1) {
            float r = o / l;
            if (p.derotate_out) r = block_wht128(r, sm_wht, dim);
            const int64_t off = (static_cast<int64_t>(seq) * p.Hq + head0 + g) * kHeadDim + dim;
            if (p.io_dtype == TQ_DTYPE_F16)
                static_cast<__half*>(p.out)[off] = __float2half_rn(r);
            else
                static_cast<__nv_bfloat16*>(p.out)[off] = __float2bfloat16_rn(r);
        } else {
            const int64_t slot = ((static_cast<int64_t>(seq) * p.Hkv * p.ngroups + blockIdx.y) * p.max_chunks + chunk) * 8 + g;
            p.ws_o[slot * kHeadDim + dim] = o;
            if (dim == 0) {
                p.ws_ml[slot * 2] = M;
                p.ws_ml[slot * 2 + 1] = l;
            }
        }
    }
}

__global__ void __launch_bounds__(kHeadDim) decode_merge_kernel(const DecodeParams p) {
    pdl_release_and_wait();
    const int head = blockIdx.x, seq = blockIdx.y, dim = threadIdx.x;
    const int L = p.seq_lens[seq];
    const int npages = min((L + kPageTokens - 1) / kPageTokens, p.max_pages);   // same cut as the partial kernel
    const int nchunks = (npages + p.chunk_pages - 1) / p.chunk_pages;
    if (nchunks <= 1) return;  // written by the partial kernel
    const int kvh = head / p.G, gi = head % p.G;
    const int by = kvh * p.ngroups + gi / 8, g = gi % 8;
    const int64_t base = (static_cast<int64_t>(seq) * p.Hkv * p.ngroups + by) * p.max_chunks;
    float M = -INFINITY;
    for (int c = 0; c < nchunks; ++c) M = fmaxf(M, p.ws_ml[((base + c) * 8 + g) * 2]);
    float o = 0.f, l = 0.f;
    for (int c = 0; c < nchunks; ++c) {
        const int64_t slot = (base + c) * 8 + g;
        const float sc = ex2(p.ws_ml[slot * 2] - M);
        o = fmaf(sc, p.ws_o[slot * kHeadDim + dim], o);
        l = fmaf(sc, p.ws_ml[slot * 2 + 1], l);
    }
    float r = o / l;
    if (p.derotate_out) {
        __shared__ float buf[kHeadDim];
        r = block_wht128(r, buf, dim);
    }
    const int64_t off = (static_cast<int64_t>(seq) * p.Hq + head) * kHeadDim + dim;
    if (p.io_dtype == TQ_DTYPE_F16)
        static_cast<__half*>(p.out)[off] = __float2half_rn(r);
    else
        static_cast<__nv_bfloat16*>(p.out)[off] = __float2bfloat16_rn(r);
}

template <int KB, int VB, bool QJL, bool SPARSE>
int launch_partial(const DecodeParams& p, dim3 grid, cudaStream_t stream) {
    constexpr int PAGE = page_bytes(KB, VB, QJL ? 1 : 0);
    constexpr size_t smem_max = kBarBytes + lut_bytes<KB>() + lut_bytes<VB>() + static_cast<size_t>(kWarps) * kStages * PAGE;
    const size_t smem = smem_max - (p.share_tables ? lut_bytes<VB>() : 0);
    static_assert(static_cast<size_t>(kWarps) * kStages * PAGE >= sizeof(float) * kWarps * 8 * kOPad,
                  "ring must hold the merge buffer");
    auto kern = decode_partial_kernel<KB, VB, QJL, SPARSE, kStages>;
    // The opt-in shared-memory size is a per-device function attribute; set once per device.
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TQ_ERR_LAUNCH;
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_max)) != cudaSuccess)
            return TQ_ERR_LAUNCH;
        configured[dev] = true;
    }
    return launch_chained(kern, grid, dim3(kThreads), smem, stream, p) == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

}  // namespace
}  // namespace tq

#include "tq_decode_umma.cuh"

namespace tq {
namespace {

template <int KB, int VB>
int dispatch_flags(const DecodeParams& p, bool qjl, bool sparse, dim3 grid, cudaStream_t stream) {
    if constexpr (KB <= 3 && VB <= 3) {
        // on request (TQ_IO_TCGEN05): the tensor-memory kernel, for 2- and 3-bit codebooks without the Sparse-V skip
        if (!sparse && p.use_tcgen05) return qjl ? launch_umma<KB, VB, true>(p, grid, stream) : launch_umma<KB, VB, false>(p, grid, stream);
    }
    if (qjl) return sparse ? launch_partial<KB, VB, true, true>(p, grid, stream) : launch_partial<KB, VB, true, false>(p, grid, stream);
    return sparse ? launch_partial<KB, VB, false, true>(p, grid, stream) : launch_partial<KB, VB, false, false>(p, grid, stream);
}

template <int KB>
int dispatch_v(const DecodeParams& p, int vb, bool qjl, bool sparse, dim3 grid, cudaStream_t stream) {
    switch (vb) {
#ifndef TQ_DEC_QUICK
        case 2: return dispatch_flags<KB, 2>(p, qjl, sparse, grid, stream);
        case 4: return dispatch_flags<KB, 4>(p, qjl, sparse, grid, stream);
#endif
        case 3: return dispatch_flags<KB, 3>(p, qjl, sparse, grid, stream);
    }
    return TQ_ERR_UNSUPPORTED;
}

}  // namespace
}  // namespace tq

using namespace tq;

extern "C" int tq_decode_auto_chunk_pages(int num_seqs, int num_kv_heads, int num_q_heads, int max_pages_per_seq) {
    if (num_seqs <= 0 || num_kv_heads <= 0 || num_q_heads <= 0 || max_pages_per_seq <= 0) return TQ_ERR_ARG;
    if (num_q_heads % num_kv_heads) return TQ_ERR_ARG;   // also num_q_heads < num_kv_heads: no query group
    // Sizes come from the longest sequence; chunks beyond a shorter sequence's end exit at once.
    // Measured on batch 64 x 8192 tokens with 1, 2, 4 and 8 KV heads per GPU (chunk sizes 32..512 pages):
    //  * about 1024 CTAs (1.7 waves of 148 SMs x 4 CTAs) is the flat optimum, with a power-of-two number
    //    of chunks so that all chunks of a sequence are alike (64-page chunks for 1-2 heads, 128 for 4,
    //    128..256 for 8); uneven splits such as 57 or 74 pages lose 5-10 %;
    //  * a CTA keeps >= 64 pages (16 per warp) so that its prologue (lookup-table fill, query fragments,
    //    first copies) stays amortised, unless that leaves the GPU less than half full (small batches):
    //    then chunks shrink down to 16 pages (see below);
    //  * at most 256 pages per CTA bound the longest CTA when sequence lengths are skewed.
    const int G = num_q_heads / num_kv_heads;
    const int ngroups = (G + 7) / 8;
    const long long pairs = 1LL * num_seqs * num_kv_heads * ngroups;
    const long long slots = 148LL * 4;
    auto ceil_div = [](long long a, long long b) { return (a + b - 1) / b; };
    long long chunks = 1;
    while (pairs * chunks * 2 <= 1024 + pairs * chunks / 2) chunks *= 2;   // power of two nearest to 1024 / pairs
    long long max_big = max_pages_per_seq / 64;
    if (max_big < 1) max_big = 1;
    while (chunks > max_big) chunks /= 2;
    if (chunks < 1) chunks = 1;
    if (pairs * chunks < slots / 2) {
        // Small batches: the smallest power-of-two chunk (>= 16 pages) that keeps the grid within the resident slots.
        // Measured on 1, 2 and 4 sequences of 32768, 16384 and 8192 tokens (8 KV heads): 32-page chunks (512 CTAs)
        // 32.8 / 27.8 / 25.3 us against 35.2 / 32.0 / 30.0 us for the 27-28 pages that fill every slot: the warps of a
        // CTA share a chunk evenly only when it is a multiple of 4 pages, and every extra CTA pays its set-up.
        long long most = slots / pairs;
        if (most < 1) most = 1;
        long long cp = 16;
        while (cp < ceil_div(max_pages_per_seq, most)) cp *= 2;
        if (cp > max_pages_per_seq) cp = max_pages_per_seq;
        return static_cast<int>(cp > 256 ? 256 : cp);
    }
    // Fewer CTAs than resident slots (a GPU that holds one or two KV heads of a sharded batch): an uneven chunk count
    // that fills the slots beats the power of two (64 sequence-heads: 9 chunks of 57 pages = 576 CTAs measured 37.7 us
    // against 39.5 us for 8 x 64), as long as chunks stay >= 32 pages.
    if (pairs * chunks <= slots) {
        const long long fill = slots / pairs;
        if (fill > chunks && max_pages_per_seq / fill >= 32) chunks = fill;
    }
    long long cp = ceil_div(max_pages_per_seq, chunks);
    if (cp > 256) cp = 256;
    return static_cast<int>(cp);
}

extern "C" int64_t tq_decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads, int max_pages_per_seq,
                                             int chunk_pages) {
    if (num_seqs <= 0 || num_kv_heads <= 0 || num_q_heads <= 0 || max_pages_per_seq <= 0) return TQ_ERR_ARG;
    if (num_q_heads % num_kv_heads) return TQ_ERR_ARG;
    if (chunk_pages <= 0) chunk_pages = tq_decode_auto_chunk_pages(num_seqs, num_kv_heads, num_q_heads, max_pages_per_seq);
    const int G = num_q_heads / num_kv_heads;
    const int ngroups = (G + 7) / 8;
    const int64_t max_chunks = (max_pages_per_seq + chunk_pages - 1) / chunk_pages;
    const int64_t slots = static_cast<int64_t>(num_seqs) * num_kv_heads * ngroups * max_chunks * 8;
    return slots * (kHeadDim + 2) * static_cast<int64_t>(sizeof(float));
}

extern "C" int tq_decode_paged(void* out, const void* q_rot, const void* q_proj, int io_dtype, const void* cache,
                               int64_t num_blocks, int block_size, const int32_t* block_tables, int64_t bt_stride,
                               const int32_t* seq_lens, const float* k_centroids, const float* v_centroids,
                               float sm_scale, float corr_scale, float sparse_thresh, void* workspace,
                               int64_t workspace_bytes, int32_t* status, uint32_t* skip_stats, int num_seqs,
                               int num_q_heads, int num_kv_heads, int max_pages_per_seq, int k_bits, int v_bits,
                               int use_qjl, int chunk_pages, tq_stream_t stream) {
    if (num_seqs == 0) return TQ_OK;
    if (!out || !q_rot || !cache || !block_tables || !seq_lens || !k_centroids || !v_centroids) return TQ_ERR_ARG;
    if (num_seqs < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || max_pages_per_seq <= 0 || num_blocks <= 0) return TQ_ERR_ARG;
    if (num_q_heads % num_kv_heads) return TQ_ERR_ARG;
    const int rotate_q = (io_dtype & TQ_IO_ROTATE_Q) ? 1 : 0, derotate_out = (io_dtype & TQ_IO_DEROTATE_OUT) ? 1 : 0;
    const int use_tcgen05 = (io_dtype & TQ_IO_TCGEN05) ? 1 : 0;
    io_dtype &= 0xff;
    if (io_dtype != TQ_DTYPE_F16 && io_dtype != TQ_DTYPE_BF16) return TQ_ERR_UNSUPPORTED;
    if (rotate_q && q_proj) return TQ_ERR_ARG;   // S q' cannot be derived from an unrotated query
    if (block_size < kPageTokens || (block_size & (block_size - 1))) return TQ_ERR_UNSUPPORTED;  // 16, 32, 64, ...
    if (k_bits < 2 || k_bits > 4 || v_bits < 2 || v_bits > 4) return TQ_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(q_rot) | reinterpret_cast<uintptr_t>(out) |
         reinterpret_cast<uintptr_t>(q_proj)) & 15)
        return TQ_ERR_ARG;
    if (chunk_pages <= 0) chunk_pages = tq_decode_auto_chunk_pages(num_seqs, num_kv_heads, num_q_heads, max_pages_per_seq);
    const int64_t need = tq_decode_workspace_bytes(num_seqs, num_q_heads, num_kv_heads, max_pages_per_seq, chunk_pages);
    const int max_chunks = (max_pages_per_seq + chunk_pages - 1) / chunk_pages;
    if (max_chunks > 1 && (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)))
        return TQ_ERR_WORKSPACE;
    if (num_seqs > 65535 || max_chunks > 65535) return TQ_ERR_UNSUPPORTED;

    DecodeParams p;
    p.out = out;
    p.q = q_rot;
    p.qp = q_proj;
    p.cache = static_cast<const uint8_t*>(cache);
    p.block_tables = block_tables;
    p.seq_lens = seq_lens;
    p.kc = k_centroids;
    p.vc = v_centroids;
    p.G = num_q_heads / num_kv_heads;
    p.ngroups = (p.G + 7) / 8;
    const int64_t slots = static_cast<int64_t>(num_seqs) * num_kv_heads * p.ngroups * max_chunks * 8;
    p.ws_o = static_cast<float*>(workspace);
    p.ws_ml = p.ws_o ? p.ws_o + slots * kHeadDim : nullptr;
    p.status = status;
    p.skip_stats = skip_stats;
    p.bt_stride = bt_stride;
    p.num_blocks = num_blocks;
    p.qscale = sm_scale * kLog2e;
    p.qpscale = sm_scale * corr_scale * kLog2e * 16.f;   // the sign-term query operands carry 1/16
    p.log2_thresh = sparse_thresh > 0.f ? log2f(sparse_thresh) : -INFINITY;
    p.Hq = num_q_heads;
    p.Hkv = num_kv_heads;
    p.sub_shift = 0;
    while ((kPageTokens << p.sub_shift) < block_size) ++p.sub_shift;
    p.block_stride = static_cast<int64_t>(num_kv_heads) * (block_size / kPageTokens) *
                     page_bytes(k_bits, v_bits, use_qjl ? 1 : 0);
    p.chunk_pages = chunk_pages;
    p.max_chunks = max_chunks;
    p.max_pages = max_pages_per_seq;
    p.io_dtype = io_dtype;
    p.rotate_q = rotate_q;
    p.derotate_out = derotate_out;
    p.use_tcgen05 = use_tcgen05;
    p.share_tables = (k_bits == v_bits && k_centroids == v_centroids) ? 1 : 0;

    const dim3 grid(max_chunks, num_kv_heads * p.ngroups, num_seqs);
    const bool qjl = use_qjl != 0, sparse = sparse_thresh > 0.f;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int rc;
    switch (k_bits) {
#ifndef TQ_DEC_QUICK
        case 2: rc = dispatch_v<2>(p, v_bits, qjl, sparse, grid, st); break;
        case 4: rc = dispatch_v<4>(p, v_bits, qjl, sparse, grid, st); break;
#endif
        case 3: rc = dispatch_v<3>(p, v_bits, qjl, sparse, grid, st); break;
        default: return TQ_ERR_UNSUPPORTED;
    }
    if (rc != TQ_OK) return rc;
    if (max_chunks > 1) {
        if (launch_chained(decode_merge_kernel, dim3(num_q_heads, num_seqs), dim3(kHeadDim), 0, st, p) != cudaSuccess)
            return TQ_ERR_LAUNCH;
    }
    return TQ_OK;
}

// ---------------------------------------------------------------------------------------------
// Decode without a caller-provided workspace.
//
// Some hosts of this library have no way to obtain device memory of their own: an inference
// server that hands every free byte of HBM to its KV-cache pool at start-up (a later cudaMalloc
// simply fails), or a binding in a runtime that only forwards pointers it was given and owns no
// device allocator.  For them the split-K scratch lives in a fixed array inside the library image,
// reserved on every GPU that loads the library for as long as the process runs.
// ---------------------------------------------------------------------------------------------
namespace tq {
namespace {

constexpr size_t kStaticScratchBytes = TQ_DECODE_STATIC_SCRATCH_BYTES;   // 16 MiB, the stated limit
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

// In host code `g_decode_scratch` is only a handle for the runtime, not a device address: the
// address a kernel may use comes from cudaGetSymbolAddress, asked once per device.
void* static_scratch_address(int* status) {
    static void* cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        *status = TQ_ERR_LAUNCH;
        return nullptr;
    }
    if (!cached[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_decode_scratch) != cudaSuccess || !ptr) {
            *status = TQ_ERR_LAUNCH;
            return nullptr;
        }
        cached[dev] = ptr;
    }
    *status = TQ_OK;
    return cached[dev];
}

}  // namespace
}  // namespace tq

extern "C" int tq_decode_paged_static(void* out, const void* q_rot, const void* q_proj, int io_dtype, const void* cache,
                                      int64_t num_blocks, int block_size, const int32_t* block_tables,
                                      int64_t bt_stride, const int32_t* seq_lens, const float* k_centroids,
                                      const float* v_centroids, float sm_scale, float corr_scale, float sparse_thresh,
                                      int32_t* status, uint32_t* skip_stats, int num_seqs, int num_q_heads,
                                      int num_kv_heads, int max_pages_per_seq, int k_bits, int v_bits, int use_qjl,
                                      int chunk_pages, tq_stream_t stream) {
    if (num_seqs == 0) return TQ_OK;
    if (num_seqs < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || max_pages_per_seq <= 0) return TQ_ERR_ARG;
    if (num_q_heads % num_kv_heads) return TQ_ERR_ARG;
    if (chunk_pages <= 0) chunk_pages = tq_decode_auto_chunk_pages(num_seqs, num_kv_heads, num_q_heads, max_pages_per_seq);
    // Refuse, before touching the GPU, any problem whose split-K partials do not fit the fixed array.
    const int64_t need = tq_decode_workspace_bytes(num_seqs, num_q_heads, num_kv_heads, max_pages_per_seq, chunk_pages);
    if (need < 0) return static_cast<int>(need);
    if (need > static_cast<int64_t>(tq::kStaticScratchBytes)) return TQ_ERR_WORKSPACE;
    int rc = TQ_OK;
    void* scratch = tq::static_scratch_address(&rc);
    if (rc != TQ_OK) return rc;
    // Nothing in the scratch has to start at zero: every partial a merge reads was written by the
    // partial kernel of the same call, so contents left by an earlier call are never observed.
    return tq_decode_paged(out, q_rot, q_proj, io_dtype, cache, num_blocks, block_size, block_tables, bt_stride,
                           seq_lens, k_centroids, v_centroids, sm_scale, corr_scale, sparse_thresh, scratch,
                           static_cast<int64_t>(tq::kStaticScratchBytes), status, skip_stats, num_seqs, num_q_heads,
                           num_kv_heads, max_pages_per_seq, k_bits, v_bits, use_qjl, chunk_pages, stream);
}
