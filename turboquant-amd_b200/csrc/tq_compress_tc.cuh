// Paged KV compression with the rotation on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
// Included by tq_compress.cu after tq_compress_fast.cuh (tables, quant_pair, assemble_indices and the page stores
// are shared).  fp16 / bf16 rows that still have to be rotated take this kernel when the launch is large.
//
// One CTA per SM, 16 warps = four autonomous groups of 128 threads; groups 0 and 2 compress the key rows, groups 1 and
// 3 the value rows, of alternating tiles of 128 (token, head) items.  A group works alone:
//   * its threads stage the tile's 128 rows (256 bytes each) into shared memory with 16-byte cp.async copies, placed
//     directly in the K-major operand layout of the tensor core (16-byte column chunk c of row r at c * 2048 + r * 16;
//     a warp instruction copies whole 32-byte sectors of 16 rows and writes two contiguous 256-byte runs);
//   * its first thread issues eight `tcgen05.mma kind::f16` (M = 128 rows, N = 128, K = 16 each) against the constant
//     +-1 Hadamard matrix held in shared memory in the input type: every product is exact, accumulation is fp32 in the
//     group's 128 columns of tensor memory;
//   * then one thread owns one vector: it reads its row of the unnormalised transform with `tcgen05.ld`, sums the squares
//     (the norm of the rotated vector, as the reference takes it), and runs the table-driven quantizer of the fast path
//     on its 128 values - no shuffles, no fragment bookkeeping, packing in registers, 16-byte stores.
// While a group quantizes, the copies of its next tile are in flight and the other three groups keep the SM busy.
//
// Arithmetic after the rotation is the fast path's (exact quotient, ties down, centroid picked exactly): on identical
// rotated values the indices, signs and norms are the oracle's.  The rotation is a different summation order than a
// butterfly or x @ H, as with any fast transform (the 1e-4 allowance of turboquant/core/quantizer.py:141-173 parity).
#pragma once

namespace tq {
namespace {

constexpr int kTcThreads = 512;
constexpr int kTcTile = 128;                       // rows (items) per tile
constexpr int kTcChunkStride = 2048 + 16;          // bytes between 16-byte column chunks of the staged tile: the extra 16
                                                   // bytes put the eight chunks of one 128-byte line on different banks
constexpr int kTcStageBytes = 16 * kTcChunkStride; // one tile of fp16 / bf16 rows
constexpr int kTcHBytes = 128 * 256;               // the 128 x 128 Hadamard matrix in the input type

struct TcSmem {
    static constexpr int kBars = 0;                // 4 mbarriers
    static constexpr int kTmemSlot = 64;
    static constexpr int kBad = 80;
    static constexpr int kTables = 128;            // K table, V table (kTableBytes each)
    static constexpr int kH = 128 + 2 * kTableBytes;
    static constexpr int kStage = kH + kTcHBytes;  // 4 groups x 32 KB
    static constexpr int kTotal = kStage + 4 * kTcStageBytes;
};
static_assert(TcSmem::kH % 128 == 0 && TcSmem::kTotal <= 227 * 1024, "shared memory map");

__device__ __forceinline__ void tc_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ bool tc_mbar_wait(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < (1 << 22); ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
// kind::f16 instruction descriptor: f32 accumulate, A and B of type fp16 (0) or bf16 (1), both K-major, M = N = 128
__host__ __device__ constexpr uint32_t tc_idesc(int bf16) {
    return (1u << 4) | (static_cast<uint32_t>(bf16) << 7) | (static_cast<uint32_t>(bf16) << 10) | (16u << 17) | (8u << 24);
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}

__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Half a quarter (16 dims = chunks 4 h .. 4 h + 3 of the quarter, as 8 pairs) through the table-driven quantizer:
// fills cv[4 h .. 4 h + 3] and the 16 sign bits sg (1 = negative; the upper half must be done first only in the sense
// that each half has its own accumulator); rr accumulates the squared residuals of the whole vector.
template <bool QJL>
__device__ __forceinline__ void quantize_half_fast(const uint32_t (&d)[16], const VecConsts& vc, f2& rr, float (&cv4)[4], uint32_t& sg) {
    sg = 0u;
#pragma unroll
    for (int c = 3; c >= 0; --c) {
        float k0, k1, k2, k3;
        quant_pair<QJL, false>(f2pack(__uint_as_float(d[4 * c + 2]), __uint_as_float(d[4 * c + 3])), vc, rr, sg, k2, k3);
        quant_pair<QJL, false>(f2pack(__uint_as_float(d[4 * c]), __uint_as_float(d[4 * c + 1])), vc, rr, sg, k0, k1);
        cv4[c] = fmaf(fmaf(fmaf(k3, 16.f, k2), 16.f, k1), 16.f, k0);
    }
}

template <int KB, int VB, bool QJL>
__global__ void __launch_bounds__(kTcThreads, 1) compress_paged_tc_kernel(const PagedParams p, int64_t n_tiles) {
    constexpr int PAGE = page_bytes(KB, VB, QJL ? 1 : 0);
    constexpr int KPART = k_part_bytes(KB, QJL ? 1 : 0);
    extern __shared__ __align__(128) unsigned char tsm[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(tsm + TcSmem::kBars);
    int* bad = reinterpret_cast<int*>(tsm + TcSmem::kBad);
    unsigned char* tables = tsm + TcSmem::kTables;
    const uint32_t sbase = smem_u32(tsm);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int group = warp >> 2, gw = warp & 3;            // group 0..3; warp within the group = tensor-memory lane quadrant
    const bool is_v = group & 1;
    const int row = gw * 32 + lane;                         // row of the group's tile = tensor-memory lane
    const bool bf16 = p.in_dtype == TQ_DTYPE_BF16;

    // ---- set-up ---------------------------------------------------------------------------------------------
    if (tid == 0) {
        *bad = 0;
        for (int g = 0; g < 4; ++g) tc_mbar_init(bars + g, 1);
        fence_barrier_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + TcSmem::kTmemSlot), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    __syncthreads();
    build_table<KB, QJL>(tables, p.kb, p.kc, bad);
    build_table<VB, false>(tables + kTableBytes, p.vb, nullptr, bad);
    {
        // Hadamard matrix, entry (n, k) = (-1)^popcount(n & k) as +-1.0 of the input type, in the K-major operand layout
        const uint32_t one = bf16 ? 0x3F80u : 0x3C00u;
        for (int i = tid; i < 128 * 16; i += kTcThreads) {
            const int n = i & 127, c = i >> 7;          // 16-byte chunk c holds k = 8 c .. 8 c + 7
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k0 = 8 * c + 2 * j;
                const uint32_t lo = one | ((__popc(n & k0) & 1u) << 15), hi = one | ((__popc(n & (k0 + 1)) & 1u) << 15);
                w[j] = lo | (hi << 16);
            }
            *reinterpret_cast<uint4*>(tsm + TcSmem::kH + c * 2048 + n * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tbase = *reinterpret_cast<volatile uint32_t*>(tsm + TcSmem::kTmemSlot);

    if (*bad == 0) {
        const uint32_t stage = sbase + TcSmem::kStage + group * kTcStageBytes;
        const uint32_t dcol = tbase + group * 128 + (static_cast<uint32_t>(gw * 32) << 16);
        constexpr uint32_t kBias = kMagicBits * static_cast<uint32_t>(kCellStride);
        const uint32_t tab = is_v ? smem_u32(tables + kTableBytes) + (lane & 15) * 8 - kBias
                                  : smem_u32(tables) + (QJL ? (lane & 7) * 16 : (lane & 15) * 8) - kBias;
        const void* src_base = is_v ? p.value : p.key;
        const int64_t st_t = is_v ? p.vs_t : p.ks_t, st_h = is_v ? p.vs_h : p.ks_h;
        const int64_t tile_step = static_cast<int64_t>(gridDim.x) * 2;

        // Copies of one tile: thread `row` knows where its own row starts; an instruction copies, for 4 rows, one
        // 128-byte line each (eight 16-byte chunks), so lanes fetch the row starts they need by shuffle.  Rows past the
        // end of the input are filled with zeros: their lanes of the product are then zero and quantize harmlessly.
        auto stage_tile = [&](int64_t tile) {
            const ItemId id = identify_item(p, tile * kTcTile + row);
            const uint16_t* mine = static_cast<const uint16_t*>(src_base) + id.tok * st_t + id.head * st_h;
            const unsigned long long addr = reinterpret_cast<unsigned long long>(mine);
#pragma unroll
            for (int rg = 0; rg < 8; ++rg) {
                const int r_local = 4 * rg + (lane >> 3);
                const unsigned long long a = __shfl_sync(0xffffffffu, addr, r_local);
                const int live = __shfl_sync(0xffffffffu, id.live ? 1 : 0, r_local);
                const uint32_t dst = stage + (gw * 32 + r_local) * 16 + (lane & 7) * kTcChunkStride;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (live)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + half * 8 * kTcChunkStride),
                                     "l"(a + (8 * half + (lane & 7)) * 16) : "memory");
                    else
                        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dst + half * 8 * kTcChunkStride), "r"(0u) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };

        int64_t tile = static_cast<int64_t>(blockIdx.x) * 2 + (group >> 1);
        uint32_t phase = 0;
        bool failed = false;
        if (tile < n_tiles) stage_tile(tile);
        for (; tile < n_tiles && !failed; tile += tile_step) {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");     // this thread's reads of the previous tile are done
            asm volatile("bar.sync %0, 128;" ::"r"(1 + group) : "memory");
            if (gw == 0 && lane == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t idesc = tc_idesc(bf16 ? 1 : 0);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    tc_mma_f16(tbase + group * 128, tc_desc(stage + ks * 2 * kTcChunkStride, kTcChunkStride, 128),
                               tc_desc(sbase + TcSmem::kH + ks * 4096, 2048, 128), idesc, ks ? 1u : 0u);
                tc_commit(bars + group);
            }
            // where this thread's item goes (the slot look-up overlaps the product)
            const ItemPlace w = place_item<PAGE>(p, tile * kTcTile + row, 0);
            if (!tc_mbar_wait(bars + group, phase)) { failed = true; break; }
            phase ^= 1u;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // the staging buffer is free again: next tile's copies fly while this one is quantized
            if (tile + tile_step < n_tiles) stage_tile(tile + tile_step);

            // ---- pass 1: squared norm of the rotated vector (16 columns at a time, next load in flight) -----------
            f2 acc0 = f2dup(0.f), acc1 = f2dup(0.f);
            {
                uint32_t da[16], db[16];
                auto sum16 = [&](const uint32_t (&d)[16]) {
#pragma unroll
                    for (int i = 0; i < 16; i += 4) {
                        const f2 a = f2pack(__uint_as_float(d[i]), __uint_as_float(d[i + 1]));
                        const f2 b = f2pack(__uint_as_float(d[i + 2]), __uint_as_float(d[i + 3]));
                        acc0 = f2fma(a, a, acc0);
                        acc1 = f2fma(b, b, acc1);
                    }
                };
                tc_ld16(dcol, da);
#pragma unroll 1
                for (int h = 0; h < 8; h += 2) {
                    tc_wait_ld();
                    tc_ld16(dcol + (h + 1) * 16, db);
                    sum16(da);
                    tc_wait_ld();
                    if (h + 2 < 8) tc_ld16(dcol + (h + 2) * 16, da);
                    sum16(db);
                }
            }
            float s0, s1, s2, s3;
            f2unpack(acc0, s0, s1);
            f2unpack(acc1, s2, s3);
            const float ss = (s0 + s1) + (s2 + s3);
            const bool finite = ss < __uint_as_float(0x7f800000u);     // false for NaN too
            if (__any_sync(0xffffffffu, !finite)) {
                // NaN or overflow somewhere in a vector: its row of the product is replaced by zeros so that the table
                // look-ups stay in range (the stored norm still shows the bad value); rare, so a branch of its own
#pragma unroll 1
                for (int h = 0; h < 8; ++h) {
                    uint32_t d[16];
                    tc_ld16(dcol + h * 16, d);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) d[i] = finite ? d[i] : 0u;
                    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                                 ::"r"(dcol + h * 16), "r"(d[0]), "r"(d[1]), "r"(d[2]), "r"(d[3]), "r"(d[4]), "r"(d[5]), "r"(d[6]), "r"(d[7]),
                                   "r"(d[8]), "r"(d[9]), "r"(d[10]), "r"(d[11]), "r"(d[12]), "r"(d[13]), "r"(d[14]), "r"(d[15]) : "memory");
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            const float n_out = sqrtf(ss) * kWhtScale;                   // norm of x H with H normalised
            const float n = finite ? n_out : 0.f;
            const float den = (n + 1e-8f) * 11.313708498984761f;        // the unnormalised transform is sqrt(128) larger
            const float inv = __frcp_rn(den);
            VecConsts vc;
            vc.inv = f2dup(inv);
            vc.nden = f2dup(-den);
            vc.inv64 = f2dup(inv * kCellScale);
            vc.n = f2dup(n);
            vc.tab = tab;
            // ---- pass 2: quantize and store quarter by quarter; the quarter's upper 16 columns are loaded while the
            // previous half is quantized, its lower 16 while the upper half is ------------------------------------
            f2 rr = f2dup(0.f);
            {
                uint32_t dhi[16], dlo[16];
                tc_ld16(dcol + 16, dhi);
#pragma unroll 1
                for (int qt = 0; qt < 4; ++qt) {
                    float cvh[4], cvl[4];
                    uint32_t sg_hi, sg_lo;
                    tc_wait_ld();
                    tc_ld16(dcol + qt * 32, dlo);
                    if (is_v) quantize_half_fast<false>(dhi, vc, rr, cvh, sg_hi);
                    else quantize_half_fast<QJL>(dhi, vc, rr, cvh, sg_hi);
                    tc_wait_ld();
                    if (qt < 3) tc_ld16(dcol + (qt + 1) * 32 + 16, dhi);
                    if (is_v) quantize_half_fast<false>(dlo, vc, rr, cvl, sg_lo);
                    else quantize_half_fast<QJL>(dlo, vc, rr, cvl, sg_lo);
                    const float cv[8] = {cvl[0], cvl[1], cvl[2], cvl[3], cvh[0], cvh[1], cvh[2], cvh[3]};
                    Packed q;
                    q.norm = n_out;
                    q.rnorm = 0.f;                               // the residual norm is complete after the last quarter
                    q.signs = QJL ? ~prmt(sg_lo, sg_hi, 0x5410) : 0u;
                    if (is_v) {
                        assemble_indices<VB, true>(cv, q);
                        if (w.live) store_v_fast<VB>(w.page + KPART, w.t, qt, q);
                    } else {
                        assemble_indices<KB, false>(cv, q);
                        if (w.live) store_k_fast<KB, QJL>(w.page, w.t, qt, q);
                    }
                }
            }
            if constexpr (QJL) {
                if (!is_v && w.live) {
                    float ra, rb;
                    f2unpack(rr, ra, rb);
                    constexpr int RK = 16 * (KB + 1);
                    reinterpret_cast<__half*>(w.page + 16 * RK + 32)[norm_slot(w.t)] = __float2half_rn(sqrtf(ra + rb));
                }
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (failed && p.status && lane == 0) atomicOr(p.status, TQ_STATUS_TIMEOUT);
    } else {
        // two boundaries inside one table cell: binary-search path, 8 items per warp at a time
        __shared__ float csm[16];
        if (tid < (1 << KB)) csm[tid] = p.kc[tid];
        asm volatile("bar.sync 5, 512;" ::: "memory");
        const PagedParams pc = p;
        const int64_t n_groups = (p.n_items + kTcThreads / 4 - 1) / (kTcThreads / 4);
        for (int64_t grp = blockIdx.x; grp < n_groups; grp += gridDim.x)
            compress_items_generic<KB, VB, QJL>(pc, grp * (kTcThreads / 4) + warp * kItemsPerWarp + (lane >> 2), lane, csm);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(512u) : "memory");
}

template <int KB, int VB, bool QJL>
int launch_paged_tc(const PagedParams& p, cudaStream_t st) {
    const int64_t n_tiles = (p.n_items + kTcTile - 1) / kTcTile;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TQ_ERR_LAUNCH;
    static int sm_count[64] = {0};
    if (sm_count[dev]) sms = sm_count[dev];
    else {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return TQ_ERR_LAUNCH;
        sm_count[dev] = sms;
    }
    const int64_t want = (n_tiles + 1) / 2;                 // a CTA has two tiles in flight
    const unsigned grid = static_cast<unsigned>(want < sms ? want : sms);
    static bool configured[64] = {false};
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(compress_paged_tc_kernel<KB, VB, QJL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 TcSmem::kTotal) != cudaSuccess)
            return TQ_ERR_LAUNCH;
        configured[dev] = true;
    }
    compress_paged_tc_kernel<KB, VB, QJL><<<grid, kTcThreads, TcSmem::kTotal, st>>>(p, n_tiles);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

}  // namespace
}  // namespace tq
