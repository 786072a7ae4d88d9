// Shared device helpers for the TurboQuant sm_100a kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tq_b200.h"

namespace tq {

constexpr int kHeadDim = 128;
constexpr int kPageTokens = 16;
constexpr float kWhtScale = 0.08838834764831845f;   // 2^-3.5, every |entry| of the normalised 128x128 WHT
constexpr float kLog2e = 1.4426950408889634f;

// ---- page layout (mirrors turboquant/kernels/paged_layout.py) -----------------
__host__ __device__ constexpr int k_record_bytes(int kb, int qjl) { return 16 * (kb + qjl); }
__host__ __device__ constexpr int k_norm_off(int kb, int qjl) { return 16 * k_record_bytes(kb, qjl); }
__host__ __device__ constexpr int k_part_bytes(int kb, int qjl) { return k_norm_off(kb, qjl) + 32 + 32 * qjl; }
__host__ __device__ constexpr int v_part_bytes(int vb) { return 256 * vb + 32; }
__host__ __device__ constexpr int page_bytes(int kb, int vb, int qjl) { return k_part_bytes(kb, qjl) + v_part_bytes(vb); }
__host__ __device__ constexpr int norm_slot(int t) { return (t & 7) * 2 + (t >> 3); }

// ---- small PTX wrappers ---------------------------------------------------------
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float2 unpack_half2(uint32_t x) {
    return __half22float2(*reinterpret_cast<__half2*>(&x));
}

__device__ __forceinline__ float ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// ---- mbarrier + bulk async copy (global -> this CTA's shared memory) ------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: gives up after ~2^22 polls and reports failure instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < (1 << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}

// Non-multicast bulk copy from this GPU's own global memory; dst/src 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- input element loads ----------------------------------------------------------
// Loads 4 consecutive elements starting at p (dtype: 0 = fp16, 1 = bf16, 2 = fp32) as fp32.
__device__ __forceinline__ void load4(const void* base, int64_t elem_off, int dtype, float (&x)[4]) {
    if (dtype == TQ_DTYPE_F32) {
        float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem_off);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    } else {
        uint2 v = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(base) + elem_off);
        if (dtype == TQ_DTYPE_F16) {
            float2 a = unpack_half2(v.x), b = unpack_half2(v.y);
            x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
        } else {
            x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xffff0000u);
            x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xffff0000u);
        }
    }
}

// ---- 128-point WHT over a group of 4 lanes (unnormalised) ---------------------------------------
__device__ __forceinline__ void fwht128(float (&x)[32], int lane) {
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (!(i & h)) {
                const float a = x[i], b = x[i + h];
                x[i] = a + b;
                x[i + h] = a - b;
            }
        }
    }
#pragma unroll
    for (int m = 1; m < 4; m <<= 1) {
        const float sgn = (lane & m) ? -1.f : 1.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = fmaf(sgn, x[i], __shfl_xor_sync(0xffffffffu, x[i], m));
    }
}


}  // namespace tq
