// Contiguous packed decode attention (one query row per BH, no GQA, no paging) and the
// row-wise fast Walsh-Hadamard rotation, for sm_100a.
//
// packed_attention keeps the data layout of the reference's Triton path
// (turboquant/kernels/packed_attention.py:76-227): token-major index bytes,
// sign bytes in the stride-4 order of permute_signs_for_chunked
// (turboquant/kernels/packed_compress.py:180-216) and separate fp16 norm arrays.
// With one query per K/V stream there is no group to share tensor-core tiles, so
// this kernel is plain CUDA-core code: a CTA scores 128 tokens at a time with one
// token per thread (index bits never leave registers, the codebook and the query
// sit in shared memory), applies the online softmax per tile, and accumulates V
// with one warp per token row (a lane owns the 4 dims of one packed byte).
#include "tq_common.cuh"

namespace tq {
namespace {

constexpr int kThreads = 128;

template <int BITS>
__device__ __forceinline__ uint32_t extract_idx(const uint32_t* w, int d) {
    const int bit = d * BITS, lo = bit >> 5, sh = bit & 31;
    uint32_t v = w[lo] >> sh;
    if (sh + BITS > 32) v |= w[lo + 1] << (32 - sh);
    return v & ((1u << BITS) - 1u);
}

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
    float* ws_lse;   // [BH, splits, 2]  (max, sum)
    __half* out;
    float corr_scale;
    int Sk, num_splits;
};

template <int BITS>
__global__ void __launch_bounds__(kThreads) packed_attn_partial(const PAParams p) {
    constexpr int ROW = 16 * BITS;          // index bytes per token
    constexpr int NWORD = ROW / 4;
    __shared__ __align__(16) float sq[kHeadDim];
    __shared__ __align__(16) float sqp[kHeadDim];
    __shared__ float scb[1 << BITS];
    __shared__ float spv[kThreads];         // p * v_norm of the tile's tokens
    __shared__ float sred[4];
    __shared__ __align__(16) float sacc[4][kHeadDim];

    const int bh = blockIdx.x, split = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int per = (p.Sk + p.num_splits - 1) / p.num_splits;   // tokens per split (packed_attention.py:98-100)
    const int t0 = split * per, t1 = min(t0 + per, p.Sk);

    sq[tid] = __half2float(p.Q[static_cast<int64_t>(bh) * kHeadDim + tid]);
    sqp[tid] = __half2float(p.Qp[static_cast<int64_t>(bh) * kHeadDim + tid]) * p.corr_scale;
    if (tid < (1 << BITS)) scb[tid] = p.centroids[tid];
    __syncthreads();

    float m_run = -INFINITY, l_run = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};    // this lane's 4 dims, this warp's share of tokens
    const int64_t base = static_cast<int64_t>(bh) * p.Sk;

    for (int tile = t0; tile < t1; tile += kThreads) {
        const int tok = tile + tid;
        float s = -INFINITY;
        float vn = 0.f;
        if (tok < t1) {
            uint32_t w[NWORD];
            const uint4* kp = reinterpret_cast<const uint4*>(p.k_idx + (base + tok) * ROW);
#pragma unroll
            for (int i = 0; i < NWORD / 4; ++i) {
                const uint4 v = __ldg(kp + i);
                w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
            }
            const uint4 sg = __ldg(reinterpret_cast<const uint4*>(p.k_signs + (base + tok) * 16));
            const uint32_t sw[4] = {sg.x, sg.y, sg.z, sg.w};
            float mse = 0.f, pos = 0.f, all = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float4 q4 = *reinterpret_cast<const float4*>(sq + 4 * j);
                const float4 p4 = *reinterpret_cast<const float4*>(sqp + 4 * j);
                const float qv[4] = {q4.x, q4.y, q4.z, q4.w};
                const float pv[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    mse = fmaf(qv[c], scb[extract_idx<BITS>(w, 4 * j + c)], mse);
                    // stride-4 sign order: dim 4 j + c is bit j of word c
                    pos += ((sw[c] >> j) & 1u) ? pv[c] : 0.f;
                    all += pv[c];
                }
            }
            const float kn = __half2float(p.k_norm[base + tok]);
            const float krn = __half2float(p.k_rnorm[base + tok]);
            s = fmaf(krn, 2.f * pos - all, kn * mse);
            vn = __half2float(p.v_norm[base + tok]);
        }
        // tile maximum
        float mx = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) sred[warp] = mx;
        __syncthreads();
        const float m_new = fmaxf(m_run, fmaxf(fmaxf(sred[0], sred[1]), fmaxf(sred[2], sred[3])));
        const float alpha = __expf(m_run - m_new);
        const float pr = (tok < t1) ? __expf(s - m_new) : 0.f;
        spv[tid] = pr * vn;
        float ps = pr;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        __syncthreads();   // sred reads done, spv visible
        if (lane == 0) sred[warp] = ps;
        l_run *= alpha;
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[c] *= alpha;
        m_run = m_new;
        // V: warp w takes tokens w, w+4, ... of the tile; lane owns dims 4*lane .. 4*lane+3
        const int ntile = min(kThreads, t1 - tile);
        for (int i = warp; i < ntile; i += 4) {
            const uint8_t* vr = p.v_idx + (base + tile + i) * ROW;
            uint32_t bits12;
            if constexpr (BITS == 2) bits12 = __ldg(vr + lane);
            else if constexpr (BITS == 4) bits12 = __ldg(reinterpret_cast<const uint16_t*>(vr) + lane);
            else {
                const int b = (3 * lane) >> 1;
                bits12 = ((__ldg(vr + b) | (static_cast<uint32_t>(__ldg(vr + b + 1)) << 8)) >> ((lane & 1) * 4)) & 0xfffu;
            }
            const float pvn = spv[i];
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[c] = fmaf(pvn, scb[(bits12 >> (BITS * c)) & ((1u << BITS) - 1u)], acc[c]);
        }
        __syncthreads();   // sred (sums) visible; spv free for the next tile
        l_run += sred[0] + sred[1] + sred[2] + sred[3];
        __syncthreads();
    }
    // combine the 4 warps' shares of the accumulator
    *reinterpret_cast<float4*>(&sacc[warp][4 * lane]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncthreads();
    const float o = sacc[0][tid] + sacc[1][tid] + sacc[2][tid] + sacc[3][tid];
    const int64_t slot = static_cast<int64_t>(bh) * p.num_splits + split;
    p.ws_acc[slot * kHeadDim + tid] = o;
    if (tid == 0) {
        p.ws_lse[slot * 2] = m_run;
        p.ws_lse[slot * 2 + 1] = l_run;
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
        const float w = (m == -INFINITY) ? 0.f : __expf(m - M);   // empty splits carry no weight
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
    // Enough CTAs for ~4 waves of 148 SMs x 8 CTAs, at least 256 tokens (two tiles) per split.
    int splits = (148 * 8 * 4 + BH - 1) / BH;
    const int max_splits = (Sk + 255) / 256;
    if (splits > max_splits) splits = max_splits;
    if (splits > 256) splits = 256;
    if (splits < 1) splits = 1;
    return splits;
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
    if (BH > 2147483647 / 1 || num_splits > 65535) return TQ_ERR_UNSUPPORTED;
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
    const dim3 grid(BH, num_splits);
    switch (bits) {
        case 2: packed_attn_partial<2><<<grid, kThreads, 0, st>>>(p); break;
        case 3: packed_attn_partial<3><<<grid, kThreads, 0, st>>>(p); break;
        case 4: packed_attn_partial<4><<<grid, kThreads, 0, st>>>(p); break;
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
