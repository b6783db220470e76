// Mixture-of-experts routing kernels: fused router (softmax + top-k + renormalisation + expert histogram) with its
// backward, the dispatch of token rows into the expert-major, padded activation matrix, and the weighted combine of
// the expert outputs with its backward.  All bandwidth-bound, fp32 arithmetic, no atomics on floating-point data
// (results are bit-reproducible).
//
// Reference counterparts: the eager router of megatron/model/router.py (softmax, torch.topk, renormalise) and the
// MegaBlocks / DeepSpeed scatter-gather ops the reference's MoE layers call (megatron/model/moe.py,
// megatron/model/moe_mlp.py); there the permutation runs as library kernels with a host round trip for the
// per-expert bin sizes, here positions stay on the device.
#include "neox_b200.h"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <float.h>

namespace {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

constexpr int MAX_E = 512;              // experts per router
constexpr int EPL = MAX_E / 32;         // per lane
constexpr int MAX_K = 8;                // top-k

// One warp per token: probs = softmax(logits) (fp32), the k largest with their indices (ties: lowest index), the
// weights renormalised to sum 1 when k > 1, and counts[e] += 1 for every selected expert (integer atomics).
template <typename T>
__global__ void __launch_bounds__(256) moe_router_fwd_kernel(const T* __restrict__ logits, float* __restrict__ probs,
                                                             float* __restrict__ w, long long* __restrict__ idx,
                                                             unsigned long long* __restrict__ counts, int tokens,
                                                             int E, int k) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= tokens) return;
    float v[EPL];
    float mx = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int e = i * 32 + lane;
        v[i] = e < E ? to_f(logits[(long long)t * E + e]) : -FLT_MAX;
        mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int e = i * 32 + lane;
        v[i] = e < E ? __expf(v[i] - mx) : 0.f;
        s += v[i];
    }
    s = warp_sum(s);
    const float inv = 1.0f / s;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int e = i * 32 + lane;
        v[i] *= inv;
        if (e < E) probs[(long long)t * E + e] = v[i];
    }
    float sel_w[MAX_K];
    int sel_e[MAX_K];
    float total = 0.f;
    for (int j = 0; j < k; ++j) {
        float best = -1.f;
        int be = MAX_E;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int e = i * 32 + lane;
            if (e < E && v[i] > best) {   // ascending e within a lane: the first maximum wins
                best = v[i];
                be = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ob > best || (ob == best && oe < be)) {
                best = ob;
                be = oe;
            }
        }
        sel_w[j] = best;
        sel_e[j] = be;
        total += best;
#pragma unroll
        for (int i = 0; i < EPL; ++i)
            if (i * 32 + lane == be) v[i] = -2.f;   // taken
    }
    if (lane == 0) {
        const float norm = k > 1 ? 1.0f / total : 1.0f;
        for (int j = 0; j < k; ++j) {
            w[(long long)t * k + j] = sel_w[j] * norm;
            idx[(long long)t * k + j] = sel_e[j];
            atomicAdd(counts + sel_e[j], 1ull);
        }
    }
}

// dlogits = probs * (dp - sum(dp * probs)), dp = dprobs (optional) + the gradient arriving through the selected
// weights: k == 1: dw; k > 1 (w_j = p_j / S): (dw_j - sum_i dw_i w_i) / S.
template <typename T>
__global__ void __launch_bounds__(256) moe_router_bwd_kernel(const float* __restrict__ probs,
                                                             const float* __restrict__ w,
                                                             const long long* __restrict__ idx,
                                                             const float* __restrict__ dw,
                                                             const float* __restrict__ dprobs,
                                                             T* __restrict__ dlogits, int tokens, int E, int k) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= tokens) return;
    float p[EPL], dp[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int e = i * 32 + lane;
        p[i] = e < E ? probs[(long long)t * E + e] : 0.f;
        dp[i] = (e < E && dprobs) ? dprobs[(long long)t * E + e] : 0.f;
    }
    if (dw) {
        float dot = 0.f, S = 1.f;
        if (k > 1) {
            float ssel = 0.f;
            for (int j = 0; j < k; ++j) {
                const int e = (int)idx[(long long)t * k + j];
                dot += dw[(long long)t * k + j] * w[(long long)t * k + j];
                // p of the selected expert lives in lane e % 32, slot e / 32
                float pe = 0.f;
#pragma unroll
                for (int i = 0; i < EPL; ++i)
                    if (i == e / 32) pe = p[i];
                ssel += __shfl_sync(0xffffffffu, pe, e & 31);
            }
            S = ssel;
        }
        for (int j = 0; j < k; ++j) {
            const int e = (int)idx[(long long)t * k + j];
            const float g = k > 1 ? (dw[(long long)t * k + j] - dot) / S : dw[(long long)t * k + j];
#pragma unroll
            for (int i = 0; i < EPL; ++i)
                if (i * 32 + lane == e) dp[i] += g;
        }
    }
    float inner = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) inner += dp[i] * p[i];
    inner = warp_sum(inner);
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int e = i * 32 + lane;
        if (e < E) dlogits[(long long)t * E + e] = from_f<T>(p[i] * (dp[i] - inner));
    }
}

// 8 x 16-bit vector helpers
template <typename T> __device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]);
template <> __device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& q, float (&f)[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <> __device__ __forceinline__ void unpack8<__half>(const uint4& q, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __half22float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}
template <typename T> __device__ __forceinline__ uint4 pack8(const float (&f)[8]);
template <> __device__ __forceinline__ uint4 pack8<__nv_bfloat16>(const float (&f)[8]) {
    uint4 q;
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]),
                   c = __floats2bfloat162_rn(f[4], f[5]), d = __floats2bfloat162_rn(f[6], f[7]);
    q.x = *reinterpret_cast<uint32_t*>(&a); q.y = *reinterpret_cast<uint32_t*>(&b);
    q.z = *reinterpret_cast<uint32_t*>(&c); q.w = *reinterpret_cast<uint32_t*>(&d);
    return q;
}
template <> __device__ __forceinline__ uint4 pack8<__half>(const float (&f)[8]) {
    uint4 q;
    __half2 a = __floats2half2_rn(f[0], f[1]), b = __floats2half2_rn(f[2], f[3]), c = __floats2half2_rn(f[4], f[5]),
            d = __floats2half2_rn(f[6], f[7]);
    q.x = *reinterpret_cast<uint32_t*>(&a); q.y = *reinterpret_cast<uint32_t*>(&b);
    q.z = *reinterpret_cast<uint32_t*>(&c); q.w = *reinterpret_cast<uint32_t*>(&d);
    return q;
}

// Dispatch: out[row_of[t, j], :] = x[t, :] * (scale ? scale[t, j] : 1) for every assignment with row_of >= 0.
// With `other` (same layout as out) it also writes dots[t, j] = <x[t], other[row]> -- the combine's backward, where
// x is dy, scale the gates, out the gradient of the expert outputs and dots the gradient of the gates.
// One warp per assignment; cols % 8 == 0.
template <typename T>
__global__ void __launch_bounds__(256) moe_dispatch_kernel(const T* __restrict__ x, const long long* __restrict__ row_of,
                                                           const float* __restrict__ scale, T* __restrict__ out,
                                                           const T* __restrict__ other, float* __restrict__ dots,
                                                           long long assignments, int k, int cols) {
    const int lane = threadIdx.x & 31;
    const long long a = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (a >= assignments) return;
    const long long row = row_of[a];
    if (row < 0) {
        if (dots && lane == 0) dots[a] = 0.f;
        return;
    }
    const long long t = a / k;
    const float sc = scale ? scale[a] : 1.0f;
    const uint4* src = reinterpret_cast<const uint4*>(x + t * cols);
    uint4* dst = reinterpret_cast<uint4*>(out + row * cols);
    const uint4* oth = other ? reinterpret_cast<const uint4*>(other + row * cols) : nullptr;
    float dot = 0.f;
    for (int c = lane; c < cols / 8; c += 32) {
        const uint4 q = __ldg(src + c);
        if (scale || oth) {
            float f[8];
            unpack8<T>(q, f);
            if (oth) {
                float g[8];
                unpack8<T>(__ldg(oth + c), g);
#pragma unroll
                for (int i = 0; i < 8; ++i) dot += f[i] * g[i];
            }
            if (scale) {
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] *= sc;
                dst[c] = pack8<T>(f);
            } else {
                dst[c] = q;
            }
        } else {
            dst[c] = q;
        }
    }
    if (dots) {
        dot = warp_sum(dot);
        if (lane == 0) dots[a] = dot;
    }
}

// Combine: y[t, :] = sum_j (gate ? gate[t, j] : 1) * src[row_of[t, j], :] over the assignments with row_of >= 0
// (fp32 accumulation in a fixed order).  One warp per token; cols % 8 == 0.
template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const T* __restrict__ src, const long long* __restrict__ row_of,
                                                          const float* __restrict__ gate, T* __restrict__ y,
                                                          long long tokens, int k, int cols) {
    const int lane = threadIdx.x & 31;
    const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= tokens) return;
    uint4* dst = reinterpret_cast<uint4*>(y + t * cols);
    for (int c = lane; c < cols / 8; c += 32) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < k; ++j) {
            const long long row = row_of[t * k + j];
            if (row < 0) continue;
            const float g = gate ? gate[t * k + j] : 1.0f;
            float f[8];
            unpack8<T>(__ldg(reinterpret_cast<const uint4*>(src + row * cols) + c), f);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += g * f[i];
        }
        dst[c] = pack8<T>(acc);
    }
}

}  // namespace

extern "C" {

// dtype of logits / dlogits: 0 bf16, 1 fp32, 2 fp16.  counts must be zeroed by the caller.
int neox_moe_router_fwd(const void* logits, float* probs, float* w, long long* idx, long long* counts, int tokens,
                        int E, int k, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (E < 1 || E > MAX_E || k < 1 || k > MAX_K || k > E) return NEOX_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    const int grid = (tokens + 7) / 8;
    unsigned long long* c = reinterpret_cast<unsigned long long*>(counts);
    if (dtype == 0)
        moe_router_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)logits, probs, w, idx, c, tokens, E, k);
    else if (dtype == 1)
        moe_router_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)logits, probs, w, idx, c, tokens, E, k);
    else
        moe_router_fwd_kernel<__half><<<grid, 256, 0, st>>>((const __half*)logits, probs, w, idx, c, tokens, E, k);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

int neox_moe_router_bwd(const float* probs, const float* w, const long long* idx, const float* dw,
                        const float* dprobs, void* dlogits, int tokens, int E, int k, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (E < 1 || E > MAX_E || k < 1 || k > MAX_K) return NEOX_ERR_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream;
    const int grid = (tokens + 7) / 8;
    if (dtype == 0)
        moe_router_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(probs, w, idx, dw, dprobs, (__nv_bfloat16*)dlogits, tokens, E, k);
    else if (dtype == 1)
        moe_router_bwd_kernel<float><<<grid, 256, 0, st>>>(probs, w, idx, dw, dprobs, (float*)dlogits, tokens, E, k);
    else
        moe_router_bwd_kernel<__half><<<grid, 256, 0, st>>>(probs, w, idx, dw, dprobs, (__half*)dlogits, tokens, E, k);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// dtype: 0 bf16, 2 fp16 (rows are moved as 16-byte vectors: cols % 8 == 0, 16-byte aligned bases).
int neox_moe_dispatch(const void* x, const long long* row_of, const float* scale, void* out, const void* other,
                      float* dots, long long tokens, int k, int cols, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (cols % 8 || (dtype != 0 && dtype != 2)) return NEOX_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
        (reinterpret_cast<uintptr_t>(other) & 15))
        return NEOX_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const long long n = tokens * k;
    const unsigned grid = (unsigned)((n + 7) / 8);
    if (dtype == 0)
        moe_dispatch_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, row_of, scale, (__nv_bfloat16*)out,
                                                                 (const __nv_bfloat16*)other, dots, n, k, cols);
    else
        moe_dispatch_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, row_of, scale, (__half*)out,
                                                          (const __half*)other, dots, n, k, cols);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

int neox_moe_combine(const void* src, const long long* row_of, const float* gate, void* y, long long tokens, int k,
                     int cols, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (cols % 8 || (dtype != 0 && dtype != 2)) return NEOX_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(y) & 15)) return NEOX_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = (unsigned)((tokens + 7) / 8);
    if (dtype == 0)
        moe_combine_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)src, row_of, gate, (__nv_bfloat16*)y, tokens, k, cols);
    else
        moe_combine_kernel<__half><<<grid, 256, 0, st>>>((const __half*)src, row_of, gate, (__half*)y, tokens, k, cols);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

}  // extern "C"
