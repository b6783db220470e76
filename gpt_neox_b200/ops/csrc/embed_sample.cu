// Vocabulary-parallel embedding (gather forward, scatter-add backward) and the top-k / top-p logit filter used by
// sampling.
//
// Embedding: a rank owns vocabulary rows [v0, v1).  Forward copies the row of every in-range id (16-byte vectors) and
// writes zeros for ids owned by another rank, so the all-reduce over the tensor-parallel group that follows sums
// exactly one non-zero contribution per token (megatron/mpu/layers.py:98-180 of the reference does this with a mask,
// F.embedding and a masked fill).  Backward adds every gradient row into an fp32 [v1 - v0, h] buffer with vector
// atomics -- the engine passes the parameter's fp32 main-gradient view, so no vocabulary-sized bf16 gradient tensor
// and no cast/accumulate pass exist.
//
// Sampling filter: one CTA per row keeps the row in shared memory, finds the k-th largest logit and the nucleus
// threshold by bisection on the value (each probe is one block-wide count / probability-mass reduction), and writes
// -inf over everything outside (megatron/text_generation_utils.py:93-137 sorts the row instead).
#include "neox_b200.h"
#include <cuda_bf16.h>
#include <float.h>

namespace {

typedef __nv_bfloat16 bf16;

__global__ void __launch_bounds__(128) embed_fwd_kernel(const long long* __restrict__ ids, const uint4* __restrict__ w,
                                                        uint4* __restrict__ out, long long tokens, int hvec, long long v0,
                                                        long long v1) {
    for (long long t = blockIdx.x; t < tokens; t += gridDim.x) {
        const long long id = ids[t];
        uint4* o = out + t * hvec;
        if (id >= v0 && id < v1) {
            const uint4* r = w + (id - v0) * hvec;
            for (int i = threadIdx.x; i < hvec; i += blockDim.x) o[i] = __ldg(r + i);
        } else {
            for (int i = threadIdx.x; i < hvec; i += blockDim.x) o[i] = make_uint4(0, 0, 0, 0);
        }
    }
}

__global__ void __launch_bounds__(128) embed_bwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ g,
                                                        float* __restrict__ grad, long long tokens, int h, long long v0,
                                                        long long v1) {
    for (long long t = blockIdx.x; t < tokens; t += gridDim.x) {
        const long long id = ids[t];
        if (id < v0 || id >= v1) continue;
        const bf16* gr = g + t * h;
        float* dst = grad + (id - v0) * h;
        for (int i = threadIdx.x * 4; i < h; i += blockDim.x * 4) {
            const uint2 raw = *reinterpret_cast<const uint2*>(gr + i);
            float4 v;
            v.x = __uint_as_float(raw.x << 16);
            v.y = __uint_as_float(raw.x & 0xFFFF0000u);
            v.z = __uint_as_float(raw.y << 16);
            v.w = __uint_as_float(raw.y & 0xFFFF0000u);
            atomicAdd(reinterpret_cast<float4*>(dst + i), v);
        }
    }
}

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) r += red[i];
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = -FLT_MAX;
    for (int i = 0; i < (blockDim.x >> 5); ++i) r = fmaxf(r, red[i]);
    return r;
}

// out = logits where kept, -inf elsewhere.  top_k <= 0 and top_p <= 0 disable the respective filter.
__global__ void __launch_bounds__(1024) sample_filter_kernel(const float* __restrict__ logits, float* __restrict__ out,
                                                             int V, int top_k, float top_p) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const float* in = logits + (size_t)blockIdx.x * V;
    float* o = out + (size_t)blockIdx.x * V;
    float mx = -FLT_MAX, mn = FLT_MAX;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float x = in[i];
        row[i] = x;
        if (x > -FLT_MAX) {            // ignore entries that are already -inf
            mx = fmaxf(mx, x);
            mn = fminf(mn, x);
        }
    }
    mx = block_max(mx, red);
    mn = -block_max(-mn, red);
    float thr = -FLT_MAX;              // keep x >= thr
    if (top_k > 0 && top_k < V) {
        // largest t with count(x >= t) >= k  ==  the k-th largest value; 40 halvings of [mn, mx] reach fp32 resolution
        float lo = mn, hi = mx;
        for (int it = 0; it < 40; ++it) {
            const float mid = 0.5f * (lo + hi);
            float cnt = 0.f;
            for (int i = threadIdx.x; i < V; i += blockDim.x) cnt += row[i] >= mid ? 1.f : 0.f;
            cnt = block_sum(cnt, red);
            if (cnt >= (float)top_k) lo = mid; else hi = mid;
        }
        thr = lo;
    }
    if (top_p > 0.f && top_p < 1.f) {
        // A token is kept iff the probability mass of the tokens strictly above it is <= top_p (the sorted-cumsum
        // rule of the reference, shifted by one so the token that crosses the threshold stays).  mass(x > t) is a
        // non-increasing step function of t that steps exactly at row values, so bisect for the point where it
        // drops to <= top_p and snap to the row value there.  Probabilities are over the survivors of top-k.
        float z = 0.f;
        for (int i = threadIdx.x; i < V; i += blockDim.x) z += row[i] >= thr ? __expf(row[i] - mx) : 0.f;
        z = block_sum(z, red);
        float lo = (thr > -FLT_MAX ? thr : mn) - 1.f, hi = mx;       // mass above the maximum is 0: condition holds
        for (int it = 0; it < 48; ++it) {
            const float mid = 0.5f * (lo + hi);
            float m = 0.f;
            for (int i = threadIdx.x; i < V; i += blockDim.x)
                m += (row[i] > mid && row[i] >= thr) ? __expf(row[i] - mx) : 0.f;
            m = block_sum(m, red);
            if (m <= top_p * z) hi = mid; else lo = mid;
        }
        float best = -FLT_MAX;                                         // the boundary token: largest value <= hi
        for (int i = threadIdx.x; i < V; i += blockDim.x)
            if (row[i] <= hi && row[i] >= thr) best = fmaxf(best, row[i]);
        best = block_max(best, red);
        thr = fmaxf(thr, best);
    }
    for (int i = threadIdx.x; i < V; i += blockDim.x) o[i] = row[i] >= thr ? row[i] : -INFINITY;
}

}  // namespace

extern "C" int neox_embedding_fwd(const long long* ids, const void* weight, void* out, long long tokens, int h,
                                  long long v0, long long v1, void* stream) {
    if (tokens <= 0) return 0;
    if (h % 8) return NEOX_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(weight) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return NEOX_ERR_ALIGN;
    long long grid = tokens < 148LL * 16 ? tokens : 148LL * 16;
    embed_fwd_kernel<<<(unsigned)grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        ids, static_cast<const uint4*>(weight), static_cast<uint4*>(out), tokens, h / 8, v0, v1);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// grad: fp32 [v1 - v0, h], accumulated into (not cleared).
extern "C" int neox_embedding_bwd(const long long* ids, const void* g, float* grad, long long tokens, int h,
                                  long long v0, long long v1, void* stream) {
    if (tokens <= 0) return 0;
    if (h % 4) return NEOX_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(g) & 7) || (reinterpret_cast<uintptr_t>(grad) & 15)) return NEOX_ERR_ALIGN;
    long long grid = tokens < 148LL * 16 ? tokens : 148LL * 16;
    embed_bwd_kernel<<<(unsigned)grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        ids, static_cast<const bf16*>(g), grad, tokens, h, v0, v1);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// logits, out: fp32 [rows, V]; V * 4 bytes must fit in shared memory (V <= 56000).
extern "C" int neox_sample_filter(const float* logits, float* out, int rows, int V, int top_k, float top_p,
                                  void* stream) {
    if (rows <= 0) return 0;
    const int smem = V * (int)sizeof(float);
    if (smem > 224 * 1024) return NEOX_ERR_TOO_LARGE;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(sample_filter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024) !=
            cudaSuccess)
            return NEOX_ERR_LAUNCH;
        attr_set = true;
    }
    sample_filter_kernel<<<rows, 1024, smem, static_cast<cudaStream_t>(stream)>>>(logits, out, V, top_k, top_p);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
