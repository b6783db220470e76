// Softmax (masked / causal), rotary embedding, vocabulary-parallel cross-entropy pieces, fused
// Adam / Lion updates and the squared-norm reduction.  All bandwidth-bound; fp32 arithmetic.
//
// Reference counterparts: scaled_masked_softmax.h / scaled_upper_triang_masked_softmax.h (one warp per
// row, sk <= 2048) and fused_rotary_positional_embedding.h of megatron/fused_kernels, the eager
// megatron/mpu/cross_entropy.py, and apex multi_tensor_adam / DeepSpeed FusedLion.  These versions take
// any row length, any of bf16/fp16/fp32, and strided rotary inputs.
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
template <bool MAX>
__device__ __forceinline__ float block_reduce(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = MAX ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (threadIdx.x < nw) ? red[threadIdx.x] : (MAX ? -FLT_MAX : 0.f);
    if (warp == 0) {
        t = MAX ? warp_max(t) : warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// ------------------------------------------------------------------ softmax
constexpr int SM_CACHE = 16;  // elements cached per thread (256 threads -> rows up to 4096 stay in registers)

template <typename T>
__global__ void __launch_bounds__(256) softmax_fwd_kernel(const T* __restrict__ x, const uint8_t* __restrict__ mask,
                                                          T* __restrict__ y, long long rows, int sq, int sk,
                                                          int heads, int mask_batches, float scale, int causal) {
    __shared__ float red[33];
    const bool cached = sk <= SM_CACHE * (int)blockDim.x;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * sk;
        T* yr = y + row * sk;
        const int q = (int)(row % sq);
        const uint8_t* mr = nullptr;
        if (mask) {
            const long long b = row / ((long long)heads * sq);
            mr = mask + ((mask_batches == 1 ? 0 : b) * sq + q) * (long long)sk;
        }
        const int limit = causal ? q + 1 : sk;  // columns >= limit are excluded (output exactly 0)
        float v[SM_CACHE];
        float mx = -FLT_MAX;
        auto fetch = [&](int c) -> float {
            float t = to_f<T>(xr[c]) * scale;
            if (mr && mr[c]) t = -10000.0f;
            return t;
        };
        if (cached) {
#pragma unroll
            for (int j = 0; j < SM_CACHE; ++j) {
                const int c = threadIdx.x + j * blockDim.x;
                v[j] = (c < limit) ? fetch(c) : -FLT_MAX;
                mx = fmaxf(mx, v[j]);
            }
        } else {
            for (int c = threadIdx.x; c < limit; c += blockDim.x) mx = fmaxf(mx, fetch(c));
        }
        mx = block_reduce<true>(mx, red);
        float s = 0.f;
        if (cached) {
#pragma unroll
            for (int j = 0; j < SM_CACHE; ++j) {
                const int c = threadIdx.x + j * blockDim.x;
                v[j] = (c < limit) ? __expf(v[j] - mx) : 0.f;
                s += v[j];
            }
        } else {
            for (int c = threadIdx.x; c < limit; c += blockDim.x) s += __expf(fetch(c) - mx);
        }
        s = block_reduce<false>(s, red);
        const float inv = 1.0f / s;
        if (cached) {
#pragma unroll
            for (int j = 0; j < SM_CACHE; ++j) {
                const int c = threadIdx.x + j * blockDim.x;
                if (c < sk) yr[c] = from_f<T>(v[j] * inv);
            }
        } else {
            for (int c = threadIdx.x; c < sk; c += blockDim.x)
                yr[c] = from_f<T>(c < limit ? __expf(fetch(c) - mx) * inv : 0.f);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) softmax_bwd_kernel(const T* __restrict__ g, const T* __restrict__ y,
                                                          T* __restrict__ dx, long long rows, int sk, float scale) {
    __shared__ float red[33];
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* gr = g + row * sk;
        const T* yr = y + row * sk;
        T* dr = dx + row * sk;
        float s = 0.f;
        for (int c = threadIdx.x; c < sk; c += blockDim.x) s += to_f<T>(gr[c]) * to_f<T>(yr[c]);
        s = block_reduce<false>(s, red);
        for (int c = threadIdx.x; c < sk; c += blockDim.x) {
            const float yv = to_f<T>(yr[c]);
            dr[c] = from_f<T>(scale * yv * (to_f<T>(gr[c]) - s));
        }
    }
}

// Rows of up to 2048 16-bit elements: one WARP per row, the row held in registers as NC chunks of 8 elements per lane
// (16-byte accesses, all of a lane's loads issued before the first use), maxima and sums by shuffles.  Chunks that lie
// wholly behind the causal limit are never read.  Needs sk % 8 == 0, sk <= 256 * NC, 16-byte aligned x / y and an
// 8-byte aligned mask; the caller checks.  Same arithmetic as softmax_fwd_kernel.
template <typename T, int NC>
__global__ void __launch_bounds__(256) softmax_fwd_warp_kernel(const T* __restrict__ x, const uint8_t* __restrict__ mask,
                                                               T* __restrict__ y, long long rows, int sq, int sk,
                                                               int heads, int mask_batches, float scale, int causal) {
    const int lane = threadIdx.x & 31;
    const int nchunk = sk >> 3;
    const int wpc = blockDim.x >> 5;                                     // warps (= rows in flight) per CTA
    const long long wstride = (long long)gridDim.x * wpc;
    for (long long row = (long long)blockIdx.x * wpc + (threadIdx.x >> 5); row < rows; row += wstride) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + row * sk);
        uint4* yr = reinterpret_cast<uint4*>(y + row * sk);
        const int q = (int)(row % sq);
        const uint2* mr = nullptr;
        if (mask) {
            const long long b = row / ((long long)heads * sq);
            mr = reinterpret_cast<const uint2*>(mask + ((mask_batches == 1 ? 0 : b) * sq + q) * (long long)sk);
        }
        const int limit = causal ? q + 1 : sk;
        uint4 raw[NC];
        uint2 mraw[NC];
#pragma unroll
        for (int j = 0; j < NC; ++j) {
            const int ch = lane + j * 32;
            const bool live = ch < nchunk && ch * 8 < limit;
            raw[j] = live ? __ldg(xr + ch) : make_uint4(0, 0, 0, 0);
            mraw[j] = (live && mr) ? __ldg(mr + ch) : make_uint2(0, 0);
        }
        float v[NC][8];
        float mx = -FLT_MAX;
#pragma unroll
        for (int j = 0; j < NC; ++j) {
            const int c0 = (lane + j * 32) * 8;
            const T* e = reinterpret_cast<const T*>(&raw[j]);
            const uint8_t* mb = reinterpret_cast<const uint8_t*>(&mraw[j]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float t = to_f<T>(e[i]) * scale;
                if (mb[i]) t = -10000.0f;
                v[j][i] = (c0 + i < limit) ? t : -FLT_MAX;        // limit <= sk, so dead chunks land here too
                mx = fmaxf(mx, v[j][i]);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NC; ++j) {
            const int c0 = (lane + j * 32) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[j][i] = (c0 + i < limit) ? __expf(v[j][i] - mx) : 0.f;
                s += v[j][i];
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float inv = 1.0f / s;
#pragma unroll
        for (int j = 0; j < NC; ++j) {
            const int ch = lane + j * 32;
            if (ch < nchunk) {
                uint4 o;
                T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
                for (int i = 0; i < 8; ++i) oe[i] = from_f<T>(v[j][i] * inv);
                yr[ch] = o;
            }
        }
    }
}

// Backward of the same rows: dx = scale * y * (g - sum(g * y)); g and y stay packed in registers between the passes.
template <typename T, int NC>
__global__ void __launch_bounds__(256) softmax_bwd_warp_kernel(const T* __restrict__ g, const T* __restrict__ y,
                                                               T* __restrict__ dx, long long rows, int sk, float scale) {
    const int lane = threadIdx.x & 31;
    const int nchunk = sk >> 3;
    const int wpc = blockDim.x >> 5;                                     // warps (= rows in flight) per CTA
    const long long wstride = (long long)gridDim.x * wpc;
    for (long long row = (long long)blockIdx.x * wpc + (threadIdx.x >> 5); row < rows; row += wstride) {
        const uint4* gr = reinterpret_cast<const uint4*>(g + row * sk);
        const uint4* yr = reinterpret_cast<const uint4*>(y + row * sk);
        uint4* dr = reinterpret_cast<uint4*>(dx + row * sk);
        uint4 graw[NC], yraw[NC];
#pragma unroll
        for (int j = 0; j < NC; ++j) {
            const int ch = lane + j * 32;
            graw[j] = ch < nchunk ? __ldg(gr + ch) : make_uint4(0, 0, 0, 0);
            yraw[j] = ch < nchunk ? __ldg(yr + ch) : make_uint4(0, 0, 0, 0);
        }
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NC; ++j) {
            const T* ge = reinterpret_cast<const T*>(&graw[j]);
            const T* ye = reinterpret_cast<const T*>(&yraw[j]);
#pragma unroll
            for (int i = 0; i < 8; ++i) s += to_f<T>(ge[i]) * to_f<T>(ye[i]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
#pragma unroll
        for (int j = 0; j < NC; ++j) {
            const int ch = lane + j * 32;
            if (ch < nchunk) {
                const T* ge = reinterpret_cast<const T*>(&graw[j]);
                const T* ye = reinterpret_cast<const T*>(&yraw[j]);
                uint4 o;
                T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
                for (int i = 0; i < 8; ++i) oe[i] = from_f<T>(scale * to_f<T>(ye[i]) * (to_f<T>(ge[i]) - s));
                dr[ch] = o;
            }
        }
    }
}

// ------------------------------------------------------------------ rotary
// x: [s, b, h, d] with element strides (ss, sb, sh) and unit stride on d; out: contiguous [s, b, h, d].
// First `rot` dims rotated with cos/sin [s, rot] (fp32), remaining dims copied.
template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const T* __restrict__ x, T* __restrict__ out,
                                                   const float* __restrict__ cs, const float* __restrict__ sn, int s,
                                                   int b, int h, int d, int rot, long long ss, long long sb,
                                                   long long sh, int inverse) {
    const long long total = (long long)s * b * h * d;
    const int half = rot >> 1;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int e = (int)(i % d);
        long long r = i / d;
        const int hh = (int)(r % h);
        r /= h;
        const int bb = (int)(r % b);
        const int sI = (int)(r / b);
        const T* xp = x + sI * ss + bb * sb + hh * sh;
        float v = to_f<T>(xp[e]);
        if (e < rot) {
            const float c = cs[(long long)sI * rot + e];
            float sv = sn[(long long)sI * rot + e];
            if (inverse) sv = -sv;
            const float other = (e < half) ? -to_f<T>(xp[e + half]) : to_f<T>(xp[e - half]);
            v = v * c + other * sv;
        }
        out[i] = from_f<T>(v);
    }
}

// Same operation with vector accesses of BYTES (16 or 8) bytes: one work item is the pair of chunks (e, e + rot/2) of
// one head -- it reads both once and writes both -- or one chunk of the unrotated tail.  Needs rot/2, d - rot and the
// strides to be multiples of the chunk (BYTES / sizeof(T) elements) and BYTES-aligned bases; the caller checks.
template <int BYTES> struct RopeVec;
template <> struct RopeVec<16> { using type = uint4; };
template <> struct RopeVec<8> { using type = uint2; };

template <typename T, int BYTES>
__global__ void __launch_bounds__(256) rope_vec_kernel(const T* __restrict__ x, T* __restrict__ out,
                                                       const float* __restrict__ cs, const float* __restrict__ sn,
                                                       int s, int b, int h, int d, int rot, long long ss, long long sb,
                                                       long long sh, int inverse) {
    using VT = typename RopeVec<BYTES>::type;
    constexpr int V = BYTES / (int)sizeof(T);
    const int half = rot >> 1;
    const int npair = half / V;
    const int items = npair + (d - rot) / V;
    const long long total = (long long)s * b * h * items;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int it = (int)(i % items);
        long long r = i / items;
        const int hh = (int)(r % h);
        r /= h;
        const int bb = (int)(r % b);
        const int sI = (int)(r / b);
        const T* xp = x + sI * ss + bb * sb + hh * sh;
        T* op = out + (((long long)sI * b + bb) * h + hh) * d;
        if (it >= npair) {
            const int e0 = rot + (it - npair) * V;
            *reinterpret_cast<VT*>(op + e0) = __ldg(reinterpret_cast<const VT*>(xp + e0));
            continue;
        }
        const int e0 = it * V;
        const VT ulo = __ldg(reinterpret_cast<const VT*>(xp + e0));
        const VT uhi = __ldg(reinterpret_cast<const VT*>(xp + e0 + half));
        const T* lo = reinterpret_cast<const T*>(&ulo);
        const T* hi = reinterpret_cast<const T*>(&uhi);
        const float* cp = cs + (long long)sI * rot + e0;
        const float* sp = sn + (long long)sI * rot + e0;
        VT olo, ohi;
        T* ol = reinterpret_cast<T*>(&olo);
        T* oh = reinterpret_cast<T*>(&ohi);
#pragma unroll
        for (int j = 0; j < V; j += 2) {                       // V is even; the tables are read 8 bytes at a time
            const float2 c0 = __ldg(reinterpret_cast<const float2*>(cp + j));
            const float2 c1 = __ldg(reinterpret_cast<const float2*>(cp + half + j));
            float2 s0 = __ldg(reinterpret_cast<const float2*>(sp + j));
            float2 s1 = __ldg(reinterpret_cast<const float2*>(sp + half + j));
            if (inverse) {
                s0 = make_float2(-s0.x, -s0.y);
                s1 = make_float2(-s1.x, -s1.y);
            }
            const float a0 = to_f<T>(lo[j]), b0 = to_f<T>(hi[j]);
            const float a1 = to_f<T>(lo[j + 1]), b1 = to_f<T>(hi[j + 1]);
            ol[j] = from_f<T>(a0 * c0.x - b0 * s0.x);
            ol[j + 1] = from_f<T>(a1 * c0.y - b1 * s0.y);
            oh[j] = from_f<T>(b0 * c1.x + a0 * s1.x);
            oh[j + 1] = from_f<T>(b1 * c1.y + a1 * s1.y);
        }
        *reinterpret_cast<VT*>(op + e0) = olo;
        *reinterpret_cast<VT*>(op + e0 + half) = ohi;
    }
}

// In-place rotary embedding of the first `rot` dims of every head of q and k (views of one packed QKV tensor): one
// thread owns the pair (e, e + rot/2), so nothing is read after it was overwritten.  cs / sn: [s, rot] fp32.
template <typename T>
__global__ void __launch_bounds__(256) rope_qk_inplace_kernel(T* __restrict__ q, T* __restrict__ k,
                                                              const float* __restrict__ cs, const float* __restrict__ sn,
                                                              int s, int b, int hq, int hk, int rot, long long q_ss,
                                                              long long q_sb, long long q_sh, long long k_ss,
                                                              long long k_sb, long long k_sh, int inverse) {
    const int half = rot >> 1;
    const int heads = hq + hk;
    const long long total = (long long)s * b * heads * half;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int e = (int)(i % half);
        long long r = i / half;
        const int hh = (int)(r % heads);
        r /= heads;
        const int bb = (int)(r % b);
        const int sI = (int)(r / b);
        T* xp = hh < hq ? q + sI * q_ss + bb * q_sb + hh * q_sh : k + sI * k_ss + bb * k_sb + (hh - hq) * k_sh;
        const float a = to_f<T>(xp[e]), c2 = to_f<T>(xp[e + half]);
        const float* cr = cs + (long long)sI * rot;
        const float* sr = sn + (long long)sI * rot;
        const float sg = inverse ? -1.f : 1.f;
        xp[e] = from_f<T>(a * cr[e] - c2 * sr[e] * sg);
        xp[e + half] = from_f<T>(c2 * cr[e + half] + a * sr[e + half] * sg);
    }
}

// ------------------------------------------------------------------ cross entropy
template <typename T>
__global__ void __launch_bounds__(256) row_max_kernel(const T* __restrict__ x, float* __restrict__ out, int rows,
                                                      int cols) {
    __shared__ float red[33];
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + (size_t)row * cols;
        float m = -FLT_MAX;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, to_f<T>(xr[c]));
        m = block_reduce<true>(m, red);
        if (threadIdx.x == 0) out[row] = m;
    }
}

// stats[row] = (sum_c exp(x - max), x[target - v0] - max if this shard owns the target else 0)
template <typename T>
__global__ void __launch_bounds__(256) ce_stats_kernel(const T* __restrict__ x, const long long* __restrict__ target,
                                                       const float* __restrict__ row_max, float* __restrict__ stats,
                                                       int rows, int cols, int v0) {
    __shared__ float red[33];
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + (size_t)row * cols;
        const float m = row_max[row];
        float s = 0.f;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) s += __expf(to_f<T>(xr[c]) - m);
        s = block_reduce<false>(s, red);
        if (threadIdx.x == 0) {
            const long long t = target[row] - v0;
            stats[2 * row] = s;
            stats[2 * row + 1] = (t >= 0 && t < cols) ? to_f<T>(xr[t]) - m : 0.f;
        }
    }
}

// grad = (exp(x - max) / sum_exp - [c == target - v0]) * g[row]
template <typename T>
__global__ void __launch_bounds__(256) ce_bwd_kernel(const T* __restrict__ x, const long long* __restrict__ target,
                                                     const float* __restrict__ row_max, const float* __restrict__ stats,
                                                     const float* __restrict__ g, T* __restrict__ grad, int rows,
                                                     int cols, int v0) {
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + (size_t)row * cols;
        T* gr = grad + (size_t)row * cols;
        const float m = row_max[row], inv = 1.0f / stats[2 * row], gv = g[row];
        const long long t = target[row] - v0;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            float p = __expf(to_f<T>(xr[c]) - m) * inv;
            if (c == t) p -= 1.0f;
            gr[c] = from_f<T>(p * gv);
        }
    }
}

// Single-pass (online) statistics for bf16 logits with cols % 8 == 0: one sweep of 16-byte loads keeps a running
// (max, sum of exp relative to that max) per thread, merged across the CTA at the end.
//   row_max[row] = max_c x,   stats[row] = (sum_c exp(x - row_max), x[target - v0] (raw) if owned else 0)
// The caller turns these local quantities into global ones after the tensor-parallel all-reduce of the maxima.
__global__ void __launch_bounds__(256) ce_online_bf16_kernel(const __nv_bfloat16* __restrict__ x,
                                                             const long long* __restrict__ target,
                                                             float* __restrict__ row_max, float* __restrict__ stats,
                                                             int rows, int cols, int v0) {
    __shared__ float red_m[8], red_s[8];
    const int nvec = cols >> 3;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
        float m = -FLT_MAX, s = 0.f;
        for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
            const uint4 u = __ldg(xr + c);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
            float v[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[2 * i] = __uint_as_float(w[i] << 16);
                v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
            }
            float vm = v[0];
#pragma unroll
            for (int i = 1; i < 8; ++i) vm = fmaxf(vm, v[i]);
            if (vm > m) {
                s *= __expf(m - vm);
                m = vm;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) s += __expf(v[i] - m);
        }
        // merge (m, s) pairs: warp, then CTA
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
            const float nm = fmaxf(m, om);
            s = s * __expf(m - nm) + os * __expf(om - nm);
            m = nm;
        }
        __syncthreads();
        if (lane == 0) {
            red_m[warp] = m;
            red_s[warp] = s;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float gm = red_m[0], gs = red_s[0];
            for (int i = 1; i < (int)(blockDim.x >> 5); ++i) {
                const float nm = fmaxf(gm, red_m[i]);
                gs = gs * __expf(gm - nm) + red_s[i] * __expf(red_m[i] - nm);
                gm = nm;
            }
            const long long t = target[row] - v0;
            row_max[row] = gm;
            stats[2 * row] = gs;
            stats[2 * row + 1] = (t >= 0 && t < cols) ? __bfloat162float(x[(size_t)row * cols + t]) : 0.f;
        }
    }
}

// Vectorised backward for bf16, cols % 8 == 0 (same math as ce_bwd_kernel).
__global__ void __launch_bounds__(256) ce_bwd_bf16_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const long long* __restrict__ target,
                                                          const float* __restrict__ row_max,
                                                          const float* __restrict__ stats, const float* __restrict__ g,
                                                          __nv_bfloat16* __restrict__ grad, int rows, int cols, int v0) {
    const int nvec = cols >> 3;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
        uint4* gr = reinterpret_cast<uint4*>(grad + (size_t)row * cols);
        const float m = row_max[row], inv = 1.0f / stats[2 * row], gv = g[row];
        const long long t = target[row] - v0;
        for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
            const uint4 u = __ldg(xr + c);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
            float p[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                p[2 * i] = __expf(__uint_as_float(w[i] << 16) - m) * inv;
                p[2 * i + 1] = __expf(__uint_as_float(w[i] & 0xFFFF0000u) - m) * inv;
            }
            const long long d = t - (long long)c * 8;
            if (d >= 0 && d < 8) {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (i == (int)d) p[i] -= 1.0f;
            }
            uint4 o;
            uint32_t ow[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __nv_bfloat162 h2 = __floats2bfloat162_rn(p[2 * i] * gv, p[2 * i + 1] * gv);
                ow[i] = *reinterpret_cast<uint32_t*>(&h2);
            }
            o = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            gr[c] = o;
        }
    }
}

// ------------------------------------------------------------------ optimizers
template <typename OUT>
__global__ void __launch_bounds__(256) adam_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                                   const float* __restrict__ g, OUT* __restrict__ out, long long n,
                                                   float lr, float b1, float b2, float eps, float wd, float bc1,
                                                   float bc2, float gs, int adamw) {
    const float step = lr / bc1;
    const float isb2 = rsqrtf(bc2);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float gi = g[i] * gs;
        float pi = p[i];
        if (!adamw && wd != 0.f) gi += wd * pi;
        const float mi = b1 * m[i] + (1.f - b1) * gi;
        const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
        m[i] = mi;
        v[i] = vi;
        float upd = step * (mi / (sqrtf(vi) * isb2 + eps));
        if (adamw && wd != 0.f) upd += lr * wd * pi;
        pi -= upd;
        p[i] = pi;
        if (out) out[i] = from_f<OUT>(pi);
    }
}

// Adam(W) with block-wise 8-bit states: one CTA per block of 256 elements.  m is stored as round(127 m / absmax),
// v as round(255 sqrt(v / max)); a step de-quantises, applies the fp32 recurrences, re-quantises with the block's
// new maxima (two block reductions) and updates the fp32 parameter (+ optional 16-bit model copy).
template <typename OUT>
__global__ void __launch_bounds__(256) adam8bit_kernel(float* __restrict__ p, int8_t* __restrict__ qm,
                                                       uint8_t* __restrict__ qv, float* __restrict__ sm,
                                                       float* __restrict__ sv, const float* __restrict__ g,
                                                       OUT* __restrict__ out, long long n, float lr, float b1, float b2,
                                                       float eps, float wd, float bc1, float bc2, float gs, int adamw) {
    __shared__ float red[33];
    const long long blk = blockIdx.x;
    const long long i = blk * 256 + threadIdx.x;
    const bool live = i < n;
    float pi = live ? p[i] : 0.f;
    float gi = live ? g[i] * gs : 0.f;
    if (!adamw && wd != 0.f) gi += wd * pi;
    const float r = (float)qv[i] * (1.0f / 255.0f);
    float mi = (float)qm[i] * (sm[blk] * (1.0f / 127.0f));
    float vi = r * r * sv[blk];
    mi = b1 * mi + (1.f - b1) * gi;
    vi = b2 * vi + (1.f - b2) * gi * gi;
    const float amax = fmaxf(block_reduce<true>(fabsf(mi), red), 1e-30f);
    const float vmax = fmaxf(block_reduce<true>(vi, red), 1e-38f);
    qm[i] = (int8_t)__float2int_rn(mi / amax * 127.0f);
    qv[i] = (uint8_t)__float2int_rn(sqrtf(vi / vmax) * 255.0f);
    if (threadIdx.x == 0) {
        sm[blk] = amax;
        sv[blk] = vmax;
    }
    if (live) {
        float upd = (mi / bc1) / (sqrtf(vi / bc2) + eps);
        if (adamw && wd != 0.f) upd += wd * pi;
        pi -= lr * upd;
        p[i] = pi;
        if (out) out[i] = from_f<OUT>(pi);
    }
}

// The same update with one WARP per block of 256 elements: a lane owns 8 consecutive elements (16-byte accesses to the
// fp32 arrays, 8-byte accesses to the quantised states), the two maxima are warp shuffles, nothing goes through shared
// memory.  Needs 16-byte aligned p / g / out and 8-byte aligned qm / qv; the caller checks.
template <typename OUT>
__global__ void __launch_bounds__(256) adam8bit_warp_kernel(float* __restrict__ p, int8_t* __restrict__ qm,
                                                            uint8_t* __restrict__ qv, float* __restrict__ sm,
                                                            float* __restrict__ sv, const float* __restrict__ g,
                                                            OUT* __restrict__ out, long long n, long long nblocks,
                                                            float lr, float b1, float b2, float eps, float wd, float bc1,
                                                            float bc2, float gs, int adamw) {
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long blk = warp; blk < nblocks; blk += nwarps) {
        const long long i0 = blk * 256 + lane * 8;
        const bool full = i0 + 8 <= n;
        float pv[8], gv[8];
        if (full) {
            const float4 p0 = *reinterpret_cast<const float4*>(p + i0), p1 = *reinterpret_cast<const float4*>(p + i0 + 4);
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(g + i0));
            const float4 g1 = __ldg(reinterpret_cast<const float4*>(g + i0 + 4));
            pv[0] = p0.x, pv[1] = p0.y, pv[2] = p0.z, pv[3] = p0.w, pv[4] = p1.x, pv[5] = p1.y, pv[6] = p1.z, pv[7] = p1.w;
            gv[0] = g0.x, gv[1] = g0.y, gv[2] = g0.z, gv[3] = g0.w, gv[4] = g1.x, gv[5] = g1.y, gv[6] = g1.z, gv[7] = g1.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool live = i0 + j < n;
                pv[j] = live ? p[i0 + j] : 0.f;
                gv[j] = live ? g[i0 + j] : 0.f;
            }
        }
        const uint2 um = *reinterpret_cast<const uint2*>(qm + i0);          // the states are padded to whole blocks
        const uint2 uv = *reinterpret_cast<const uint2*>(qv + i0);
        const int8_t* m8 = reinterpret_cast<const int8_t*>(&um);
        const uint8_t* v8 = reinterpret_cast<const uint8_t*>(&uv);
        const float smb = sm[blk] * (1.0f / 127.0f), svb = sv[blk];
        float mi[8], vi[8], am = 0.f, vm = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float gi = gv[j] * gs;
            if (!adamw && wd != 0.f) gi += wd * pv[j];
            const float r = (float)v8[j] * (1.0f / 255.0f);
            mi[j] = b1 * ((float)m8[j] * smb) + (1.f - b1) * gi;
            vi[j] = b2 * (r * r * svb) + (1.f - b2) * gi * gi;
            am = fmaxf(am, fabsf(mi[j]));
            vm = fmaxf(vm, vi[j]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
            vm = fmaxf(vm, __shfl_xor_sync(0xffffffffu, vm, o));
        }
        const float amax = fmaxf(am, 1e-30f), vmax = fmaxf(vm, 1e-38f);
        uint2 om, ov;
        int8_t* om8 = reinterpret_cast<int8_t*>(&om);
        uint8_t* ov8 = reinterpret_cast<uint8_t*>(&ov);
        __align__(16) OUT o16[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            om8[j] = (int8_t)__float2int_rn(mi[j] / amax * 127.0f);
            ov8[j] = (uint8_t)__float2int_rn(sqrtf(vi[j] / vmax) * 255.0f);
            float upd = (mi[j] / bc1) / (sqrtf(vi[j] / bc2) + eps);
            if (adamw && wd != 0.f) upd += wd * pv[j];
            pv[j] -= lr * upd;
            o16[j] = from_f<OUT>(pv[j]);
        }
        *reinterpret_cast<uint2*>(qm + i0) = om;
        *reinterpret_cast<uint2*>(qv + i0) = ov;
        if (lane == 0) {
            sm[blk] = amax;
            sv[blk] = vmax;
        }
        if (full) {
            *reinterpret_cast<float4*>(p + i0) = make_float4(pv[0], pv[1], pv[2], pv[3]);
            *reinterpret_cast<float4*>(p + i0 + 4) = make_float4(pv[4], pv[5], pv[6], pv[7]);
            if (out) {
                constexpr int NV = 8 * (int)sizeof(OUT) / 16;
#pragma unroll
                for (int q = 0; q < NV; ++q)
                    reinterpret_cast<uint4*>(out + i0)[q] = reinterpret_cast<const uint4*>(o16)[q];
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (i0 + j < n) {
                    p[i0 + j] = pv[j];
                    if (out) out[i0 + j] = o16[j];
                }
        }
    }
}

template <typename OUT>
__global__ void __launch_bounds__(256) lion_kernel(float* __restrict__ p, float* __restrict__ m,
                                                   const float* __restrict__ g, OUT* __restrict__ out, long long n,
                                                   float lr, float b1, float b2, float wd, float gs) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float gi = g[i] * gs;
        float pi = p[i] * (1.f - lr * wd);
        const float mi = m[i];
        const float c = mi * b1 + gi * (1.f - b1);
        pi -= lr * ((c > 0.f) ? 1.f : (c < 0.f ? -1.f : 0.f));
        m[i] = mi * b2 + gi * (1.f - b2);
        p[i] = pi;
        if (out) out[i] = from_f<OUT>(pi);
    }
}

// 16-byte loads over the aligned body (two independent accumulators per thread), scalar loads for the ragged
// head / tail; one atomic per CTA.
__global__ void __launch_bounds__(256) sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
    __shared__ float red[33];
    const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * blockDim.x;
    long long head = (4 - ((reinterpret_cast<uintptr_t>(x) >> 2) & 3)) & 3;      // floats before a 16-byte boundary
    if (head > n) head = n;
    const long long nvec = (n - head) >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x + head);
    float s0 = 0.f, s1 = 0.f;
    for (long long i = tid; i < nvec; i += nthreads) {
        const float4 v = x4[i];
        s0 += v.x * v.x + v.y * v.y;
        s1 += v.z * v.z + v.w * v.w;
    }
    for (long long i = tid; i < head; i += nthreads) s0 += x[i] * x[i];
    for (long long i = head + (nvec << 2) + tid; i < n; i += nthreads) s1 += x[i] * x[i];
    const float s = block_reduce<false>(s0 + s1, red);
    if (threadIdx.x == 0) atomicAdd(out, s);
}

int grid_for(long long n, int per_sm = 8) {
    long long b = (n + 255) / 256;
    const long long cap = (long long)neox_sm_count() * per_sm;
    return (int)(b < cap ? (b > 0 ? b : 1) : cap);
}
int row_grid(long long rows) {
    const long long cap = (long long)neox_sm_count() * 8;
    return (int)(rows < cap ? (rows > 0 ? rows : 1) : cap);
}

#define DISPATCH(dtype, CALL)                          \
    do {                                               \
        if (dtype == 0) { using T = __nv_bfloat16; CALL; } \
        else if (dtype == 1) { using T = float; CALL; }    \
        else { using T = __half; CALL; }                   \
    } while (0)

// 16-bit types only (dtype 0 = bf16, 2 = fp16)
#define DISPATCH16(dtype, CALL)                            \
    do {                                                   \
        if (dtype == 0) { using T = __nv_bfloat16; CALL; } \
        else { using T = __half; CALL; }                   \
    } while (0)

}  // namespace

extern "C" {

int neox_softmax_fwd(const void* x, const void* mask, void* y, long long rows, int sq, int sk, int heads,
                     int mask_batches, float scale, int causal, int dtype, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype != 1 && sk % 8 == 0 && sk <= 2048 &&
        ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(mask) & 7) == 0) {
        // the 8-chunk variant needs ~160 registers: 128-thread CTAs keep 12 warps per SM resident instead of 8
        const int threads = sk <= 1024 ? 256 : 128;
        const long long ctas = (rows + threads / 32 - 1) / (threads / 32);      // one pass: a warp per row
        const unsigned grid = (unsigned)(ctas < 2147483647LL ? ctas : 2147483647LL);
#define NEOX_SOFTMAX_FWD_WARP(NC)                                                                                      \
    DISPATCH16(dtype, (softmax_fwd_warp_kernel<T, NC><<<grid, threads, 0, st>>>(                                           \
                          (const T*)x, (const uint8_t*)mask, (T*)y, rows, sq, sk, heads, mask_batches, scale, causal)))
        if (sk <= 256) NEOX_SOFTMAX_FWD_WARP(1);
        else if (sk <= 512) NEOX_SOFTMAX_FWD_WARP(2);
        else if (sk <= 1024) NEOX_SOFTMAX_FWD_WARP(4);
        else NEOX_SOFTMAX_FWD_WARP(8);
#undef NEOX_SOFTMAX_FWD_WARP
        return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
    }
    const int threads = sk <= 512 ? 64 : 256;
    DISPATCH(dtype, (softmax_fwd_kernel<T><<<row_grid(rows), threads, 0, st>>>(
                        (const T*)x, (const uint8_t*)mask, (T*)y, rows, sq, sk, heads, mask_batches, scale, causal)));
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
int neox_softmax_bwd(const void* g, const void* y, void* dx, long long rows, int sk, float scale, int dtype,
                     void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype != 1 && sk % 8 == 0 && sk <= 2048 &&
        ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0) {
        const int threads = sk <= 1024 ? 256 : 128;
        const long long ctas = (rows + threads / 32 - 1) / (threads / 32);      // one pass: a warp per row
        const unsigned grid = (unsigned)(ctas < 2147483647LL ? ctas : 2147483647LL);
#define NEOX_SOFTMAX_BWD_WARP(NC)                                                                                      \
    DISPATCH16(dtype, (softmax_bwd_warp_kernel<T, NC><<<grid, threads, 0, st>>>((const T*)g, (const T*)y, (T*)dx, rows,   \
                                                                                sk, scale)))
        if (sk <= 256) NEOX_SOFTMAX_BWD_WARP(1);
        else if (sk <= 512) NEOX_SOFTMAX_BWD_WARP(2);
        else if (sk <= 1024) NEOX_SOFTMAX_BWD_WARP(4);
        else NEOX_SOFTMAX_BWD_WARP(8);
#undef NEOX_SOFTMAX_BWD_WARP
        return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
    }
    const int threads = sk <= 512 ? 64 : 256;
    DISPATCH(dtype, (softmax_bwd_kernel<T><<<row_grid(rows), threads, 0, st>>>((const T*)g, (const T*)y, (T*)dx, rows,
                                                                              sk, scale)));
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
int neox_rope(const void* x, void* out, const float* cs, const float* sn, int s, int b, int h, int d, int rot,
              long long ss, long long sb, long long sh, int inverse, int dtype, void* stream) {
    const long long total = (long long)s * b * h * d;
    if (total <= 0) return 0;
    if (rot % 2 || rot > d) return NEOX_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    for (int bytes = 16; bytes >= 8; bytes >>= 1) {            // widest vector access the shape allows
        const int vec = bytes / (dtype == 1 ? 4 : 2);
        const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) |
                               reinterpret_cast<uintptr_t>(cs) | reinterpret_cast<uintptr_t>(sn)) &
                              (uintptr_t)(bytes - 1)) == 0;
        if (!aligned || rot == 0 || (rot / 2) % vec || (d - rot) % vec || d % vec || ss % vec || sb % vec || sh % vec)
            continue;
        const long long items = (long long)s * b * h * ((rot / 2 + d - rot) / vec);
        if (bytes == 16) {
            DISPATCH(dtype, (rope_vec_kernel<T, 16><<<grid_for(items, 16), 256, 0, st>>>(
                                (const T*)x, (T*)out, cs, sn, s, b, h, d, rot, ss, sb, sh, inverse)));
        } else {
            DISPATCH(dtype, (rope_vec_kernel<T, 8><<<grid_for(items, 16), 256, 0, st>>>(
                                (const T*)x, (T*)out, cs, sn, s, b, h, d, rot, ss, sb, sh, inverse)));
        }
        return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
    }
    DISPATCH(dtype, (rope_kernel<T><<<grid_for(total, 16), 256, 0, st>>>((const T*)x, (T*)out, cs, sn, s, b, h, d, rot,
                                                                         ss, sb, sh, inverse)));
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
int neox_rope_qk_inplace(void* q, void* k, const float* cs, const float* sn, int s, int b, int hq, int hk, int rot,
                         long long q_ss, long long q_sb, long long q_sh, long long k_ss, long long k_sb, long long k_sh,
                         int inverse, int dtype, void* stream) {
    const long long total = (long long)s * b * (hq + hk) * (rot / 2);
    if (total <= 0) return 0;
    if (rot % 2) return NEOX_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dtype, (rope_qk_inplace_kernel<T><<<grid_for(total, 16), 256, 0, st>>>(
                        (T*)q, (T*)k, cs, sn, s, b, hq, hk, rot, q_ss, q_sb, q_sh, k_ss, k_sb, k_sh, inverse)));
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
int neox_row_max(const void* x, float* out, int rows, int cols, int dtype, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dtype, (row_max_kernel<T><<<row_grid(rows), 256, 0, st>>>((const T*)x, out, rows, cols)));
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
int neox_ce_stats(const void* x, const long long* target, const float* row_max, float* stats, int rows, int cols,
                  int v0, int dtype, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dtype, (ce_stats_kernel<T><<<row_grid(rows), 256, 0, st>>>((const T*)x, target, row_max, stats, rows,
                                                                       cols, v0)));
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
// bf16 only, cols % 8 == 0: local row maximum, sum of exp relative to it, and the raw target logit in one pass.
int neox_ce_online_bf16(const void* x, const long long* target, float* row_max, float* stats, int rows, int cols,
                        int v0, void* stream) {
    if (rows <= 0) return 0;
    if (cols % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return NEOX_ERR_ALIGN;
    ce_online_bf16_kernel<<<row_grid(rows), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, target, row_max,
                                                                            stats, rows, cols, v0);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
int neox_ce_bwd(const void* x, const long long* target, const float* row_max, const float* stats, const float* g,
                void* grad, int rows, int cols, int v0, int dtype, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == 0 && cols % 8 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) &&
        !(reinterpret_cast<uintptr_t>(grad) & 15)) {
        ce_bwd_bf16_kernel<<<row_grid(rows), 256, 0, st>>>((const __nv_bfloat16*)x, target, row_max, stats, g,
                                                          (__nv_bfloat16*)grad, rows, cols, v0);
        return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
    }
    DISPATCH(dtype, (ce_bwd_kernel<T><<<row_grid(rows), 256, 0, st>>>((const T*)x, target, row_max, stats, g, (T*)grad,
                                                                     rows, cols, v0)));
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
int neox_adam_step(float* p, float* m, float* v, const float* g, void* out, int out_dtype, long long n, float lr,
                   float b1, float b2, float eps, float wd, float bc1, float bc2, float gs, int adamw, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int grid = grid_for(n, 16);
    if (!out || out_dtype == 1)
        adam_kernel<float><<<grid, 256, 0, st>>>(p, m, v, g, (float*)out, n, lr, b1, b2, eps, wd, bc1, bc2, gs, adamw);
    else if (out_dtype == 0)
        adam_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, m, v, g, (__nv_bfloat16*)out, n, lr, b1, b2, eps, wd, bc1,
                                                          bc2, gs, adamw);
    else
        adam_kernel<__half><<<grid, 256, 0, st>>>(p, m, v, g, (__half*)out, n, lr, b1, b2, eps, wd, bc1, bc2, gs, adamw);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
// qm / qv hold ceil(n / 256) * 256 quantised states, sm / sv one fp32 scale per block of 256.
int neox_adam8bit_step(float* p, void* qm, void* qv, float* sm, float* sv, const float* g, void* out, int out_dtype,
                       long long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, float gs,
                       int adamw, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const long long blocks = (n + 255) / 256;
    if (blocks > 2147483647LL) return NEOX_ERR_TOO_LARGE;
    const unsigned grid = (unsigned)blocks;
    int8_t* m8 = static_cast<int8_t*>(qm);
    uint8_t* v8 = static_cast<uint8_t*>(qv);
    if (((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
        ((reinterpret_cast<uintptr_t>(qm) | reinterpret_cast<uintptr_t>(qv)) & 7) == 0) {
        const unsigned wgrid = (unsigned)((blocks + 7) / 8);             // one warp per block of 256 elements
        if (!out || out_dtype == 1)
            adam8bit_warp_kernel<float><<<wgrid, 256, 0, st>>>(p, m8, v8, sm, sv, g, (float*)out, n, blocks, lr, b1, b2,
                                                               eps, wd, bc1, bc2, gs, adamw);
        else if (out_dtype == 0)
            adam8bit_warp_kernel<__nv_bfloat16><<<wgrid, 256, 0, st>>>(p, m8, v8, sm, sv, g, (__nv_bfloat16*)out, n, blocks,
                                                                       lr, b1, b2, eps, wd, bc1, bc2, gs, adamw);
        else
            adam8bit_warp_kernel<__half><<<wgrid, 256, 0, st>>>(p, m8, v8, sm, sv, g, (__half*)out, n, blocks, lr, b1, b2,
                                                                eps, wd, bc1, bc2, gs, adamw);
        return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
    }
    if (!out || out_dtype == 1)
        adam8bit_kernel<float><<<grid, 256, 0, st>>>(p, m8, v8, sm, sv, g, (float*)out, n, lr, b1, b2, eps, wd, bc1, bc2,
                                                     gs, adamw);
    else if (out_dtype == 0)
        adam8bit_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, m8, v8, sm, sv, g, (__nv_bfloat16*)out, n, lr, b1, b2,
                                                             eps, wd, bc1, bc2, gs, adamw);
    else
        adam8bit_kernel<__half><<<grid, 256, 0, st>>>(p, m8, v8, sm, sv, g, (__half*)out, n, lr, b1, b2, eps, wd, bc1,
                                                      bc2, gs, adamw);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
int neox_lion_step(float* p, float* m, const float* g, void* out, int out_dtype, long long n, float lr, float b1,
                   float b2, float wd, float gs, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int grid = grid_for(n, 16);
    if (!out || out_dtype == 1) lion_kernel<float><<<grid, 256, 0, st>>>(p, m, g, (float*)out, n, lr, b1, b2, wd, gs);
    else if (out_dtype == 0)
        lion_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, m, g, (__nv_bfloat16*)out, n, lr, b1, b2, wd, gs);
    else lion_kernel<__half><<<grid, 256, 0, st>>>(p, m, g, (__half*)out, n, lr, b1, b2, wd, gs);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
// out += sum(x^2); the caller zeroes `out` first.
int neox_sumsq_f32(const float* x, long long n, float* out, void* stream) {
    if (n <= 0) return 0;
    sumsq_kernel<<<grid_for((n + 3) / 4, 8), 256, 0, (cudaStream_t)stream>>>(x, n, out);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

}  // extern "C"
