// Bandwidth-bound row kernels: LayerNorm / RMSNorm forward+backward and the fused bias / activation /
// residual element-wise ops.  One CTA per row (grid-stride over rows), 16-byte vector accesses, the
// row is held in registers between the statistics pass and the normalisation pass so every input
// byte is read from HBM exactly once.  fp32 statistics for all storage dtypes (bf16 / fp16 / fp32).
//
// Replaces apex fused_layer_norm_cuda / FastLayerNormFN (megatron/model/fused_layer_norm.py:123-153),
// the TorchScript bias_gelu (activations.py:78-112), the gated-activation glue (transformer.py:190-206)
// and bias_dropout_add (fused_bias_dropout.py:28-55) of the reference.
#include "neox_b200.h"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace {

constexpr int MAXV = 4;  // vectors of 8 elements cached per thread

template <typename T>
struct Vec8;
template <>
struct Vec8<__nv_bfloat16> {
    typedef uint4 Raw;   // 8 packed elements: what a prefetch keeps in registers
    static __device__ __forceinline__ Raw raw_load(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
    static __device__ __forceinline__ void unpack(const Raw& u, float (&v)[8]) {
        uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        uint4 u = *reinterpret_cast<const uint4*>(p);
        uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <>
struct Vec8<__half> {
    typedef uint4 Raw;
    static __device__ __forceinline__ Raw raw_load(const __half* p) { return *reinterpret_cast<const uint4*>(p); }
    static __device__ __forceinline__ void unpack(const Raw& u, float (&v)[8]) {
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
        uint4 u = *reinterpret_cast<const uint4*>(p);
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
        uint4 u;
        __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = u;
    }
};
template <>
struct Vec8<float> {
    struct Raw {
        float4 a, b;
    };
    static __device__ __forceinline__ Raw raw_load(const float* p) {
        Raw r;
        r.a = *reinterpret_cast<const float4*>(p);
        r.b = *reinterpret_cast<const float4*>(p + 4);
        return r;
    }
    static __device__ __forceinline__ void unpack(const Raw& r, float (&v)[8]) {
        v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
    }
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over the CTA; every thread receives the result.  `red` is a 33-float shared scratch.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
    if (warp == 0) {
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ void block_sum2(float& a, float& b, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    __syncthreads();
    if (lane == 0) {
        red[warp] = a;
        red[33 + warp] = b;
    }
    __syncthreads();
    float ta = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
    float tb = (threadIdx.x < nw) ? red[33 + threadIdx.x] : 0.f;
    if (warp == 0) {
        ta = warp_sum(ta);
        tb = warp_sum(tb);
        if (lane == 0) {
            red[32] = ta;
            red[65] = tb;
        }
    }
    __syncthreads();
    a = red[32];
    b = red[65];
}

// ------------------------------------------------------------------ LayerNorm
// RMS == false: y = (x - mean) * rstd * gamma + beta,   stat0 = mean, stat1 = rstd
// RMS == true : y = x * rinv * gamma + beta with rinv = 1 / (sqrt(mean(x^2)) + eps),  stat1 = rinv
template <typename T, bool RMS>
__global__ void __launch_bounds__(256) norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                       const T* __restrict__ beta, T* __restrict__ y,
                                                       float* __restrict__ stat0, float* __restrict__ stat1,
                                                       int rows, int cols, float eps) {
    __shared__ float red[66];
    const int nvec = cols >> 3;
    const bool cached = nvec <= MAXV * (int)blockDim.x;
    // Cached path: the next row's (packed) data is requested before this row's reductions start, so two rows per
    // CTA are in flight and the loads overlap the block-wide sums.
    typename Vec8<T>::Raw nxt[MAXV];
    auto fetch = [&](int r) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int c = threadIdx.x + j * blockDim.x;
            if (c < nvec) nxt[j] = Vec8<T>::raw_load(x + (size_t)r * cols + c * 8);
        }
    };
    if (cached && (int)blockIdx.x < rows) fetch(blockIdx.x);
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + (size_t)row * cols;
        T* yr = y + (size_t)row * cols;
        float v[MAXV][8];
        float s = 0.f;
        if (cached) {
#pragma unroll
            for (int j = 0; j < MAXV; ++j) {
                const int c = threadIdx.x + j * blockDim.x;
                if (c < nvec) {
                    Vec8<T>::unpack(nxt[j], v[j]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) s += RMS ? v[j][i] * v[j][i] : v[j][i];
                }
            }
            if (row + (int)gridDim.x < rows) fetch(row + gridDim.x);
        } else {
            for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
                float t[8];
                Vec8<T>::load(xr + c * 8, t);
#pragma unroll
                for (int i = 0; i < 8; ++i) s += RMS ? t[i] * t[i] : t[i];
            }
        }
        s = block_sum(s, red);
        float mean = 0.f, scale;
        if (RMS) {
            scale = 1.0f / (sqrtf(s / cols) + eps);
        } else {
            mean = s / cols;
            float q = 0.f;
            if (cached) {
#pragma unroll
                for (int j = 0; j < MAXV; ++j) {
                    const int c = threadIdx.x + j * blockDim.x;
                    if (c < nvec) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float d = v[j][i] - mean;
                            q += d * d;
                        }
                    }
                }
            } else {
                for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
                    float t[8];
                    Vec8<T>::load(xr + c * 8, t);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float d = t[i] - mean;
                        q += d * d;
                    }
                }
            }
            q = block_sum(q, red);
            scale = rsqrtf(q / cols + eps);
        }
        if (threadIdx.x == 0) {
            if (stat0) stat0[row] = mean;
            stat1[row] = scale;
        }
        auto emit = [&](int c, float (&t)[8]) {
            float g[8], b[8], o[8];
            Vec8<T>::load(gamma + c * 8, g);
            if (beta) Vec8<T>::load(beta + c * 8, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = (t[i] - mean) * scale * g[i] + (beta ? b[i] : 0.f);
            Vec8<T>::store(yr + c * 8, o);
        };
        if (cached) {
#pragma unroll
            for (int j = 0; j < MAXV; ++j) {
                const int c = threadIdx.x + j * blockDim.x;
                if (c < nvec) emit(c, v[j]);
            }
        } else {
            for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
                float t[8];
                Vec8<T>::load(xr + c * 8, t);
                emit(c, t);
            }
        }
    }
}

// Backward.  Column sums (dgamma, dbeta) are accumulated per CTA in registers (cached path) or in
// global partial rows (generic path) and written to partial[blockIdx.x][cols]; a second kernel
// reduces the partial rows.  partial layout: [2][nblk][cols] fp32.
template <typename T, bool RMS>
__global__ void __launch_bounds__(256) norm_bwd_kernel(const T* __restrict__ g, const T* __restrict__ x,
                                                       const T* __restrict__ gamma, const float* __restrict__ stat0,
                                                       const float* __restrict__ stat1, T* dx,
                                                       float* __restrict__ partial, int rows, int cols, float eps,
                                                       const T* add) {
    // add (optional, may alias dx): dx = gradient through the norm + add -- lets the caller fold the other
    // gradient contributions of the norm's input (residual path, a sibling norm) into this pass
    __shared__ float red[66];
    const int nvec = cols >> 3;
    const bool cached = nvec <= MAXV * (int)blockDim.x;
    float* pg = partial + (size_t)blockIdx.x * cols;
    float* pb = partial + ((size_t)gridDim.x + blockIdx.x) * cols;
    float ag[MAXV][8], ab[MAXV][8];
    if (cached) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i) ag[j][i] = ab[j][i] = 0.f;
    } else {
        for (int c = threadIdx.x; c < cols; c += blockDim.x) pg[c] = pb[c] = 0.f;
    }
    typename Vec8<T>::Raw nx[MAXV], ng[MAXV];      // next row, packed (see the forward kernel)
    float n_mean = 0.f, n_sc = 0.f;                 // ... and its saved statistics
    auto fetch = [&](int r) {
        n_mean = RMS ? 0.f : stat0[r];
        n_sc = stat1[r];
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int c = threadIdx.x + j * blockDim.x;
            if (c < nvec) {
                nx[j] = Vec8<T>::raw_load(x + (size_t)r * cols + c * 8);
                ng[j] = Vec8<T>::raw_load(g + (size_t)r * cols + c * 8);
            }
        }
    };
    if (cached && (int)blockIdx.x < rows) fetch(blockIdx.x);
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + (size_t)row * cols;
        const T* gr = g + (size_t)row * cols;
        T* dr = dx + (size_t)row * cols;
        float mean, sc;
        float s1 = 0.f, s2 = 0.f;
        float xv[MAXV][8], gv[MAXV][8];
        if (cached) {
            mean = n_mean;
            sc = n_sc;
#pragma unroll
            for (int j = 0; j < MAXV; ++j) {
                const int c = threadIdx.x + j * blockDim.x;
                if (c < nvec) {
                    Vec8<T>::unpack(nx[j], xv[j]);
                    Vec8<T>::unpack(ng[j], gv[j]);
                }
            }
            if (row + (int)gridDim.x < rows) fetch(row + gridDim.x);
#pragma unroll
            for (int j = 0; j < MAXV; ++j) {
                const int c = threadIdx.x + j * blockDim.x;
                if (c < nvec) {
                    float gm[8];
                    Vec8<T>::load(gamma + c * 8, gm);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float xh = RMS ? xv[j][i] : (xv[j][i] - mean) * sc;
                        const float gg = gv[j][i] * gm[i];
                        s1 += gg;
                        s2 += gg * xh;
                        ag[j][i] += gv[j][i] * (RMS ? xv[j][i] * sc : xh);
                        ab[j][i] += gv[j][i];
                        gv[j][i] = gg;   // keep g*gamma
                        xv[j][i] = xh;   // keep xhat (LN) or x (RMS)
                    }
                }
            }
        } else {
            mean = RMS ? 0.f : stat0[row];
            sc = stat1[row];
            for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
                float xt[8], gt[8], gm[8];
                Vec8<T>::load(xr + c * 8, xt);
                Vec8<T>::load(gr + c * 8, gt);
                Vec8<T>::load(gamma + c * 8, gm);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float xh = RMS ? xt[i] : (xt[i] - mean) * sc;
                    const float gg = gt[i] * gm[i];
                    s1 += gg;
                    s2 += gg * xh;
                    pg[c * 8 + i] += gt[i] * (RMS ? xt[i] * sc : xh);
                    pb[c * 8 + i] += gt[i];
                }
            }
        }
        block_sum2(s1, s2, red);
        // LN : dx = sc * (gg - s1/n - xhat * s2/n)
        // RMS: y = x*sc*gamma, sc = 1/(r+eps), r = sqrt(mean x^2) -> dx = gg*sc - x * s2 * sc^2 / (n * r)
        float k1, k2;
        if (RMS) {
            const float r = 1.0f / sc - eps;
            k1 = 0.f;
            k2 = (r > 0.f) ? s2 * sc * sc / (cols * r) : 0.f;
        } else {
            k1 = s1 / cols;
            k2 = s2 / cols;
        }
        auto emit = [&](int c, const float (&xh)[8], const float (&gg)[8]) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = RMS ? gg[i] * sc - xh[i] * k2 : sc * (gg[i] - k1 - xh[i] * k2);
            if (add) {
                float a8[8];
                Vec8<T>::load(add + (size_t)row * cols + c * 8, a8);
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] += a8[i];
            }
            Vec8<T>::store(dr + c * 8, o);
        };
        if (cached) {
#pragma unroll
            for (int j = 0; j < MAXV; ++j) {
                const int c = threadIdx.x + j * blockDim.x;
                if (c < nvec) emit(c, xv[j], gv[j]);
            }
        } else {
            for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
                float xt[8], gt[8], gm[8], xh[8], gg[8];
                Vec8<T>::load(xr + c * 8, xt);
                Vec8<T>::load(gr + c * 8, gt);
                Vec8<T>::load(gamma + c * 8, gm);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    xh[i] = RMS ? xt[i] : (xt[i] - mean) * sc;
                    gg[i] = gt[i] * gm[i];
                }
                emit(c, xh, gg);
            }
        }
    }
    if (cached) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int c = threadIdx.x + j * blockDim.x;
            if (c < nvec) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    pg[c * 8 + i] = ag[j][i];
                    pb[c * 8 + i] = ab[j][i];
                }
            }
        }
    }
}

// out0[c] = sum_r partial[r][c], out1[c] = sum_r partial[nblk + r][c].  A CTA owns 32 columns; its 8 warps take
// every 8th partial row (coalesced 128-byte reads), then the 8 row lanes are added in a fixed order -- about 190 CTAs
// for 6144 columns instead of the 24 a thread-per-column loop gave, which was latency-bound on ~600 serial loads.
__global__ void __launch_bounds__(256) colreduce_kernel(const float* __restrict__ partial, float* __restrict__ out0,
                                                        float* __restrict__ out1, int nblk, int cols) {
    __shared__ float sa[8][33], sb[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + tx;
    float a = 0.f, b = 0.f;
    if (c < cols) {
        for (int r = ty; r < nblk; r += 8) {
            a += partial[(size_t)r * cols + c];
            b += partial[((size_t)nblk + r) * cols + c];
        }
    }
    sa[ty][tx] = a;
    sb[ty][tx] = b;
    __syncthreads();
    if (ty == 0 && c < cols) {
        float ta = 0.f, tb = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            ta += sa[j][tx];
            tb += sb[j][tx];
        }
        out0[c] = ta;
        if (out1) out1[c] = tb;
    }
}

int pick_threads(int cols) {
    int t = 32;
    while (t < 256 && t * 8 < cols) t <<= 1;
    return t;
}

template <bool RMS>
int launch_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* s0, float* s1, int rows,
                    int cols, float eps, int dtype, cudaStream_t st) {
    if (cols % 8) return NEOX_ERR_SHAPE;
    if (rows <= 0) return 0;
    const int threads = pick_threads(cols);
    const int grid = rows < neox_sm_count() * 8 ? rows : neox_sm_count() * 8;
#define LAUNCH(T)                                                                                                   \
    norm_fwd_kernel<T, RMS><<<grid, threads, 0, st>>>((const T*)x, (const T*)gamma, (const T*)beta, (T*)y, s0, s1, \
                                                      rows, cols, eps)
    if (dtype == 0) LAUNCH(__nv_bfloat16);
    else if (dtype == 1) LAUNCH(float);
    else LAUNCH(__half);
#undef LAUNCH
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

template <bool RMS>
int launch_norm_bwd(const void* g, const void* x, const void* gamma, const float* s0, const float* s1, void* dx,
                    float* d0, float* d1, float* ws, int rows, int cols, float eps, int dtype, cudaStream_t st,
                    const void* add = nullptr) {
    if (cols % 8) return NEOX_ERR_SHAPE;
    if (rows <= 0) return 0;
    const int threads = pick_threads(cols);
    const int nblk = neox_norm_bwd_blocks(rows);
#define LAUNCH(T)                                                                                                    \
    norm_bwd_kernel<T, RMS><<<nblk, threads, 0, st>>>((const T*)g, (const T*)x, (const T*)gamma, s0, s1, (T*)dx, ws, \
                                                      rows, cols, eps, (const T*)add)
    if (dtype == 0) LAUNCH(__nv_bfloat16);
    else if (dtype == 1) LAUNCH(float);
    else LAUNCH(__half);
#undef LAUNCH
    colreduce_kernel<<<(cols + 31) / 32, 256, 0, st>>>(ws, d0, d1, nblk, cols);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// ------------------------------------------------------------------ element-wise
__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float gelu_f(float x) {
    return 0.5f * x * (1.0f + tanh_fast(0.7978845608028654f * x * (1.0f + 0.044715f * x * x)));
}
__device__ __forceinline__ float dgelu_f(float x) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    const float t = tanh_fast(k0 * x * (1.0f + k1 * x * x));
    return 0.5f * x * ((1.0f - t * t) * (k0 + 3.0f * k0 * k1 * x * x)) + 0.5f * (1.0f + t);
}
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + __expf(-x)); }

// mode 0: out = g * gelu'(a)                    (a = pre-activation)
// mode 1: out = gelu(a + bias)                  (bias per column, may be null)
// mode 2: out = g * gelu'(a + bias)
// mode 3: out = a + bias + r                    (bias + residual add)
template <typename T, int MODE>
__global__ void __launch_bounds__(256) ew_kernel(const T* __restrict__ a, const T* __restrict__ b2,
                                                 const T* __restrict__ bias, T* __restrict__ out, long long nvec,
                                                 int colvec) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
        float va[8], vb[8], bb[8], o[8];
        Vec8<T>::load(a + i * 8, va);
        if (MODE == 0 || MODE == 2 || MODE == 3) Vec8<T>::load(b2 + i * 8, vb);
        const bool hb = (MODE != 0) && bias != nullptr;
        if (hb) Vec8<T>::load(bias + (i % colvec) * 8, bb);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float xa = va[k] + (hb ? bb[k] : 0.f);
            if (MODE == 0) o[k] = vb[k] * dgelu_f(va[k]);
            else if (MODE == 1) o[k] = gelu_f(xa);
            else if (MODE == 2) o[k] = vb[k] * dgelu_f(xa);
            else o[k] = xa + vb[k];
        }
        Vec8<T>::store(out + i * 8, o);
    }
}

// gated activations: x = [up | gate] halves of the last dim; out = act(gate) * up
// kind 0 geglu, 1 swiglu, 2 reglu, 3 bilinear, 4 glu(sigmoid)
__device__ __forceinline__ float gate_act(int kind, float t) {
    switch (kind) {
        case 0: return gelu_f(t);
        case 1: return t * sigmoid_f(t);
        case 2: return fmaxf(t, 0.f);
        case 3: return t;
        default: return sigmoid_f(t);
    }
}
__device__ __forceinline__ float gate_dact(int kind, float t) {
    switch (kind) {
        case 0: return dgelu_f(t);
        case 1: { const float s = sigmoid_f(t); return s * (1.0f + t * (1.0f - s)); }
        case 2: return t > 0.f ? 1.f : 0.f;
        case 3: return 1.f;
        default: { const float s = sigmoid_f(t); return s * (1.0f - s); }
    }
}
template <typename T>
__global__ void __launch_bounds__(256) gated_fwd_kernel(const T* __restrict__ x, T* __restrict__ out, long long rows,
                                                        int cols, int kind) {
    const int cv = cols >> 3;
    const long long n = rows * cv;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cv;
        const int c = (int)(i % cv) * 8;
        float up[8], gt[8], o[8];
        Vec8<T>::load(x + r * 2 * cols + c, up);
        Vec8<T>::load(x + r * 2 * cols + cols + c, gt);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = gate_act(kind, gt[k]) * up[k];
        Vec8<T>::store(out + r * cols + c, o);
    }
}
template <typename T>
__global__ void __launch_bounds__(256) gated_bwd_kernel(const T* __restrict__ g, const T* __restrict__ x,
                                                        T* __restrict__ dx, long long rows, int cols, int kind) {
    const int cv = cols >> 3;
    const long long n = rows * cv;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cv;
        const int c = (int)(i % cv) * 8;
        float up[8], gt[8], gg[8], du[8], dg[8];
        Vec8<T>::load(x + r * 2 * cols + c, up);
        Vec8<T>::load(x + r * 2 * cols + cols + c, gt);
        Vec8<T>::load(g + r * cols + c, gg);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            du[k] = gg[k] * gate_act(kind, gt[k]);
            dg[k] = gg[k] * up[k] * gate_dact(kind, gt[k]);
        }
        Vec8<T>::store(dx + r * 2 * cols + c, du);
        Vec8<T>::store(dx + r * 2 * cols + cols + c, dg);
    }
}

// ---------------------------------------------------------------- bias + dropout + residual add (training)
// Philox-4x32-10 counter-based generator (Salmon et al., SC'11): the mask of element i is a pure function of
// (seed, offset, i), so the backward kernel regenerates it instead of reading a stored mask, and a recomputed
// forward (activation checkpointing) reproduces it from the replayed generator state.
__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
        c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
        k.x += 0x9E3779B9u;
        k.y += 0xBB67AE85u;
    }
    return c;
}

// keep[k] for the 8 elements of vector i: two Philox blocks, element kept when its 32 random bits >= threshold
__device__ __forceinline__ void dropout_keep8(unsigned long long seed, unsigned long long offset, long long i,
                                              uint32_t threshold, bool (&keep)[8]) {
    const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
    const unsigned long long c0 = offset + 2ULL * (unsigned long long)i;
    const uint4 a = philox4x32_10(make_uint4((uint32_t)c0, (uint32_t)(c0 >> 32), 0u, 0u), key);
    const uint4 b = philox4x32_10(make_uint4((uint32_t)(c0 + 1), (uint32_t)((c0 + 1) >> 32), 0u, 0u), key);
    const uint32_t r[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) keep[k] = r[k] >= threshold;
}

// out = residual + dropout(x + bias)        (residual may be null: plain dropout of x + bias)
template <typename T>
__global__ void __launch_bounds__(256) bias_dropout_add_kernel(const T* __restrict__ x, const T* __restrict__ bias,
                                                               const T* __restrict__ residual, T* __restrict__ out,
                                                               long long nvec, int colvec, uint32_t threshold,
                                                               float scale, unsigned long long seed,
                                                               unsigned long long offset) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
        float v[8], bb[8], rr[8], o[8];
        bool keep[8];
        Vec8<T>::load(x + i * 8, v);
        if (bias) Vec8<T>::load(bias + (i % colvec) * 8, bb);
        if (residual) Vec8<T>::load(residual + i * 8, rr);
        dropout_keep8(seed, offset, i, threshold, keep);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float t = v[k] + (bias ? bb[k] : 0.f);
            o[k] = (keep[k] ? t * scale : 0.f) + (residual ? rr[k] : 0.f);
        }
        Vec8<T>::store(out + i * 8, o);
    }
}

// dx = g * mask * scale  (the gradient of the residual is g itself; the bias gradient is the column sum of dx)
template <typename T>
__global__ void __launch_bounds__(256) dropout_bwd_kernel(const T* __restrict__ g, T* __restrict__ dx, long long nvec,
                                                          uint32_t threshold, float scale, unsigned long long seed,
                                                          unsigned long long offset) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
        float v[8], o[8];
        bool keep[8];
        Vec8<T>::load(g + i * 8, v);
        dropout_keep8(seed, offset, i, threshold, keep);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = keep[k] ? v[k] * scale : 0.f;
        Vec8<T>::store(dx + i * 8, o);
    }
}

int ew_grid(long long nvec) {
    long long b = (nvec + 255) / 256;
    const long long cap = (long long)neox_sm_count() * 16;
    return (int)(b < cap ? (b > 0 ? b : 1) : cap);
}

template <int MODE>
int launch_ew(const void* a, const void* b, const void* bias, void* out, long long n, int cols, int dtype,
              cudaStream_t st) {
    if (n % 8 || (cols % 8)) return NEOX_ERR_SHAPE;
    if (n == 0) return 0;
    const long long nvec = n / 8;
    const int grid = ew_grid(nvec);
#define LAUNCH(T) ew_kernel<T, MODE><<<grid, 256, 0, st>>>((const T*)a, (const T*)b, (const T*)bias, (T*)out, nvec, cols / 8)
    if (dtype == 0) LAUNCH(__nv_bfloat16);
    else if (dtype == 1) LAUNCH(float);
    else LAUNCH(__half);
#undef LAUNCH
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}


// ------------------------------------------------------------------ column sums (bias gradients)
// partial[blockIdx.y][c] = sum over this CTA's rows of g[r][c]; a CTA is 32 column lanes (8 columns each) x 8 row
// lanes.  The second pass adds the partial rows in a fixed order (bit-reproducible) and stores or accumulates.
template <typename T>
__global__ void __launch_bounds__(256) colsum_partial_kernel(const T* __restrict__ g, float* __restrict__ partial,
                                                             long long rows, int cols, long long ld) {
    __shared__ float sh[8][256];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int col0 = blockIdx.x * 256 + tx * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (col0 < cols) {
        for (long long r = (long long)blockIdx.y * 8 + ty; r < rows; r += (long long)gridDim.y * 8) {
            float v[8];
            Vec8<T>::load(g + r * ld + col0, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += v[i];
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sh[ty][tx * 8 + i] = acc[i];
    __syncthreads();
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c < cols) {
        float t = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) t += sh[j][threadIdx.x];
        partial[(size_t)blockIdx.y * cols + c] = t;
    }
}

template <typename OUT>
__global__ void __launch_bounds__(256) colsum_final_kernel(const float* __restrict__ partial, OUT* __restrict__ out,
                                                           int nblk, int cols, int accumulate) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float a = 0.f;
    for (int r = 0; r < nblk; ++r) a += partial[(size_t)r * cols + c];
    if (accumulate) a += (float)out[c];
    out[c] = (OUT)a;
}

}  // namespace

extern "C" {

int neox_norm_bwd_blocks(int rows) {
    const int cap = neox_sm_count() * 2;
    return rows < cap ? (rows > 0 ? rows : 1) : cap;
}

// out[c] (+)= sum_r g[r, c] for a [rows, cols] 16-bit matrix with row pitch ld (cols % 8 == 0, ld % 8 == 0);
// dtype of g: 0 bf16, 2 fp16; out_dtype: 1 fp32 (may accumulate), else the type of g (store only).
// ws: at least neox_colsum_blocks(rows) * cols floats of scratch.
int neox_colsum_blocks(long long rows) {
    long long b = (rows + 63) / 64;
    const long long cap = 64;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}
int neox_colsum(const void* g, void* out, float* ws, long long rows, int cols, long long ld, int dtype, int out_dtype,
                int accumulate, void* stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if ((cols % 8) || (ld % 8) || (dtype != 0 && dtype != 2)) return NEOX_ERR_SHAPE;
    if (accumulate && out_dtype != 1) return NEOX_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    const int nblk = neox_colsum_blocks(rows);
    dim3 grid((cols + 255) / 256, nblk);
    if (dtype == 0) colsum_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)g, ws, rows, cols, ld);
    else colsum_partial_kernel<__half><<<grid, 256, 0, st>>>((const __half*)g, ws, rows, cols, ld);
    const int fg = (cols + 255) / 256;
    if (out_dtype == 1) colsum_final_kernel<float><<<fg, 256, 0, st>>>(ws, (float*)out, nblk, cols, accumulate);
    else if (dtype == 0) colsum_final_kernel<__nv_bfloat16><<<fg, 256, 0, st>>>(ws, (__nv_bfloat16*)out, nblk, cols, 0);
    else colsum_final_kernel<__half><<<fg, 256, 0, st>>>(ws, (__half*)out, nblk, cols, 0);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

int neox_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                       int rows, int cols, float eps, int dtype, void* stream) {
    return launch_norm_fwd<false>(x, gamma, beta, y, mean, rstd, rows, cols, eps, dtype, (cudaStream_t)stream);
}
int neox_layernorm_bwd(const void* g, const void* x, const void* gamma, const float* mean, const float* rstd,
                       void* dx, float* dgamma, float* dbeta, float* ws, int rows, int cols, int dtype, void* stream) {
    return launch_norm_bwd<false>(g, x, gamma, mean, rstd, dx, dgamma, dbeta, ws, rows, cols, 0.f, dtype,
                                  (cudaStream_t)stream);
}
// dx = (gradient through the norm) + add; add has the shape of dx and may be dx itself.
int neox_layernorm_bwd_add(const void* g, const void* x, const void* gamma, const float* mean, const float* rstd,
                           void* dx, float* dgamma, float* dbeta, float* ws, int rows, int cols, int dtype,
                           const void* add, void* stream) {
    return launch_norm_bwd<false>(g, x, gamma, mean, rstd, dx, dgamma, dbeta, ws, rows, cols, 0.f, dtype,
                                  (cudaStream_t)stream, add);
}
int neox_rmsnorm_bwd_add(const void* g, const void* x, const void* scale, const float* rinv, void* dx, float* dscale,
                         float* dbias, float* ws, int rows, int cols, float eps, int dtype, const void* add,
                         void* stream) {
    return launch_norm_bwd<true>(g, x, scale, nullptr, rinv, dx, dscale, dbias, ws, rows, cols, eps, dtype,
                                 (cudaStream_t)stream, add);
}
int neox_rmsnorm_fwd(const void* x, const void* scale, const void* bias, void* y, float* rinv, int rows, int cols,
                     float eps, int dtype, void* stream) {
    return launch_norm_fwd<true>(x, scale, bias, y, nullptr, rinv, rows, cols, eps, dtype, (cudaStream_t)stream);
}
int neox_rmsnorm_bwd(const void* g, const void* x, const void* scale, const float* rinv, void* dx, float* dscale,
                     float* dbias, float* ws, int rows, int cols, float eps, int dtype, void* stream) {
    return launch_norm_bwd<true>(g, x, scale, nullptr, rinv, dx, dscale, dbias, ws, rows, cols, eps, dtype,
                                 (cudaStream_t)stream);
}
int neox_dgelu_mul(const void* g, const void* pre, void* out, long long n, int dtype, void* stream) {
    return launch_ew<0>(pre, g, nullptr, out, n, 8, dtype, (cudaStream_t)stream);
}
int neox_bias_gelu_fwd(const void* x, const void* bias, void* out, long long rows, int cols, int dtype, void* stream) {
    return launch_ew<1>(x, nullptr, bias, out, rows * cols, cols, dtype, (cudaStream_t)stream);
}
int neox_bias_gelu_bwd(const void* g, const void* x, const void* bias, void* dx, long long rows, int cols, int dtype,
                       void* stream) {
    return launch_ew<2>(x, g, bias, dx, rows * cols, cols, dtype, (cudaStream_t)stream);
}
int neox_bias_residual_add(const void* x, const void* bias, const void* residual, void* out, long long rows, int cols,
                           int dtype, void* stream) {
    return launch_ew<3>(x, residual, bias, out, rows * cols, cols, dtype, (cudaStream_t)stream);
}
// out = residual + dropout(x + bias, p) with the Philox stream (seed, offset); consumes 2 * rows * cols / 8 counter
// values starting at `offset`.  bias and residual may be null.
int neox_bias_dropout_add_fwd(const void* x, const void* bias, const void* residual, void* out, long long rows,
                              int cols, float p, unsigned long long seed, unsigned long long offset, int dtype,
                              void* stream) {
    if (cols % 8 || p < 0.f || p >= 1.f) return NEOX_ERR_SHAPE;
    const long long nvec = rows * cols / 8;
    if (nvec == 0) return 0;
    const uint32_t thr = (uint32_t)fmin(4294967295.0, (double)p * 4294967296.0);
    const float scale = 1.0f / (1.0f - p);
    const int grid = ew_grid(nvec);
    cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH(T) bias_dropout_add_kernel<T><<<grid, 256, 0, st>>>((const T*)x, (const T*)bias, (const T*)residual, (T*)out, nvec, cols / 8, thr, scale, seed, offset)
    if (dtype == 0) LAUNCH(__nv_bfloat16);
    else if (dtype == 1) LAUNCH(float);
    else LAUNCH(__half);
#undef LAUNCH
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
int neox_dropout_bwd(const void* g, void* dx, long long n, float p, unsigned long long seed, unsigned long long offset,
                     int dtype, void* stream) {
    if (n % 8 || p < 0.f || p >= 1.f) return NEOX_ERR_SHAPE;
    const long long nvec = n / 8;
    if (nvec == 0) return 0;
    const uint32_t thr = (uint32_t)fmin(4294967295.0, (double)p * 4294967296.0);
    const float scale = 1.0f / (1.0f - p);
    const int grid = ew_grid(nvec);
    cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH(T) dropout_bwd_kernel<T><<<grid, 256, 0, st>>>((const T*)g, (T*)dx, nvec, thr, scale, seed, offset)
    if (dtype == 0) LAUNCH(__nv_bfloat16);
    else if (dtype == 1) LAUNCH(float);
    else LAUNCH(__half);
#undef LAUNCH
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
int neox_gated_act_fwd(const void* x, void* out, long long rows, int cols, int kind, int dtype, void* stream) {
    if (cols % 8) return NEOX_ERR_SHAPE;
    if (rows == 0) return 0;
    const int grid = ew_grid(rows * (cols / 8));
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == 0) gated_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, rows, cols, kind);
    else if (dtype == 1) gated_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)x, (float*)out, rows, cols, kind);
    else gated_fwd_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, (__half*)out, rows, cols, kind);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
int neox_gated_act_bwd(const void* g, const void* x, void* dx, long long rows, int cols, int kind, int dtype,
                       void* stream) {
    if (cols % 8) return NEOX_ERR_SHAPE;
    if (rows == 0) return 0;
    const int grid = ew_grid(rows * (cols / 8));
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == 0) gated_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)x, (__nv_bfloat16*)dx, rows, cols, kind);
    else if (dtype == 1) gated_bwd_kernel<float><<<grid, 256, 0, st>>>((const float*)g, (const float*)x, (float*)dx, rows, cols, kind);
    else gated_bwd_kernel<__half><<<grid, 256, 0, st>>>((const __half*)g, (const __half*)x, (__half*)dx, rows, cols, kind);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

}  // extern "C"

// =====================================================================================================
// Allocation-free LayerNorm backward (declared in neox_noalloc.h; no counterpart in the reference).
//
// neox_layernorm_bwd() above needs a caller-provided scratch buffer for the per-CTA partial sums of
// dgamma / dbeta.  Some callers cannot provide one: a process whose device memory is already fully
// reserved (for instance by a framework's caching allocator that was sized to the whole GPU), or a
// latency-critical path that must not hit cudaMalloc's implicit device synchronisation.  For them the
// scratch lives in a file-scope device array that is part of the loaded library image.
//
// Rules that follow from that design:
//   * limits: cols <= NEOX_NOALLOC_MAX_COLS, and the kernel uses at most NEOX_NOALLOC_MAX_BLOCKS CTAs;
//     larger requests are rejected with NEOX_ERR_TOO_LARGE (see neox_noalloc_last_error());
//   * the array costs NEOX_NOALLOC_MAX_BLOCKS * NEOX_NOALLOC_MAX_COLS * 2 * 4 bytes (20 MiB) on every GPU
//     that loads the library, until the process exits;
//   * in host code the array's name is only a stand-in for the symbol, not a device address: the device
//     address is looked up with cudaGetSymbolAddress once per device (with that device current) by the
//     first call on that device, which therefore should be made before any stream capture begins;
//   * every call on a device uses the same array.  The kernel fully overwrites the part it reads (nothing
//     has to be zero on entry, and stale contents of earlier calls are never read), but two calls that
//     overlap on the GPU (different streams) race on it: serialise them.
//   * the entry point calls no cudaMalloc / cudaFree and no allocating library routine.
#include "neox_noalloc.h"
#include <stdio.h>

static __device__ __align__(256) float g_noalloc_scratch[2LL * NEOX_NOALLOC_MAX_BLOCKS * NEOX_NOALLOC_MAX_COLS];

namespace {
constexpr int NOALLOC_MAX_DEV = 64;
float* g_noalloc_ptr[NOALLOC_MAX_DEV] = {nullptr};   // idempotent per-device cache: racing first calls store the same value
// One message buffer per host thread: a refusal on one thread cannot tear or overwrite the text another thread
// is about to read through neox_noalloc_last_error().
thread_local char g_noalloc_err[256] = "";

int noalloc_fail(int code, const char* fmt, long long a, long long b) {
    snprintf(g_noalloc_err, sizeof(g_noalloc_err), fmt, a, b);
    return code;
}

// Device address of the scratch array on the current device (looked up once per device).
int noalloc_scratch(float** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEV)
        return noalloc_fail(NEOX_ERR_DRIVER, "no current CUDA device (index %lld, limit %lld)", dev, NOALLOC_MAX_DEV);
    if (!g_noalloc_ptr[dev]) {
        float* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return noalloc_fail(NEOX_ERR_DRIVER, "cudaGetSymbolAddress failed with code %lld on device %lld", (long long)e, dev);
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return 0;
}
}  // namespace

extern "C" const char* neox_noalloc_last_error() { return g_noalloc_err; }

extern "C" int neox_layernorm_bwd_noalloc(const void* g, const void* x, const void* gamma, const float* mean,
                                          const float* rstd, void* dx, float* dgamma, float* dbeta, int rows,
                                          int cols, int dtype, void* stream) {
    if (cols <= 0 || rows < 0 || cols % 8)
        return noalloc_fail(NEOX_ERR_SHAPE, "cols must be a positive multiple of 8 (got %lld; rows %lld)", cols, rows);
    if (cols > NEOX_NOALLOC_MAX_COLS)
        return noalloc_fail(NEOX_ERR_TOO_LARGE, "cols = %lld exceeds the built-in scratch limit of %lld columns", cols,
                            NEOX_NOALLOC_MAX_COLS);
    const int nblk = neox_norm_bwd_blocks(rows);
    if (nblk > NEOX_NOALLOC_MAX_BLOCKS)
        return noalloc_fail(NEOX_ERR_TOO_LARGE, "this GPU would use %lld CTAs, the built-in scratch holds %lld", nblk,
                            NEOX_NOALLOC_MAX_BLOCKS);
    float* ws = nullptr;
    const int rc = noalloc_scratch(&ws);
    if (rc) return rc;
    g_noalloc_err[0] = 0;
    return launch_norm_bwd<false>(g, x, gamma, mean, rstd, dx, dgamma, dbeta, ws, rows, cols, 0.f, dtype,
                                  static_cast<cudaStream_t>(stream));
}
