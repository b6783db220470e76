// Mamba selective scan (S6), forward and backward, channel-last layouts, state size 16.
//
//     delta = softplus(dt + dt_bias)
//     h_t[j] = exp(delta_t * A[c][j]) * h_{t-1}[j] + delta_t * B_t[j] * u_t        (c = channel, j = state index)
//     y_t    = sum_j C_t[j] * h_t[j] + D[c] * u_t,      out_t = y_t * silu(z_t)
//
// One thread owns one channel and keeps its 16 states in registers; consecutive threads own consecutive channels, so
// every load of u / dt / z ([b, l, d], d contiguous) is coalesced and B_t / C_t ([b, l, 16]) are broadcast from
// shared memory.  The forward stores the state at the start of every 32-step chunk; the backward walks the chunks in
// reverse, recomputes the 32 states of a chunk into shared memory from its checkpoint and then runs the adjoint
// recurrence backwards through them, so no per-step state is ever written to global memory.  Gradients that sum over
// channels (dB, dC) are reduced inside the warp before one atomicAdd per warp; dA, dD and d(dt_bias) accumulate in
// registers over time and are added once per (batch, channel).
//
// Same contract as mamba_ssm's selective_scan_fn as used by megatron/model/mamba/mamba.py:207-300 of the reference
// (delta_softplus = True, D, z and delta_bias given).
#include "neox_b200.h"
#include <cuda_bf16.h>

namespace {

typedef __nv_bfloat16 bf16;
constexpr int NS = 16;        // state size
constexpr int CHUNK = 32;     // steps between checkpoints
constexpr int FWD_THREADS = 128;
constexpr int BWD_THREADS = 64;

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

__global__ void __launch_bounds__(FWD_THREADS)
scan_fwd_kernel(const bf16* __restrict__ u, const bf16* __restrict__ dt, const float* __restrict__ A,
                const float* __restrict__ B, const float* __restrict__ C, const float* __restrict__ D,
                const bf16* __restrict__ z, const float* __restrict__ bias, bf16* __restrict__ out,
                float* __restrict__ ckpt, int l, int d, int nchk) {
    __shared__ float sB[CHUNK][NS], sC[CHUNK][NS];
    const int b = blockIdx.y;
    const int c = blockIdx.x * FWD_THREADS + threadIdx.x;
    const bool live = c < d;
    float a[NS], h[NS];
#pragma unroll
    for (int j = 0; j < NS; ++j) {
        a[j] = live ? A[(size_t)c * NS + j] : 0.f;
        h[j] = 0.f;
    }
    const float Dc = live ? D[c] : 0.f, bc = live ? bias[c] : 0.f;
    for (int t0 = 0, ck = 0; t0 < l; t0 += CHUNK, ++ck) {
        const int steps = min(CHUNK, l - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < steps * NS; i += FWD_THREADS) {
            sB[i / NS][i % NS] = B[((size_t)b * l + t0) * NS + i];
            sC[i / NS][i % NS] = C[((size_t)b * l + t0) * NS + i];
        }
        __syncthreads();
        if (!live) continue;
        float* cp = ckpt + (((size_t)b * nchk + ck) * d + c) * NS;
#pragma unroll
        for (int j = 0; j < NS; j += 4) *reinterpret_cast<float4*>(cp + j) = make_float4(h[j], h[j + 1], h[j + 2], h[j + 3]);
        for (int s = 0; s < steps; ++s) {
            const size_t o = ((size_t)b * l + t0 + s) * d + c;
            const float uv = __bfloat162float(u[o]);
            const float delta = softplus_f(__bfloat162float(dt[o]) + bc);
            const float du = delta * uv;
            float y = Dc * uv;
#pragma unroll
            for (int j = 0; j < NS; ++j) {
                h[j] = __expf(delta * a[j]) * h[j] + du * sB[s][j];
                y += sC[s][j] * h[j];
            }
            const float zv = __bfloat162float(z[o]);
            out[o] = __float2bfloat16(y * zv * sigmoid_f(zv));
        }
    }
}

// Shared memory: states of one chunk, hs[(s * NS + j) * BWD_THREADS + tid]  (s = 0 is the checkpoint, s = k the state
// after step k - 1), then B, C and the per-step reduction scratch.
__global__ void __launch_bounds__(BWD_THREADS)
scan_bwd_kernel(const bf16* __restrict__ u, const bf16* __restrict__ dt, const float* __restrict__ A,
                const float* __restrict__ B, const float* __restrict__ C, const float* __restrict__ D,
                const bf16* __restrict__ z, const float* __restrict__ bias, const float* __restrict__ ckpt,
                const bf16* __restrict__ gout, bf16* __restrict__ gu, bf16* __restrict__ gdt, bf16* __restrict__ gz,
                float* __restrict__ gA, float* __restrict__ gB, float* __restrict__ gC, float* __restrict__ gD,
                float* __restrict__ gbias, int l, int d, int nchk) {
    extern __shared__ float smem[];
    float* hs = smem;                                           // (CHUNK + 1) * NS * BWD_THREADS
    float* sB = hs + (CHUNK + 1) * NS * BWD_THREADS;            // CHUNK * NS
    float* sC = sB + CHUNK * NS;
    const int b = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31;
    const int c_raw = blockIdx.x * BWD_THREADS + tid;
    // Threads past the last channel run the same instruction stream on the last channel's data (so every shuffle
    // below is executed by full, converged warps) and are masked out of every store and every sum.
    const bool live = c_raw < d;
    const int c = live ? c_raw : d - 1;
    const float mask = live ? 1.f : 0.f;
    float a[NS], gh[NS], ga[NS];
#pragma unroll
    for (int j = 0; j < NS; ++j) {
        a[j] = A[(size_t)c * NS + j];
        gh[j] = 0.f;
        ga[j] = 0.f;
    }
    const float Dc = D[c], bc = bias[c];
    float gDc = 0.f, gbc = 0.f;
    for (int ck = nchk - 1; ck >= 0; --ck) {
        const int t0 = ck * CHUNK;
        const int steps = min(CHUNK, l - t0);
        __syncthreads();
        for (int i = tid; i < steps * NS; i += BWD_THREADS) {
            sB[i] = B[((size_t)b * l + t0) * NS + i];
            sC[i] = C[((size_t)b * l + t0) * NS + i];
        }
        __syncthreads();
        // ---- recompute the states of this chunk
        {
            float h[NS];
            const float* cp = ckpt + (((size_t)b * nchk + ck) * d + c) * NS;
#pragma unroll
            for (int j = 0; j < NS; ++j) {
                h[j] = cp[j];
                hs[(0 * NS + j) * BWD_THREADS + tid] = h[j];
            }
            for (int s = 0; s < steps; ++s) {
                const size_t o = ((size_t)b * l + t0 + s) * d + c;
                const float uv = __bfloat162float(u[o]);
                const float delta = softplus_f(__bfloat162float(dt[o]) + bc);
                const float du = delta * uv;
#pragma unroll
                for (int j = 0; j < NS; ++j) {
                    h[j] = __expf(delta * a[j]) * h[j] + du * sB[s * NS + j];
                    hs[((s + 1) * NS + j) * BWD_THREADS + tid] = h[j];
                }
            }
        }
        // ---- adjoint recurrence, backwards through the chunk
        for (int s = steps - 1; s >= 0; --s) {
            float pb[NS], pc[NS];      // this channel's contributions to dB_t and dC_t
            const size_t o = ((size_t)b * l + t0 + s) * d + c;
            const float uv = __bfloat162float(u[o]);
            const float x = __bfloat162float(dt[o]) + bc;
            const float delta = softplus_f(x);
            const float zv = __bfloat162float(z[o]);
            const float sz = sigmoid_f(zv);
            const float go = __bfloat162float(gout[o]) * mask;
            float y = Dc * uv;
#pragma unroll
            for (int j = 0; j < NS; ++j) y += sC[s * NS + j] * hs[((s + 1) * NS + j) * BWD_THREADS + tid];
            const float g_z = go * y * sz * (1.f + zv * (1.f - sz));
            const float gy = go * zv * sz;
            gDc += gy * uv;
            float g_u = gy * Dc, g_delta = 0.f;
#pragma unroll
            for (int j = 0; j < NS; ++j) {
                const float hcur = hs[((s + 1) * NS + j) * BWD_THREADS + tid];
                const float hprev = hs[(s * NS + j) * BWD_THREADS + tid];
                pc[j] = gy * hcur;
                const float g = gh[j] + gy * sC[s * NS + j];      // adjoint of h_t[j]
                const float dA = __expf(delta * a[j]);
                const float gdA = g * hprev * dA;                  // d/d(delta * a[j])
                g_delta += gdA * a[j] + g * sB[s * NS + j] * uv;
                ga[j] += gdA * delta;
                pb[j] = g * delta * uv;
                g_u += g * delta * sB[s * NS + j];
                gh[j] = g * dA;
            }
            const float g_dt = g_delta * sigmoid_f(x);             // softplus'
            gbc += g_dt;
            if (live) {
                gz[o] = __float2bfloat16(g_z);
                gu[o] = __float2bfloat16(g_u);
                gdt[o] = __float2bfloat16(g_dt);
            }
            // ---- sum dB_t / dC_t over the channels of this warp, one atomic per warp and state index
#pragma unroll
            for (int j = 0; j < NS; ++j) {
                float vb = pb[j], vc = pc[j];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    vb += __shfl_xor_sync(0xffffffffu, vb, off);
                    vc += __shfl_xor_sync(0xffffffffu, vc, off);
                }
                if (lane == j) {
                    atomicAdd(gB + ((size_t)b * l + t0 + s) * NS + j, vb);
                    atomicAdd(gC + ((size_t)b * l + t0 + s) * NS + j, vc);
                }
            }
        }
    }
    if (live) {
#pragma unroll
        for (int j = 0; j < NS; ++j) atomicAdd(gA + (size_t)c * NS + j, ga[j]);
        atomicAdd(gD + c, gDc);
        atomicAdd(gbias + c, gbc);
    }
}

constexpr int BWD_SMEM = ((CHUNK + 1) * NS * BWD_THREADS + 2 * CHUNK * NS) * (int)sizeof(float);

}  // namespace

extern "C" int neox_selective_scan_fwd(const void* u, const void* dt, const float* A, const float* B, const float* C,
                                       const float* D, const void* z, const float* bias, void* out, float* ckpt, int b,
                                       int l, int d, int n, void* stream) {
    if (n != NS) return NEOX_ERR_SHAPE;
    if (b <= 0 || l <= 0 || d <= 0) return 0;
    const int nchk = (l + CHUNK - 1) / CHUNK;
    dim3 grid((d + FWD_THREADS - 1) / FWD_THREADS, b);
    scan_fwd_kernel<<<grid, FWD_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf16*>(u), static_cast<const bf16*>(dt), A, B, C, D, static_cast<const bf16*>(z), bias,
        static_cast<bf16*>(out), ckpt, l, d, nchk);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// gA, gB, gC, gD, gbias must be zero on entry (they are accumulated with atomics).
extern "C" int neox_selective_scan_bwd(const void* u, const void* dt, const float* A, const float* B, const float* C,
                                       const float* D, const void* z, const float* bias, const float* ckpt,
                                       const void* gout, void* gu, void* gdt, void* gz, float* gA, float* gB, float* gC,
                                       float* gD, float* gbias, int b, int l, int d, int n, void* stream) {
    if (n != NS) return NEOX_ERR_SHAPE;
    if (b <= 0 || l <= 0 || d <= 0) return 0;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess)
            return NEOX_ERR_LAUNCH;
        attr_set = true;
    }
    const int nchk = (l + CHUNK - 1) / CHUNK;
    dim3 grid((d + BWD_THREADS - 1) / BWD_THREADS, b);
    scan_bwd_kernel<<<grid, BWD_THREADS, BWD_SMEM, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf16*>(u), static_cast<const bf16*>(dt), A, B, C, D, static_cast<const bf16*>(z), bias, ckpt,
        static_cast<const bf16*>(gout), static_cast<bf16*>(gu), static_cast<bf16*>(gdt), static_cast<bf16*>(gz), gA, gB,
        gC, gD, gbias, l, d, nchk);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
