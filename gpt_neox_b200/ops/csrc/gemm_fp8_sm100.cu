// FP8 GEMM on the fp8 tensor cores of sm_100a (tcgen05.mma.kind::f8f6f4, 128 x 256 x 32 per instruction) with
// per-tensor scaling, plus the cast kernels that produce its operands.
//
//     D = epilogue( alpha * inv_scale_a * inv_scale_b * op(A_q) * op(B_q) )
//
// A_q / B_q hold E4M3 or E5M2 bytes (chosen per operand), `inv_scale_*` are device-resident floats written by the
// cast kernel, so no host synchronisation sits between the cast and the GEMM.  The pipeline is the one of the bf16
// kernel (gemm_sm100.cu): TMA -> 4-stage mbarrier ring (128 bytes of K per stage row, i.e. 128 fp8 elements) -> one
// MMA-issuing thread -> two double-buffered 256-column fp32 accumulators in tensor memory -> four epilogue warps with
// the shared fused epilogue (bias, GeLU, residual / fp32 gradient accumulation).  Both operands may be K-major or
// MN-major, so forward (x W^T), data gradient (dy W) and weight gradient (dy^T x) all read the SAME quantised copy of
// each tensor: no transposed fp8 copies exist.
//
// Casting is per tensor: amax pass, then cast with scale = fp8_max / (amax * 2^margin) ("current" scaling), or a cast
// with a scale derived from an amax history while recording the new amax ("delayed" scaling, the recipe Transformer
// Engine applies in the reference: megatron/model/transformer_engine.py).
//
// All barrier waits are bounded; on a time-out the kernel records a code in the status word, leaves its loops, frees
// its tensor memory and returns.
#include "gemm_common.cuh"
#include "neox_b200.h"
#include <cuda_fp8.h>

using namespace sm100;
using namespace gemm;

namespace {

constexpr int BK8 = 128;              // fp8 elements (= bytes) of K per pipeline stage
constexpr int UMMA_K8 = 32;           // K of one kind::f8f6f4 instruction
constexpr int MN_CHUNK8 = 128;        // elements of the MN dimension per 128-byte swizzle row (MN-major operands)
static_assert(BM * BK8 == A_STAGE_BYTES && BN * BK8 == B_STAGE_BYTES, "fp8 stages reuse the bf16 stage sizes");

struct Fp8Extra {
    const float* inv_scale_a;         // device scalars; NULL = 1
    const float* inv_scale_b;
    int a_fmt, b_fmt;                 // 0 = E4M3, 1 = E5M2
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const GemmParams p, const Fp8Extra x) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* tfull = empty + STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 4);
        }
        fence_barrier_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_m = (p.M + BM - 1) / BM;
    const int num_n = (p.N + BN - 1) / BN;
    const int ntiles = num_m * num_n;
    const int nk = (p.K + BK8 - 1) / BK8;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                int m_blk, n_blk;
                tile_coords(tile, num_m, num_n, m_blk, n_blk);
                for (int kb = 0; kb < nk; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1)) {
                        atomicExch(p.status, 111);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[stage], A_STAGE_BYTES + B_STAGE_BYTES);
                    uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
                    uint8_t* b_dst = sB + stage * B_STAGE_BYTES;
                    if (!p.a_mn) {
                        tma_load_2d(a_dst, &tmA, &full[stage], kb * BK8, m_blk * BM);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / MN_CHUNK8; ++j)
                            tma_load_2d(a_dst + j * (MN_CHUNK8 * BK8), &tmA, &full[stage], m_blk * BM + j * MN_CHUNK8,
                                        kb * BK8);
                    }
                    if (!p.b_mn) {
                        tma_load_2d(b_dst, &tmB, &full[stage], kb * BK8, n_blk * BN);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / MN_CHUNK8; ++j)
                            tma_load_2d(b_dst + j * (MN_CHUNK8 * BK8), &tmB, &full[stage], n_blk * BN + j * MN_CHUNK8,
                                        kb * BK8);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc_f8(BM, BN, p.a_mn, p.b_mn, x.a_fmt, x.b_fmt);
            // operand descriptors: constant upper half; lower half = stage base + k-step offset (16-byte units).
            // K-major: the next 32 elements of K are 32 bytes further along each swizzled 128-byte row.  MN-major:
            // they are the next 32 rows of 128 bytes; 8-row groups are 1024 bytes apart and 128-element chunks of
            // the MN dimension MN_CHUNK8 * BK8 bytes apart.
            const uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA), p.a_mn ? MN_CHUNK8 * BK8 : 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(sB), p.b_mn ? MN_CHUNK8 * BK8 : 16);
            const uint32_t a_step = (p.a_mn ? UMMA_K8 * 128 : UMMA_K8) >> 4;
            const uint32_t b_step = (p.b_mn ? UMMA_K8 * 128 : UMMA_K8) >> 4;
            int stage = 0;
            uint32_t phase = 0;
            int buf = 0;
            uint32_t bphase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                if (!mbar_wait(&tempty[buf], bphase ^ 1)) {
                    atomicExch(p.status, 112);
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < nk; ++kb) {
                    if (!mbar_wait(&full[stage], phase)) {
                        atomicExch(p.status, 113);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + stage * (A_STAGE_BYTES >> 4);
                    const uint32_t b_lo = b_lo0 + stage * (B_STAGE_BYTES >> 4);
#pragma unroll
                    for (int k = 0; k < BK8 / UMMA_K8; ++k)
                        umma_ss_lohi<false, true>(tmem_d, a_lo + k * a_step, desc_hi, b_lo + k * b_step, desc_hi, idesc,
                                                  (kb | k) != 0);
                    umma_commit(&empty[stage]);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(&tfull[buf]);
                buf ^= 1;
                if (buf == 0) bphase ^= 1;
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps (2..5)
        GemmParams pe = p;
        if (x.inv_scale_a) pe.alpha *= __ldg(x.inv_scale_a);
        if (x.inv_scale_b) pe.alpha *= __ldg(x.inv_scale_b);
        const int q = warp & 3;
        int buf = 0;
        uint32_t bphase = 0;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
            int m_blk, n_blk;
            tile_coords(tile, num_m, num_n, m_blk, n_blk);
            if (!mbar_wait_warp(&tfull[buf], bphase)) {
                if (lane == 0) atomicExch(p.status, 114);
                break;
            }
            tc_fence_after();
            const int row = m_blk * BM + q * 32 + lane;
            const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int col0 = n_blk * BN + c * 32;
                if (col0 >= p.N) break;  // warp-uniform
                uint32_t r[32];
                tmem_ld_32x32(taddr + c * 32, r);
                tmem_wait_ld();
                if (row < p.M) epilogue_chunk(r, row, col0, pe);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[buf]);
            buf ^= 1;
            if (buf == 0) bphase ^= 1;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------ casts
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

__device__ __forceinline__ float abs_max8(const uint4& r) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    float m = 0.f;
#pragma unroll
    for (int t = 0; t < 4; ++t) m = fmaxf(m, fmaxf(fabsf(bf16_lo(w[t])), fabsf(bf16_hi(w[t]))));
    return m;
}

// amax[0] = max(amax[0], max |x|); non-negative floats order like their bit patterns, so an integer atomicMax does it.
// NaN / Inf inputs are ignored here (the overflow check of the loss scaler owns them).
__global__ void __launch_bounds__(256) fp8_amax_kernel(const bf16* __restrict__ x, long long n, float* __restrict__ amax) {
    const long long nv = n / 8;
    const uint4* x4 = reinterpret_cast<const uint4*>(x);
    float m = 0.f;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x)
        m = fmaxf(m, abs_max8(__ldg(x4 + i)));
    if (blockIdx.x == 0)
        for (long long i = nv * 8 + threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, fabsf(__bfloat162float(x[i])));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0 && m > 0.f && m < 3.0e38f) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));
}

__device__ __forceinline__ float scale_from_amax(float amax, float fp8_max, float margin_mult) {
    return (amax > 0.f && amax < 3.0e38f) ? fp8_max / (amax * margin_mult) : 1.f;
}

template <bool E5M2>
__device__ __forceinline__ uint32_t cast4(float a, float b, float c, float d) {
    const __nv_fp8_interpretation_t k = E5M2 ? __NV_E5M2 : __NV_E4M3;
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, k);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, k);
    return lo | (hi << 16);
}

// q = fp8(x * scale).  scale = *scale_in when from_amax == 0, else fp8_max / (*scale_in * margin_mult).  Thread 0
// of block 0 publishes 1 / scale.  `record` (optional) accumulates max |x| for a delayed-scaling history.
template <bool E5M2>
__global__ void __launch_bounds__(256) fp8_cast_kernel(const bf16* __restrict__ x, unsigned char* __restrict__ q,
                                                       long long n, const float* __restrict__ scale_in, int from_amax,
                                                       float fp8_max, float margin_mult, float* __restrict__ inv_out,
                                                       float* __restrict__ record) {
    const float s0 = *scale_in;
    const float scale = from_amax ? scale_from_amax(s0, fp8_max, margin_mult) : s0;
    if (blockIdx.x == 0 && threadIdx.x == 0 && inv_out) *inv_out = 1.f / scale;
    const long long nv = n / 8;
    const uint4* x4 = reinterpret_cast<const uint4*>(x);
    uint2* q2 = reinterpret_cast<uint2*>(q);
    float m = 0.f;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
        const uint4 r = __ldg(x4 + i);
        if (record) m = fmaxf(m, abs_max8(r));
        uint2 o;
        o.x = cast4<E5M2>(bf16_lo(r.x) * scale, bf16_hi(r.x) * scale, bf16_lo(r.y) * scale, bf16_hi(r.y) * scale);
        o.y = cast4<E5M2>(bf16_lo(r.z) * scale, bf16_hi(r.z) * scale, bf16_lo(r.w) * scale, bf16_hi(r.w) * scale);
        q2[i] = o;
    }
    if (blockIdx.x == 0)
        for (long long i = nv * 8 + threadIdx.x; i < n; i += blockDim.x) {
            const float v = __bfloat162float(x[i]);
            if (record) m = fmaxf(m, fabsf(v));
            q[i] = (unsigned char)__nv_cvt_float_to_fp8(v * scale, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
        }
    if (record) {
        m = warp_max(m);
        if ((threadIdx.x & 31) == 0 && m > 0.f && m < 3.0e38f)
            atomicMax(reinterpret_cast<int*>(record), __float_as_int(m));
    }
}

// Delayed scaling bookkeeping for one tensor role, one thread: push the amax recorded since the last call into the
// history ring, clear the recorder, and derive the scale for the next cast from the history.
//   meta[0] = scale, meta[1] = 1 / scale, meta[2] = recorder, meta[3] = ring position, meta[4 ...] = history[len]
__global__ void fp8_delayed_update_kernel(float* __restrict__ meta, int len, float fp8_max, float margin_mult,
                                          int most_recent) {
    if (threadIdx.x || blockIdx.x) return;
    float* hist = meta + 4;
    int pos = (int)meta[3];
    const float cur = meta[2];
    hist[pos] = cur;
    meta[2] = 0.f;
    meta[3] = (float)((pos + 1) % len);
    float amax = cur;
    if (!most_recent)
        for (int i = 0; i < len; ++i) amax = fmaxf(amax, hist[i]);
    if (amax > 0.f && amax < 3.0e38f) {
        const float s = fp8_max / (amax * margin_mult);
        meta[0] = s;
        meta[1] = 1.f / s;
    } else if (meta[0] == 0.f) {
        meta[0] = 1.f;
        meta[1] = 1.f;
    }
}

int cast_grid(long long n) {
    long long g = (n / 8 + 255) / 256;
    const long long cap = 148LL * 8;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

// amax[0] = max(amax[0], max |x|) over n bf16 elements (x 16-byte aligned).  The caller zeroes amax.
extern "C" int neox_fp8_amax(const void* x, long long n, float* amax, void* stream) {
    if (n <= 0) return 0;
    if (reinterpret_cast<uintptr_t>(x) & 15) return NEOX_ERR_ALIGN;
    fp8_amax_kernel<<<cast_grid(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const bf16*>(x), n, amax);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// q[i] = fp8(x[i] * scale); see fp8_cast_kernel for the meaning of scale_in / from_amax.  margin: the scale is
// divided by 2^margin.  inv_out (device float) receives 1 / scale; record may be NULL.
extern "C" int neox_fp8_cast(const void* x, void* q, long long n, const float* scale_in, int from_amax, int e5m2,
                             int margin, float* inv_out, float* record, void* stream) {
    if (n <= 0) return 0;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7)) return NEOX_ERR_ALIGN;
    const float mm = exp2f((float)margin);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (e5m2)
        fp8_cast_kernel<true><<<cast_grid(n), 256, 0, st>>>(static_cast<const bf16*>(x), static_cast<unsigned char*>(q),
                                                            n, scale_in, from_amax, 57344.f, mm, inv_out, record);
    else
        fp8_cast_kernel<false><<<cast_grid(n), 256, 0, st>>>(static_cast<const bf16*>(x), static_cast<unsigned char*>(q),
                                                             n, scale_in, from_amax, 448.f, mm, inv_out, record);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// meta: device floats [4 + len] (layout at fp8_delayed_update_kernel), zero-initialised by the caller.
extern "C" int neox_fp8_delayed_update(float* meta, int len, int e5m2, int margin, int most_recent, void* stream) {
    if (len <= 0) return NEOX_ERR_SHAPE;
    fp8_delayed_update_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(meta, len, e5m2 ? 57344.f : 448.f,
                                                                               exp2f((float)margin), most_recent);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// A, B: fp8 bytes.  A is [M, K] (a_mn = 0) or [K, M] (a_mn = 1) with a row pitch of lda BYTES; B is [N, K] or
// [K, N] likewise.  a_fmt / b_fmt: 0 = E4M3, 1 = E5M2.  inv_scale_a / inv_scale_b: device floats multiplied into
// alpha (NULL = 1).  Everything after them is the epilogue of neox_gemm_bf16.
extern "C" int neox_gemm_fp8(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                             long long ldd, int a_mn, int b_mn, int a_fmt, int b_fmt, const float* inv_scale_a,
                             const float* inv_scale_b, int d_fp32, const void* bias, const void* add, long long ldadd,
                             int add_fp32, void* preact, long long ldpre, const void* aux, long long ldaux, int act,
                             float alpha, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 16) || (ldb % 16))
        return NEOX_ERR_ALIGN;
    if ((a_fmt | b_fmt) & ~1) return NEOX_ERR_SHAPE;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;

    CUtensorMap tmA, tmB;
    int rc;
    if (!a_mn) rc = neox_make_tmap_u8_2d(&tmA, A, K, M, lda, BK8, BM);
    else rc = neox_make_tmap_u8_2d(&tmA, A, M, K, lda, MN_CHUNK8, BK8);
    if (rc) return rc;
    if (!b_mn) rc = neox_make_tmap_u8_2d(&tmB, B, K, N, ldb, BK8, BN);
    else rc = neox_make_tmap_u8_2d(&tmB, B, N, K, ldb, MN_CHUNK8, BK8);
    if (rc) return rc;

    GemmParams p;
    p.M = M; p.N = N; p.K = K;
    p.a_mn = a_mn; p.b_mn = b_mn;
    p.D = D; p.ldd = ldd; p.d_fp32 = d_fp32;
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.add = add; p.ldadd = ldadd; p.add_fp32 = add_fp32;
    p.preact = static_cast<__nv_bfloat16*>(preact); p.ldpre = ldpre;
    p.aux = static_cast<const __nv_bfloat16*>(aux); p.ldaux = ldaux;
    p.act = act; p.alpha = alpha;
    p.status = status;
    p.row_ptrs = nullptr;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    bool vec = al16(D) && (ldd % 8 == 0);
    if (bias) vec = vec && al16(bias);
    if (add) vec = vec && al16(add) && (ldadd % 8 == 0);
    if (preact) vec = vec && al16(preact) && (ldpre % 8 == 0);
    if (aux) vec = vec && al16(aux) && (ldaux % 8 == 0);
    p.vec_ok = vec ? 1 : 0;
    Fp8Extra x{inv_scale_a, inv_scale_b, a_fmt, b_fmt};

    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_fp8_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
            cudaSuccess)
            return NEOX_ERR_LAUNCH;
        attr_set = true;
    }
    const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN;
    int grid = num_m * num_n;
    const int sms = neox_sm_count();
    if (grid > sms) grid = sms;
    gemm_fp8_tcgen05_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p, x);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
