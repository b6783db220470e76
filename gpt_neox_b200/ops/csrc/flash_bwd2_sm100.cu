// Flash attention backward for sm_100a with 128 x 128 score blocks and gradient operands kept in tensor memory
// (the default backward; csrc/flash_bwd_sm100.cu is the earlier 64-wide, shared-memory-operand form).
//
//   delta   D[b,h,q] = sum_d dO * O                                          (one warp per row)
//   dkv     one CTA per (128-key tile, batch, kv head); for every 128-query block that can see the tile:
//               S^T = K Q^T,  dP^T = V dO^T            (keys on the TMEM lanes, queries on the columns)
//               P^T = exp2(S^T * scale - lse),  dS^T = P^T (dP^T - D)      written back over S^T / dP^T as packed
//               16-bit pairs and consumed from TENSOR MEMORY as the A operand of
//               dV += P^T dO,  dK += dS^T Q            (accumulators resident in TMEM over the whole loop and over
//               the query heads of a GQA group: no atomics, bit-reproducible);
//           the issue order  dV(i), S^T(i+1), dK(i), dP^T(i+1)  keeps the tensor pipe fed while the sixteen compute
//           warps (four per TMEM lane quarter, 32 score columns per thread) work on the other half of the block;
//   dq      one CTA per (128-query tile, batch, head); loops over 128-key blocks:  S = Q K^T,  dP = dO V^T
//           (dP double-buffered in TMEM),  dS = P (dP - D)  over dP,  dQ += dS K  with dS read from tensor memory.
//
// Per 16-row operand slice a tcgen05.mma fetches its A and B operands at about 64 bytes per clock, which is what
// bounds these kernels: 128-wide blocks and TMEM-resident P / dS halve the operand traffic of the 64-wide form.
// The softmax scale of dS is applied once to dK and dQ in the epilogues.  Head sizes 64 / 96 / 128, bf16 or fp16.
// Replaces the flash-attn 2 backward behind megatron/model/transformer.py:627-744.  Every wait is bounded.
#include "sm100_ptx.cuh"
#include "neox_b200.h"
#include <cuda_fp16.h>
#include <math.h>

using namespace sm100;

namespace {

constexpr int CH = 128 * 128;            // one [128 rows x 64 x 16-bit] swizzled chunk
constexpr float LOG2E = 1.4426950408889634f;
constexpr int PARTS = 4;                 // compute warps per TMEM lane quarter
constexpr int CPT = 128 / PARTS;         // score columns per compute thread (32)
constexpr int THREADS = 128 + PARTS * 128;

struct Bwd2Params {
    int sq, sk, b, hq, hkv;
    float scale, scale_log2;
    int causal, window;
    const float* slopes;
    const float* lse;    // [b, hq, sq] natural log
    const float* delta;  // [b, hq, sq]
    void *dq, *dk, *dv;  // [s, b, h, d] views of 16-bit elements; element strides of (s, b, h) below
    long long dq_s[3], dk_s[3], dv_s[3];
    int* status;
};

template <bool FP16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    if (FP16) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    return pack_bf16x2(lo, hi);
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t idesc16(int M, int N, int b_mn, bool fp16) {
    uint32_t d = 0;
    d |= 1u << 4;
    d |= (fp16 ? 0u : 1u) << 7;
    d |= (fp16 ? 0u : 1u) << 10;
    d |= (uint32_t)(b_mn & 1) << 16;
    d |= (uint32_t)(N >> 3) << 17;
    d |= (uint32_t)(M >> 4) << 24;
    return d;
}

__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void wait_ld_dep(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                   "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                   "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

// ------------------------------------------------------------------ delta
// One thread per 8 elements (16-byte loads), d / 8 threads per row, rows packed into the warp; the partial sums of a row
// are combined with shuffles inside groups of 16 lanes (d / 8 <= 16).
template <bool FP16>
__global__ void __launch_bounds__(256) delta2_kernel(const uint4* __restrict__ o, const uint4* __restrict__ dout,
                                                     float* __restrict__ delta, long long rows, int sq, int b, int hq,
                                                     int tpr) {
    const int sub = threadIdx.x & 15;                                  // position inside the 16-lane group
    const long long row = (blockIdx.x * 256LL + threadIdx.x) >> 4;     // one row per 16-lane group
    float s = 0.f;
    if (row < rows && sub < tpr) {
        const uint4 a = o[row * tpr + sub], g = dout[row * tpr + sub];
        const uint32_t av[4] = {a.x, a.y, a.z, a.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (FP16) {
                const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&av[k]));
                const float2 fg = __half22float2(*reinterpret_cast<const __half2*>(&gv[k]));
                s += fa.x * fg.x + fa.y * fg.y;
            } else {
                s += bf16_lo(av[k]) * bf16_lo(gv[k]) + bf16_hi(av[k]) * bf16_hi(gv[k]);
            }
        }
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (row < rows && sub == 0) {
        const int h = (int)(row % hq);
        const long long t = row / hq;
        const int bb = (int)(t % b);
        const int q = (int)(t / b);
        delta[((size_t)bb * hq + h) * sq + q] = s;
    }
}

template <int D>
struct B2Cfg {
    static constexpr int NCH = (D == 64) ? 1 : 2;
    static constexpr int TILE = NCH * CH;            // one 128-row operand tile
    static constexpr int OFF_R0 = 0;                 // resident tile 0 (K in dkv, Q in dq)
    static constexpr int OFF_R1 = TILE;              // resident tile 1 (V in dkv, dO in dq)
    static constexpr int OFF_S = 2 * TILE;           // 2 stages x (tile a, tile b)
    static constexpr int OFF_MISC = 6 * TILE;
    static constexpr int MISC = 8192;
    static constexpr int SMEM = OFF_MISC + MISC + 1024;
};

// TMEM column of the packed 16-bit A-operand slice for contraction step kk (16 rows of the contraction): compute
// part p packs its 32 columns into the first 16 columns of its own 32-column range.
__device__ __forceinline__ uint32_t packed_col(int kk) { return (uint32_t)((kk >> 1) * 32 + (kk & 1) * 8); }

// =================================================================== dK / dV
template <int D, bool FP16>
__global__ void __launch_bounds__(THREADS, 1)
flash_bwd2_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                      const Bwd2Params p) {
    using C = B2Cfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem + C::OFF_R0;
    uint8_t* sV = smem + C::OFF_R1;
    uint8_t* sStage = smem + C::OFF_S;   // stage st: Q at st*2*TILE, dO at st*2*TILE + TILE
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_MISC);
    uint64_t* kv_full = bars;            // 1
    uint64_t* st_full = bars + 1;        // 2  Q_i / dO_i landed
    uint64_t* st_empty = bars + 3;       // 2
    uint64_t* s_full = bars + 5;         // 1  S^T in TMEM
    uint64_t* dp_full = bars + 6;        // 1  dP^T in TMEM
    uint64_t* p_full = bars + 7;         // 1  P^T written over S^T
    uint64_t* ds_full = bars + 8;        // 1  dS^T written over dP^T
    uint64_t* acc_full = bars + 9;       // 1  dK, dV final
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kv0 = blockIdx.x * 128;
    const int bb = blockIdx.y / p.hkv, hk = blockIdx.y % p.hkv;
    const int G = p.hq / p.hkv;
    const int off = p.sk - p.sq;
    int q_lo = 0, q_hi = p.sq;       // query rows that can attend to this key tile
    if (p.causal) q_lo = max(0, kv0 - off);
    if (p.window >= 0) q_hi = min(p.sq, kv0 + 127 - off + p.window + 1);
    const int ib = q_lo / 128;
    const int ie = (q_hi + 127) / 128;
    const int nq = max(ie - ib, 0);
    const int niter = nq * G;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&st_full[i], 1);
            mbar_init(&st_empty[i], 1);
        }
        mbar_init(s_full, 1);
        mbar_init(dp_full, 1);
        mbar_init(p_full, 4 * PARTS);
        mbar_init(ds_full, 4 * PARTS);
        mbar_init(acc_full, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t TM_ST = tmem_base, TM_DPT = tmem_base + 128, TM_DV = tmem_base + 256, TM_DK = tmem_base + 384;

    if (warp == 0) {
        if (lane == 0 && niter > 0) {
            mbar_expect_tx(kv_full, 2 * C::TILE);
#pragma unroll
            for (int c = 0; c < C::NCH; ++c) {
                tma_load_4d(sK + c * CH, &tmK, kv_full, c * 64, hk, bb, kv0);
                tma_load_4d(sV + c * CH, &tmV, kv_full, c * 64, hk, bb, kv0);
            }
            for (int it = 0; it < niter; ++it) {
                const int st = it & 1;
                if (!mbar_wait(&st_empty[st], ((it >> 1) & 1) ^ 1)) {
                    atomicExch(p.status, 321);
                    break;
                }
                const int h = hk * G + it / nq;
                const int qi0 = (ib + it % nq) * 128;
                mbar_expect_tx(&st_full[st], 2 * C::TILE);
                uint8_t* base = sStage + st * 2 * C::TILE;
#pragma unroll
                for (int c = 0; c < C::NCH; ++c) {
                    tma_load_4d(base + c * CH, &tmQ, &st_full[st], c * 64, h, bb, qi0);
                    tma_load_4d(base + C::TILE + c * CH, &tmdO, &st_full[st], c * 64, h, bb, qi0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && niter > 0) {
            const uint32_t id_s = idesc16(128, 128, 0, FP16);   // S^T = K Q^T   (both K-major)
            const uint32_t id_g = idesc16(128, D, 1, FP16);     // dV = P^T dO   (A from TMEM, B MN-major)
            const uint32_t hi = smem_desc_hi_sw128(1024);
            const uint32_t k_lo = smem_desc_lo(smem_u32(sK), 16), v_lo = smem_desc_lo(smem_u32(sV), 16);
            bool ok = mbar_wait(kv_full, 0);
            if (!ok) atomicExch(p.status, 322);
            auto scores = [&](int it, bool second) -> bool {      // S^T (first) or dP^T (second) of block `it`
                const int st = it & 1;
                if (!mbar_wait(&st_full[st], (it >> 1) & 1)) return false;
                tc_fence_after();
                const uint32_t b_lo = smem_desc_lo(smem_u32(sStage + st * 2 * C::TILE + (second ? C::TILE : 0)), 16);
                const uint32_t a_lo = second ? v_lo : k_lo;
                const uint32_t td = second ? TM_DPT : TM_ST;
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t o = ((k >> 2) * CH + (k & 3) * 32) >> 4;
                    umma_ss_lohi<false, false>(td, a_lo + o, hi, b_lo + o, hi, id_s, k != 0 ? 1u : 0u);
                }
                umma_commit(second ? dp_full : s_full);
                return true;
            };
            auto grad = [&](int it, bool second) {                 // dV += P^T dO (first) or dK += dS^T Q (second)
                const int st = it & 1;
                const uint32_t b_lo =
                    smem_desc_lo(smem_u32(sStage + st * 2 * C::TILE + (second ? 0 : C::TILE)), CH);
                const uint32_t ta = second ? TM_DPT : TM_ST;
                const uint32_t td = second ? TM_DK : TM_DV;
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    umma_ts(td, ta + packed_col(k), b_lo + k * 128, hi, id_g, (it | k) != 0 ? 1u : 0u);
            };
            if (ok && !(scores(0, false) && scores(0, true))) {
                atomicExch(p.status, 323);
                ok = false;
            }
            for (int it = 0; it < niter && ok; ++it) {
                if (!mbar_wait(p_full, it & 1)) { atomicExch(p.status, 324); break; }
                tc_fence_after();
                grad(it, false);
                if (it + 1 < niter && !scores(it + 1, false)) { atomicExch(p.status, 325); break; }
                if (!mbar_wait(ds_full, it & 1)) { atomicExch(p.status, 326); break; }
                tc_fence_after();
                grad(it, true);
                umma_commit(&st_empty[it & 1]);
                if (it + 1 < niter && !scores(it + 1, true)) { atomicExch(p.status, 327); break; }
            }
            umma_commit(acc_full);
        }
    } else if (warp >= 4) {
        const int part = (warp - 4) >> 2;                  // which 32-query slice of the block this warp owns
        const int qtr = warp & 3;
        const int row = qtr * 32 + lane;           // key row inside the tile
        const uint32_t lane_base = uint32_t(qtr * 32) << 16;
        const uint32_t col0 = lane_base + part * CPT;
        const int kv = kv0 + row;
        bool ok = true;
        // raw loads only: the first instruction that touches a loaded value stalls the warp until the load returns,
        // so nothing is computed from them before the iteration that uses them
        auto load_stats = [&](int it, float& lse_o, float& dl_o) {
            const int hh = hk * G + it / nq;
            const int q = (ib + it % nq) * 128 + part * CPT + lane;
            const size_t idx = ((size_t)bb * p.hq + hh) * p.sq + min(q, p.sq - 1);
            lse_o = __ldg(p.lse + idx);
            dl_o = __ldg(p.delta + idx);
        };
        float lse_n = 0.f, dl_n = 0.f;
        if (niter > 0) load_stats(0, lse_n, dl_n);
        for (int it = 0; it < niter; ++it) {
            const int h = hk * G + it / nq;
            const int qb0 = (ib + it % nq) * 128;
            const int qc0 = qb0 + part * CPT;
            // lane l holds the statistics of query column l of this warp's slice (broadcast with shuffles below).
            // They were loaded during the previous iteration: a global load issued here would sit on the critical
            // path of the block (measured: ~2800 cycles).
            const bool qin = qc0 + lane < p.sq;
            const float lse_l = qin ? lse_n * LOG2E : INFINITY, dl_l = qin ? dl_n : 0.f;
            if (it + 1 < niter) load_stats(it + 1, lse_n, dl_n);
            const bool need_mask = (kv0 + 127 >= p.sk) || (qb0 + 127 >= p.sq) || (p.causal && kv0 + 127 > qb0 + off) ||
                                   (p.window >= 0 && kv0 < qb0 + 127 + off - p.window);
            const float slope = p.slopes ? p.slopes[h] * LOG2E : 0.f;
            if (!mbar_wait_warp(s_full, it & 1)) {
                if (lane == 0) atomicExch(p.status, 328);
                ok = false;
                break;
            }
            tc_fence_after();
            float pf[CPT];
            {
                uint32_t r[32];
                tmem_ld_32x32(TM_ST + col0, r);
                wait_ld_dep(r);
                // The compute warps are bound by instruction issue (four warps per scheduler, every predicated-off
                // instruction still takes a slot), so the common unmasked block gets a loop of its own.
                if (!(need_mask || p.slopes)) {
#pragma unroll
                    for (int c = 0; c < CPT; ++c)
                        pf[c] = ex2(fmaf(__uint_as_float(r[c]), p.scale_log2, -__shfl_sync(0xffffffffu, lse_l, c)));
                } else {
#pragma unroll
                    for (int c = 0; c < CPT; ++c) {
                        float t = fmaf(__uint_as_float(r[c]), p.scale_log2, -__shfl_sync(0xffffffffu, lse_l, c));
                        const int qpos = qc0 + c + off;
                        if (p.slopes) t -= slope * fabsf((float)(qpos - kv));
                        const bool dead = (kv >= p.sk) || (p.causal && kv > qpos) ||
                                          (p.window >= 0 && kv < qpos - p.window);
                        pf[c] = dead ? 0.f : ex2(t);   // query rows beyond sq have lse = +inf, i.e. 0 already
                    }
                }
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) pk[c] = pack16<FP16>(pf[2 * c], pf[2 * c + 1]);
                tmem_st_32x16(TM_ST + col0, pk);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
            if (!mbar_wait_warp(dp_full, it & 1)) {
                if (lane == 0) atomicExch(p.status, 329);
                ok = false;
                break;
            }
            tc_fence_after();
            {
                uint32_t r[32];
                tmem_ld_32x32(TM_DPT + col0, r);
                wait_ld_dep(r);
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float d0 = pf[2 * c] * (__uint_as_float(r[2 * c]) - __shfl_sync(0xffffffffu, dl_l, 2 * c));
                    const float d1 =
                        pf[2 * c + 1] * (__uint_as_float(r[2 * c + 1]) - __shfl_sync(0xffffffffu, dl_l, 2 * c + 1));
                    pk[c] = pack16<FP16>(d0, d1);
                }
                tmem_st_32x16(TM_DPT + col0, pk);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(ds_full);
        }
        if (niter > 0 && ok) {
            if (!mbar_wait_warp(acc_full, 0)) {
                if (lane == 0) atomicExch(p.status, 330);
                ok = false;
            }
            tc_fence_after();
        }
        ok = __all_sync(0xffffffffu, ok);
        const bool live = kv < p.sk;
        if (ok && part < D / 32) {       // part c writes columns [32c, 32c + 32) of dV and dK
            uint16_t* dkp = reinterpret_cast<uint16_t*>(p.dk) + (long long)(live ? kv : 0) * p.dk_s[0] +
                            bb * p.dk_s[1] + hk * p.dk_s[2] + part * 32;
            uint16_t* dvp = reinterpret_cast<uint16_t*>(p.dv) + (long long)(live ? kv : 0) * p.dv_s[0] +
                            bb * p.dv_s[1] + hk * p.dv_s[2] + part * 32;
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                uint32_t r[32];
                if (niter > 0) {
                    tmem_ld_32x32((which ? TM_DK : TM_DV) + lane_base + part * 32, r);
                    wait_ld_dep(r);
                } else {
#pragma unroll
                    for (int k = 0; k < 32; ++k) r[k] = 0;
                }
                const float sc = which ? p.scale : 1.0f;
                uint16_t* dst = which ? dkp : dvp;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    uint4 q;
                    q.x = pack16<FP16>(__uint_as_float(r[u * 8 + 0]) * sc, __uint_as_float(r[u * 8 + 1]) * sc);
                    q.y = pack16<FP16>(__uint_as_float(r[u * 8 + 2]) * sc, __uint_as_float(r[u * 8 + 3]) * sc);
                    q.z = pack16<FP16>(__uint_as_float(r[u * 8 + 4]) * sc, __uint_as_float(r[u * 8 + 5]) * sc);
                    q.w = pack16<FP16>(__uint_as_float(r[u * 8 + 6]) * sc, __uint_as_float(r[u * 8 + 7]) * sc);
                    if (live) reinterpret_cast<uint4*>(dst)[u] = q;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// =================================================================== dQ
template <int D, bool FP16>
__global__ void __launch_bounds__(THREADS, 1)
flash_bwd2_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                     const Bwd2Params p) {
    using C = B2Cfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem + C::OFF_R0;
    uint8_t* sdO = smem + C::OFF_R1;
    uint8_t* sStage = smem + C::OFF_S;   // stage st: K_j at st*2*TILE, V_j at + TILE
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_MISC);
    uint64_t* q_full = bars;             // 1
    uint64_t* st_full = bars + 1;        // 2
    uint64_t* st_empty = bars + 3;       // 2
    uint64_t* s_full = bars + 5;         // 1  S in TMEM
    uint64_t* s_empty = bars + 6;        // 1  S copied to registers
    uint64_t* dp_full = bars + 7;        // 2  dP in TMEM (double-buffered)
    uint64_t* ds_full = bars + 9;        // 2  dS written over dP
    uint64_t* acc_full = bars + 11;      // 1
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_tile = gridDim.x - 1 - blockIdx.x;
    const int q0 = q_tile * 128;
    const int bb = blockIdx.y / p.hq, h = blockIdx.y % p.hq;
    const int hk = h / (p.hq / p.hkv);
    const int off = p.sk - p.sq;
    int kv_end = p.sk, kv_begin = 0;
    if (p.causal) kv_end = min(p.sk, q0 + 128 + off);
    if (p.window >= 0) kv_begin = max(0, q0 + off - p.window);
    const int jb = kv_begin / 128;
    const int je = (kv_end + 127) / 128;
    const int niter = max(je - jb, 0);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&st_full[i], 1);
            mbar_init(&st_empty[i], 1);
            mbar_init(&dp_full[i], 1);
            mbar_init(&ds_full[i], 4 * PARTS);
        }
        mbar_init(s_full, 1);
        mbar_init(s_empty, 4 * PARTS);
        mbar_init(acc_full, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t TM_S = tmem_base, TM_DP = tmem_base + 128, TM_DQ = tmem_base + 384;

    if (warp == 0) {
        if (lane == 0 && niter > 0) {
            mbar_expect_tx(q_full, 2 * C::TILE);
#pragma unroll
            for (int c = 0; c < C::NCH; ++c) {
                tma_load_4d(sQ + c * CH, &tmQ, q_full, c * 64, h, bb, q0);
                tma_load_4d(sdO + c * CH, &tmdO, q_full, c * 64, h, bb, q0);
            }
            for (int j = 0; j < niter; ++j) {
                const int st = j & 1;
                if (!mbar_wait(&st_empty[st], ((j >> 1) & 1) ^ 1)) {
                    atomicExch(p.status, 341);
                    break;
                }
                const int kvj = (jb + j) * 128;
                mbar_expect_tx(&st_full[st], 2 * C::TILE);
                uint8_t* base = sStage + st * 2 * C::TILE;
#pragma unroll
                for (int c = 0; c < C::NCH; ++c) {
                    tma_load_4d(base + c * CH, &tmK, &st_full[st], c * 64, hk, bb, kvj);
                    tma_load_4d(base + C::TILE + c * CH, &tmV, &st_full[st], c * 64, hk, bb, kvj);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && niter > 0) {
            const uint32_t id_s = idesc16(128, 128, 0, FP16);
            const uint32_t id_g = idesc16(128, D, 1, FP16);
            const uint32_t hi = smem_desc_hi_sw128(1024);
            const uint32_t q_lo = smem_desc_lo(smem_u32(sQ), 16), do_lo = smem_desc_lo(smem_u32(sdO), 16);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicExch(p.status, 342);
            auto scores = [&](int j, bool second) -> bool {      // S = Q K_j^T (first) or dP = dO V_j^T (second)
                const int st = j & 1;
                if (!mbar_wait(&st_full[st], (j >> 1) & 1)) return false;
                if (!second && j > 0 && !mbar_wait(s_empty, (j - 1) & 1)) return false;
                tc_fence_after();
                const uint32_t b_lo = smem_desc_lo(smem_u32(sStage + st * 2 * C::TILE + (second ? C::TILE : 0)), 16);
                const uint32_t a_lo = second ? do_lo : q_lo;
                const uint32_t td = second ? TM_DP + (j & 1) * 128 : TM_S;
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t o = ((k >> 2) * CH + (k & 3) * 32) >> 4;
                    umma_ss_lohi<false, false>(td, a_lo + o, hi, b_lo + o, hi, id_s, k != 0 ? 1u : 0u);
                }
                umma_commit(second ? &dp_full[j & 1] : s_full);
                return true;
            };
            if (ok && !(scores(0, false) && scores(0, true))) {
                atomicExch(p.status, 343);
                ok = false;
            }
            for (int j = 0; j < niter && ok; ++j) {
                if (j + 1 < niter && !(scores(j + 1, false) && scores(j + 1, true))) {
                    atomicExch(p.status, 344);
                    break;
                }
                if (!mbar_wait(&ds_full[j & 1], (j >> 1) & 1)) { atomicExch(p.status, 345); break; }
                tc_fence_after();
                const uint32_t b_lo = smem_desc_lo(smem_u32(sStage + (j & 1) * 2 * C::TILE), CH);   // K_j, MN-major
                const uint32_t ta = TM_DP + (j & 1) * 128;
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    umma_ts(TM_DQ, ta + packed_col(k), b_lo + k * 128, hi, id_g, (j | k) != 0 ? 1u : 0u);
                umma_commit(&st_empty[j & 1]);
            }
            umma_commit(acc_full);
        }
    } else if (warp >= 4) {
        const int part = (warp - 4) >> 2;          // which 32-key slice of the block this warp owns
        const int qtr = warp & 3;
        const int row = qtr * 32 + lane;           // query row inside the tile
        const uint32_t lane_base = uint32_t(qtr * 32) << 16;
        const uint32_t col0 = lane_base + part * CPT;
        const int q = q0 + row;
        const int qpos = q + off;
        const bool qlive = q < p.sq;
        const size_t idx = ((size_t)bb * p.hq + h) * p.sq + (qlive ? q : 0);
        const float lse2 = qlive ? p.lse[idx] * LOG2E : INFINITY;
        const float dl = qlive ? p.delta[idx] : 0.f;
        const float slope = p.slopes ? p.slopes[h] * LOG2E : 0.f;
        bool ok = true;
        for (int j = 0; j < niter; ++j) {
            const int kvb = (jb + j) * 128;
            const int kc0 = kvb + part * CPT;
            const bool need_mask = (kvb + 127 >= p.sk) || (p.causal && kvb + 127 > q0 + off) ||
                                   (p.window >= 0 && kvb < q0 + 127 + off - p.window);
            if (!mbar_wait_warp(s_full, j & 1)) {
                if (lane == 0) atomicExch(p.status, 346);
                ok = false;
                break;
            }
            tc_fence_after();
            float pf[CPT];
            {
                uint32_t r[32];
                tmem_ld_32x32(TM_S + col0, r);
                wait_ld_dep(r);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_empty);
                if (!(need_mask || p.slopes)) {
#pragma unroll
                    for (int c = 0; c < CPT; ++c) pf[c] = ex2(fmaf(__uint_as_float(r[c]), p.scale_log2, -lse2));
                } else {
#pragma unroll
                    for (int c = 0; c < CPT; ++c) {
                        const int kvp = kc0 + c;
                        float t = fmaf(__uint_as_float(r[c]), p.scale_log2, -lse2);
                        if (p.slopes) t -= slope * fabsf((float)(qpos - kvp));
                        const bool dead = (kvp >= p.sk) || (p.causal && kvp > qpos) ||
                                          (p.window >= 0 && kvp < qpos - p.window);
                        pf[c] = dead ? 0.f : ex2(t);
                    }
                }
            }
            const uint32_t TM_DPB = TM_DP + (j & 1) * 128;
            if (!mbar_wait_warp(&dp_full[j & 1], (j >> 1) & 1)) {
                if (lane == 0) atomicExch(p.status, 347);
                ok = false;
                break;
            }
            tc_fence_after();
            {
                uint32_t r[32];
                tmem_ld_32x32(TM_DPB + col0, r);
                wait_ld_dep(r);
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float d0 = pf[2 * c] * (__uint_as_float(r[2 * c]) - dl);
                    const float d1 = pf[2 * c + 1] * (__uint_as_float(r[2 * c + 1]) - dl);
                    pk[c] = pack16<FP16>(d0, d1);
                }
                tmem_st_32x16(TM_DPB + col0, pk);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ds_full[j & 1]);
        }
        if (niter > 0 && ok) {
            if (!mbar_wait_warp(acc_full, 0)) {
                if (lane == 0) atomicExch(p.status, 348);
                ok = false;
            }
            tc_fence_after();
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok && part < D / 32) {
            uint16_t* dqp = reinterpret_cast<uint16_t*>(p.dq) + (long long)(qlive ? q : 0) * p.dq_s[0] +
                            bb * p.dq_s[1] + h * p.dq_s[2] + part * 32;
            uint32_t r[32];
            if (niter > 0) {
                tmem_ld_32x32(TM_DQ + lane_base + part * 32, r);
                wait_ld_dep(r);
            } else {
#pragma unroll
                for (int k = 0; k < 32; ++k) r[k] = 0;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                uint4 v;
                v.x = pack16<FP16>(__uint_as_float(r[u * 8 + 0]) * p.scale, __uint_as_float(r[u * 8 + 1]) * p.scale);
                v.y = pack16<FP16>(__uint_as_float(r[u * 8 + 2]) * p.scale, __uint_as_float(r[u * 8 + 3]) * p.scale);
                v.z = pack16<FP16>(__uint_as_float(r[u * 8 + 4]) * p.scale, __uint_as_float(r[u * 8 + 5]) * p.scale);
                v.w = pack16<FP16>(__uint_as_float(r[u * 8 + 6]) * p.scale, __uint_as_float(r[u * 8 + 7]) * p.scale);
                if (qlive) reinterpret_cast<uint4*>(dqp)[u] = v;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <int D, bool FP16>
int launch_bwd2(const CUtensorMap* t, const Bwd2Params& p, cudaStream_t st) {
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(flash_bwd2_dkv_kernel<D, FP16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 B2Cfg<D>::SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(flash_bwd2_dq_kernel<D, FP16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 B2Cfg<D>::SMEM) != cudaSuccess)
            return NEOX_ERR_LAUNCH;
        attr = true;
    }
    dim3 gkv((p.sk + 127) / 128, p.b * p.hkv);
    flash_bwd2_dkv_kernel<D, FP16><<<gkv, THREADS, B2Cfg<D>::SMEM, st>>>(t[0], t[1], t[2], t[3], p);
    if (cudaGetLastError() != cudaSuccess) return NEOX_ERR_LAUNCH;
    dim3 gq((p.sq + 127) / 128, p.b * p.hq);
    flash_bwd2_dq_kernel<D, FP16><<<gq, THREADS, B2Cfg<D>::SMEM, st>>>(t[0], t[1], t[2], t[3], p);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

}  // namespace

// delta_ws: fp32 scratch of b*hq*sq elements (row sums of dO*O), provided by the caller.  out / dout are contiguous
// [sq, b, hq, d]; dq / dk / dv are [s, b, h, d] views with element strides g_s = {dq_ss, dq_sb, dq_sh, dk_ss, ...,
// dv_sh} (multiples of 8 elements).  dtype: 0 = bf16, 2 = fp16.
extern "C" int neox_flash_bwd2_strided(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                       const float* lse, void* dq, void* dk, void* dv, float* delta_ws, int sq, int sk,
                                       int b, int hq, int hkv, int d, long long q_ss, long long q_sb, long long q_sh,
                                       long long k_ss, long long k_sb, long long k_sh, long long v_ss, long long v_sb,
                                       long long v_sh, const long long* g_s, float scale, int causal, int window,
                                       const float* slopes, int dtype, void* stream) {
    if (d != 64 && d != 96 && d != 128) return NEOX_ERR_SHAPE;
    if (dtype != 0 && dtype != 2) return NEOX_ERR_SHAPE;
    for (int i = 0; i < 9; ++i)
        if (g_s[i] % 8) return NEOX_ERR_ALIGN;
    if ((reinterpret_cast<uintptr_t>(dq) & 15) || (reinterpret_cast<uintptr_t>(dk) & 15) ||
        (reinterpret_cast<uintptr_t>(dv) & 15))
        return NEOX_ERR_ALIGN;
    if (sq <= 0 || sk <= 0 || b <= 0) return 0;
    if (hq % hkv) return NEOX_ERR_SHAPE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long rows = (long long)sq * b * hq;
    const bool h16 = dtype == 2;
    if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(dout) & 15)) return NEOX_ERR_ALIGN;
    const unsigned dblocks = (unsigned)((rows + 15) / 16);
    if (h16)
        delta2_kernel<true><<<dblocks, 256, 0, st>>>(static_cast<const uint4*>(out), static_cast<const uint4*>(dout),
                                                     delta_ws, rows, sq, b, hq, d / 8);
    else
        delta2_kernel<false><<<dblocks, 256, 0, st>>>(static_cast<const uint4*>(out), static_cast<const uint4*>(dout),
                                                      delta_ws, rows, sq, b, hq, d / 8);
    const long long o_sh = d, o_sb = (long long)hq * d, o_ss = (long long)b * hq * d;
    CUtensorMap t[4];
    int rc = 0;
    rc |= neox_make_tmap_bf16_4d(&t[0], q, d, hq, b, sq, q_sh, q_sb, q_ss, 64, 128);
    rc |= neox_make_tmap_bf16_4d(&t[1], k, d, hkv, b, sk, k_sh, k_sb, k_ss, 64, 128);
    rc |= neox_make_tmap_bf16_4d(&t[2], v, d, hkv, b, sk, v_sh, v_sb, v_ss, 64, 128);
    rc |= neox_make_tmap_bf16_4d(&t[3], dout, d, hq, b, sq, o_sh, o_sb, o_ss, 64, 128);
    if (rc) return NEOX_ERR_TMAP;
    Bwd2Params p;
    p.sq = sq; p.sk = sk; p.b = b; p.hq = hq; p.hkv = hkv;
    p.scale = scale; p.scale_log2 = scale * LOG2E;
    p.causal = causal; p.window = window; p.slopes = slopes;
    p.lse = lse; p.delta = delta_ws;
    p.dq = dq; p.dk = dk; p.dv = dv;
    for (int i = 0; i < 3; ++i) {
        p.dq_s[i] = g_s[i];
        p.dk_s[i] = g_s[3 + i];
        p.dv_s[i] = g_s[6 + i];
    }
    p.status = neox_status_word();
    if (!p.status) return NEOX_ERR_DRIVER;
    if (d == 64) return h16 ? launch_bwd2<64, true>(t, p, st) : launch_bwd2<64, false>(t, p, st);
    if (d == 96) return h16 ? launch_bwd2<96, true>(t, p, st) : launch_bwd2<96, false>(t, p, st);
    return h16 ? launch_bwd2<128, true>(t, p, st) : launch_bwd2<128, false>(t, p, st);
}

extern "C" int neox_flash_bwd2(const void* q, const void* k, const void* v, const void* out, const void* dout,
                               const float* lse, void* dq, void* dk, void* dv, float* delta_ws, int sq, int sk, int b,
                               int hq, int hkv, int d, long long q_ss, long long q_sb, long long q_sh, long long k_ss,
                               long long k_sb, long long k_sh, long long v_ss, long long v_sb, long long v_sh,
                               float scale, int causal, int window, const float* slopes, int dtype, void* stream) {
    const long long g_s[9] = {(long long)b * hq * d,  (long long)hq * d,  d, (long long)b * hkv * d, (long long)hkv * d, d,
                              (long long)b * hkv * d, (long long)hkv * d, d};
    return neox_flash_bwd2_strided(q, k, v, out, dout, lse, dq, dk, dv, delta_ws, sq, sk, b, hq, hkv, d, q_ss, q_sb, q_sh,
                                   k_ss, k_sb, k_sh, v_ss, v_sb, v_sh, g_s, scale, causal, window, slopes, dtype, stream);
}
