// Flash attention backward for sm_100a (tcgen05 / TMEM / TMA), three kernels:
//
//   delta      D[b,h,q] = sum_d dO * O                                   (one warp per row)
//   dkv        one CTA per (128-key tile, batch, kv head).  For every 64-query block that can see the tile it
//              forms the TRANSPOSED score tiles  S^T = K Q^T  and  dP^T = V dO^T  (128 keys x 64 queries, so each
//              thread owns one key row), turns them into P^T and dS^T in registers, stores both as bf16 K-major
//              operands and accumulates  dV += P^T dO  and  dK += dS^T Q  in tensor memory across the whole loop
//              (and across the query heads of a GQA group): no atomics, deterministic.
//   dq         one CTA per (128-query tile, batch, head); loops over 64-key blocks:  S = Q K^T,  dP = dO V^T,
//              dS in registers (thread = query row, so lse and D are per-thread scalars),  dQ += dS K  in TMEM.
//
// The Q / dO (resp. K / V) tiles are loaded once per iteration by TMA and used twice with different operand
// descriptors: K-major for the score GEMMs (contraction over the head dimension) and MN-major for the gradient
// GEMMs (contraction over the 64 rows).  Recomputing S in both kernels costs two extra GEMMs but keeps every
// accumulator resident and the result bit-reproducible.  All waits are bounded.
#include "sm100_ptx.cuh"
#include "neox_b200.h"
#include <math.h>

using namespace sm100;

namespace {

constexpr int CH128 = 128 * 128;  // [128 rows x 64 bf16] swizzled chunk
constexpr int CH64 = 64 * 128;    // [ 64 rows x 64 bf16] swizzled chunk
constexpr float LOG2E = 1.4426950408889634f;

struct BwdParams {
    int sq, sk, b, hq, hkv, d;
    float scale, scale_log2;
    int causal, window;
    const float* slopes;
    const float* lse;    // [b, hq, sq] natural log
    const float* delta;  // [b, hq, sq]
    __nv_bfloat16 *dq, *dk, *dv;  // [s, b, h, d] views; element strides of (s, b, h) below, d contiguous
    long long dq_s[3], dk_s[3], dv_s[3];
    int* status;
};

// ------------------------------------------------------------------ delta
__global__ void __launch_bounds__(256) delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                                    float* __restrict__ delta, int sq, int b, int hq, int d) {
    const long long row = blockIdx.x * 8LL + (threadIdx.x >> 5);  // row over [sq, b, hq]
    const long long rows = (long long)sq * b * hq;
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const __nv_bfloat16* op = o + row * d;
    const __nv_bfloat16* gp = dout + row * d;
    float s = 0.f;
    for (int c = lane; c < d; c += 32) s += __bfloat162float(op[c]) * __bfloat162float(gp[c]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) {
        const int h = (int)(row % hq);
        const long long t = row / hq;
        const int bb = (int)(t % b);
        const int q = (int)(t / b);
        delta[((size_t)bb * hq + h) * sq + q] = s;
    }
}

__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld_32x32(taddr, r); }
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld_32x16(taddr, r); }

constexpr int PARTS = 4;                           // softmax warps per TMEM lane quarter
constexpr int CPT = 64 / PARTS;                    // score columns per softmax thread
constexpr int BWD_THREADS = 128 + PARTS * 128;     // warp 0 TMA, warp 1 MMA, warps 4.. softmax

// CPT bf16 values (columns part * CPT ...) of one row into a K-major swizzled [rows x 64] chunk (row pitch 128 bytes).
__device__ __forceinline__ void store_row_part(uint8_t* chunk, int row, int part, const float (&v)[CPT]) {
#pragma unroll
    for (int u = 0; u < CPT / 8; ++u) {
        uint4 q;
        q.x = pack_bf16x2(v[u * 8 + 0], v[u * 8 + 1]);
        q.y = pack_bf16x2(v[u * 8 + 2], v[u * 8 + 3]);
        q.z = pack_bf16x2(v[u * 8 + 4], v[u * 8 + 5]);
        q.w = pack_bf16x2(v[u * 8 + 6], v[u * 8 + 7]);
        *reinterpret_cast<uint4*>(chunk + row * 128 + (((part * (CPT / 8) + u) ^ (row & 7)) << 4)) = q;
    }
}

template <int D>
struct BCfg {
    static constexpr int NCH = (D == 64) ? 1 : 2;
    static constexpr int BIG = NCH * CH128;    // resident 128-row tile
    static constexpr int SMALL = NCH * CH64;   // streamed 64-row tile
    static constexpr int OFF_R0 = 0;                    // resident tile 0 (K in dkv, Q in dq)
    static constexpr int OFF_R1 = BIG;                  // resident tile 1 (V in dkv, dO in dq)
    static constexpr int OFF_S = 2 * BIG;               // 2 stages x (tile a, tile b)
    static constexpr int OFF_A0 = OFF_S + 4 * SMALL;    // bf16 operand written by the compute group (P^T / dS)
    static constexpr int OFF_A1 = OFF_A0 + CH128;       // second operand (dS^T), dkv only
    static constexpr int OFF_MISC = OFF_A1 + CH128;
    static constexpr int SMEM = OFF_MISC + 4096 + 1024;
};

// =================================================================== dK / dV
template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                     const BwdParams p) {
    using C = BCfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem + C::OFF_R0;
    uint8_t* sV = smem + C::OFF_R1;
    uint8_t* sStage = smem + C::OFF_S;   // stage st: Q at st*2*SMALL, dO at st*2*SMALL + SMALL
    uint8_t* sPt = smem + C::OFF_A0;
    uint8_t* sdSt = smem + C::OFF_A1;
    float* s_lse = reinterpret_cast<float*>(smem + C::OFF_MISC);   // [4 warps][64] (log2 domain)
    float* s_dl = s_lse + 256;                                      // [4 warps][64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_dl + 256);
    uint64_t* kv_full = bars;            // 1
    uint64_t* st_full = bars + 1;        // 2  Q_i / dO_i landed
    uint64_t* st_empty = bars + 3;       // 2
    uint64_t* sdp_full = bars + 5;       // 2  S^T, dP^T ready in TMEM (double-buffered)
    uint64_t* sdp_empty = bars + 7;      // 2
    uint64_t* pds_full = bars + 9;       // 1  P^T, dS^T written to smem
    uint64_t* pds_empty = bars + 10;     // 1
    uint64_t* acc_full = bars + 11;      // 1  dK, dV final
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kv0 = blockIdx.x * 128;
    const int bb = blockIdx.y / p.hkv, hk = blockIdx.y % p.hkv;
    const int G = p.hq / p.hkv;
    const int off = p.sk - p.sq;
    // query blocks (of 64) that can attend to this key tile
    int q_lo = 0, q_hi = p.sq;
    if (p.causal) q_lo = max(0, kv0 - off);
    if (p.window >= 0) q_hi = min(p.sq, kv0 + 127 - off + p.window + 1);
    const int ib = q_lo / 64;
    const int ie = (q_hi + 63) / 64;
    const int nq = max(ie - ib, 0);
    const int niter = nq * G;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&st_full[i], 1);
            mbar_init(&st_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sdp_full[i], 1);
            mbar_init(&sdp_empty[i], 4 * PARTS);
        }
        mbar_init(pds_full, 4 * PARTS);
        mbar_init(pds_empty, 1);
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
    // Two score buffers (S^T | dP^T, 64 columns each) so that the scores of query block i + 1 are computed while
    // the softmax warps work on block i; dV and dK accumulate behind them.
    const uint32_t TM_SC = tmem_base, TM_DV = tmem_base + 256, TM_DK = tmem_base + 384;

    if (warp == 0) {
        if (lane == 0 && niter > 0) {
            mbar_expect_tx(kv_full, 2 * C::BIG);
#pragma unroll
            for (int c = 0; c < C::NCH; ++c) {
                tma_load_4d(sK + c * CH128, &tmK, kv_full, c * 64, hk, bb, kv0);
                tma_load_4d(sV + c * CH128, &tmV, kv_full, c * 64, hk, bb, kv0);
            }
            for (int it = 0; it < niter; ++it) {
                const int st = it & 1;
                if (!mbar_wait(&st_empty[st], ((it >> 1) & 1) ^ 1)) {
                    atomicExch(p.status, 301);
                    break;
                }
                const int h = hk * G + it / nq;
                const int qi0 = (ib + it % nq) * 64;
                mbar_expect_tx(&st_full[st], 2 * C::SMALL);
                uint8_t* base = sStage + st * 2 * C::SMALL;
#pragma unroll
                for (int c = 0; c < C::NCH; ++c) {
                    tma_load_4d(base + c * CH64, &tmQ, &st_full[st], c * 64, h, bb, qi0);
                    tma_load_4d(base + C::SMALL + c * CH64, &tmdO, &st_full[st], c * 64, h, bb, qi0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && niter > 0) {
            const uint32_t id_s = make_idesc_bf16(128, 64, 0, 0);    // S^T = K Q^T   (both K-major)
            const uint32_t id_g = make_idesc_bf16(128, D, 0, 1);     // dV = P^T dO   (B MN-major)
            const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV);
            const uint32_t pt_base = smem_u32(sPt), dst_base = smem_u32(sdSt);
            bool ok = mbar_wait(kv_full, 0);
            if (!ok) atomicExch(p.status, 302);
            auto issue_scores = [&](int it) -> bool {
                const int st = it & 1;
                if (!mbar_wait(&st_full[st], (it >> 1) & 1)) return false;
                if (!mbar_wait(&sdp_empty[st], ((it >> 1) & 1) ^ 1)) return false;
                tc_fence_after();
                const uint32_t TM_ST = TM_SC + st * 128, TM_DPT = TM_ST + 64;
                const uint32_t q_base = smem_u32(sStage + st * 2 * C::SMALL);
                const uint32_t do_base = q_base + C::SMALL;
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t oa = (k >> 2) * CH128 + (k & 3) * 32, ob = (k >> 2) * CH64 + (k & 3) * 32;
                    umma_bf16_ss(TM_ST, make_smem_desc_sw128(k_base + oa, 16, 1024),
                                 make_smem_desc_sw128(q_base + ob, 16, 1024), id_s, k != 0);
                }
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t oa = (k >> 2) * CH128 + (k & 3) * 32, ob = (k >> 2) * CH64 + (k & 3) * 32;
                    umma_bf16_ss(TM_DPT, make_smem_desc_sw128(v_base + oa, 16, 1024),
                                 make_smem_desc_sw128(do_base + ob, 16, 1024), id_s, k != 0);
                }
                umma_commit(&sdp_full[st]);
                return true;
            };
            if (ok && !issue_scores(0)) {
                atomicExch(p.status, 303);
                ok = false;
            }
            for (int it = 0; it < niter && ok; ++it) {
                const int st = it & 1;
                // scores of the next query block first: the softmax warps can start on them as soon as they are
                // done with this one, while the tensor core runs this block's dV / dK products
                if (it + 1 < niter && !issue_scores(it + 1)) {
                    atomicExch(p.status, 305);
                    ok = false;
                    break;
                }
                if (!mbar_wait(pds_full, it & 1)) {
                    atomicExch(p.status, 304);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t q_base = smem_u32(sStage + st * 2 * C::SMALL);
                const uint32_t do_base = q_base + C::SMALL;
#pragma unroll
                for (int k = 0; k < 4; ++k) {   // contraction over the 64 query rows
                    umma_bf16_ss(TM_DV, make_smem_desc_sw128(pt_base + k * 32, 16, 1024),
                                 make_smem_desc_sw128(do_base + k * 2048, CH64, 1024), id_g, (it | k) != 0);
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    umma_bf16_ss(TM_DK, make_smem_desc_sw128(dst_base + k * 32, 16, 1024),
                                 make_smem_desc_sw128(q_base + k * 2048, CH64, 1024), id_g, (it | k) != 0);
                }
                umma_commit(&st_empty[st]);
                umma_commit(pds_empty);
            }
            umma_commit(acc_full);
        }
    } else if (warp >= 4) {
        // Two warps share each TMEM lane quarter (= 32 key rows): warps 4-7 take query columns 0-31 of the block,
        // warps 8-11 columns 32-63, which halves the per-thread work and doubles the warps available to hide latency.
        const int cw = warp - 4;
        const int half = cw >> 2;                 // which CPT-column slice of the block this warp owns
        const int row = (warp & 3) * 32 + lane;    // key row inside the tile
        float* my_lse = s_lse + cw * CPT;          // per-warp staging: only warp-level syncs are needed
        float* my_dl = s_dl + cw * CPT;
        const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
        const int kv = kv0 + row;
        bool ok = true;
        for (int it = 0; it < niter; ++it) {
            const int h = hk * G + it / nq;
            const int qi0 = (ib + it % nq) * 64 + half * CPT;
            __syncwarp();
            if (lane < CPT) {
                const int q = qi0 + lane;
                const size_t idx = ((size_t)bb * p.hq + h) * p.sq + q;
                my_lse[lane] = (q < p.sq) ? p.lse[idx] * LOG2E : INFINITY;
                my_dl[lane] = (q < p.sq) ? p.delta[idx] : 0.f;
            }
            __syncwarp();
            if (!mbar_wait_warp(&sdp_full[it & 1], (it >> 1) & 1)) {
                if (lane == 0) atomicExch(p.status, 306);
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t TM_ST = TM_SC + (it & 1) * 128, TM_DPT = TM_ST + 64;
            float pt[CPT], ds[CPT];
            {
                uint32_t r[CPT], r2[CPT];
                tmem_ld_cols(TM_ST + lane_base + half * CPT, r);
                tmem_ld_cols(TM_DPT + lane_base + half * CPT, r2);
                tmem_wait_ld();
#pragma unroll
                for (int k = 0; k < CPT; ++k) {
                    pt[k] = __uint_as_float(r[k]);
                    ds[k] = __uint_as_float(r2[k]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sdp_empty[it & 1]);
            const float slope = p.slopes ? p.slopes[h] * LOG2E : 0.f;
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int q = qi0 + c;
                const int qpos = q + off;
                float t = pt[c] * p.scale_log2;
                if (p.slopes) t -= slope * fabsf((float)(qpos - kv));
                const bool dead = (kv >= p.sk) || (q >= p.sq) || (p.causal && kv > qpos) ||
                                  (p.window >= 0 && kv < qpos - p.window);
                const float pv = dead ? 0.f : exp2f(t - my_lse[c]);
                pt[c] = pv;
                ds[c] = pv * (ds[c] - my_dl[c]) * p.scale;
            }
            if (!mbar_wait_warp(pds_empty, (it & 1) ^ 1)) {
                if (lane == 0) atomicExch(p.status, 307);
                ok = false;
                break;
            }
            store_row_part(sPt, row, half, pt);
            store_row_part(sdSt, row, half, ds);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(pds_full);
        }
        if (niter > 0 && ok) {
            if (!mbar_wait_warp(acc_full, 0)) {
                if (lane == 0) atomicExch(p.status, 308);
                ok = false;
            }
            tc_fence_after();
        }
        // tcgen05.ld is warp-collective (.sync.aligned): every lane of the warp must execute it, so the loads are
        // guarded by warp-uniform conditions only and the per-row bound check applies to the stores.
        ok = __all_sync(0xffffffffu, ok);
        const bool live = kv < p.sk;
        if (ok && half == 0) {       // one warp per lane quarter writes the accumulators out
            __nv_bfloat16* dkp = p.dk + (long long)(live ? kv : 0) * p.dk_s[0] + bb * p.dk_s[1] + hk * p.dk_s[2];
            __nv_bfloat16* dvp = p.dv + (long long)(live ? kv : 0) * p.dv_s[0] + bb * p.dv_s[1] + hk * p.dv_s[2];
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t r[32];
                uint4 q;
                if (niter > 0) {
                    tmem_ld_cols(TM_DV + lane_base + c * 32, r);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int k = 0; k < 32; ++k) r[k] = 0;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    q.x = pack_bf16x2(__uint_as_float(r[u * 8 + 0]), __uint_as_float(r[u * 8 + 1]));
                    q.y = pack_bf16x2(__uint_as_float(r[u * 8 + 2]), __uint_as_float(r[u * 8 + 3]));
                    q.z = pack_bf16x2(__uint_as_float(r[u * 8 + 4]), __uint_as_float(r[u * 8 + 5]));
                    q.w = pack_bf16x2(__uint_as_float(r[u * 8 + 6]), __uint_as_float(r[u * 8 + 7]));
                    if (live) reinterpret_cast<uint4*>(dvp + c * 32)[u] = q;
                }
                if (niter > 0) {
                    tmem_ld_cols(TM_DK + lane_base + c * 32, r);
                    tmem_wait_ld();
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    q.x = pack_bf16x2(__uint_as_float(r[u * 8 + 0]), __uint_as_float(r[u * 8 + 1]));
                    q.y = pack_bf16x2(__uint_as_float(r[u * 8 + 2]), __uint_as_float(r[u * 8 + 3]));
                    q.z = pack_bf16x2(__uint_as_float(r[u * 8 + 4]), __uint_as_float(r[u * 8 + 5]));
                    q.w = pack_bf16x2(__uint_as_float(r[u * 8 + 6]), __uint_as_float(r[u * 8 + 7]));
                    if (live) reinterpret_cast<uint4*>(dkp + c * 32)[u] = q;
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
template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const BwdParams p) {
    using C = BCfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem + C::OFF_R0;
    uint8_t* sdO = smem + C::OFF_R1;
    uint8_t* sStage = smem + C::OFF_S;   // stage st: K_j at st*2*SMALL, V_j at + SMALL
    uint8_t* sdS = smem + C::OFF_A0;     // [128 q x 64 kv] K-major
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_MISC);
    uint64_t* q_full = bars;
    uint64_t* st_full = bars + 1;
    uint64_t* st_empty = bars + 3;
    uint64_t* sdp_full = bars + 5;       // 2  S, dP ready in TMEM (double-buffered)
    uint64_t* sdp_empty = bars + 7;      // 2
    uint64_t* ds_full = bars + 9;
    uint64_t* ds_empty = bars + 10;
    uint64_t* acc_full = bars + 11;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_tile = gridDim.x - 1 - blockIdx.x;
    const int q0 = q_tile * 128;
    const int bb = blockIdx.y / p.hq, h = blockIdx.y % p.hq;
    const int hk = h / (p.hq / p.hkv);
    const int off = p.sk - p.sq;
    int kv_end = p.sk;
    if (p.causal) kv_end = min(p.sk, q0 + 128 + off);
    int kv_begin = 0;
    if (p.window >= 0) kv_begin = max(0, q0 + off - p.window);
    const int jb = kv_begin / 64;
    const int je = (kv_end + 63) / 64;
    const int niter = max(je - jb, 0);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&st_full[i], 1);
            mbar_init(&st_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sdp_full[i], 1);
            mbar_init(&sdp_empty[i], 4 * PARTS);
        }
        mbar_init(ds_full, 4 * PARTS);
        mbar_init(ds_empty, 1);
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
    // two score buffers (S | dP, 64 columns each): the scores of key block j + 1 are computed while the softmax warps
    // work on block j; dQ accumulates behind them
    const uint32_t TM_SC = tmem_base, TM_DQ = tmem_base + 256;

    if (warp == 0) {
        if (lane == 0 && niter > 0) {
            mbar_expect_tx(q_full, 2 * C::BIG);
#pragma unroll
            for (int c = 0; c < C::NCH; ++c) {
                tma_load_4d(sQ + c * CH128, &tmQ, q_full, c * 64, h, bb, q0);
                tma_load_4d(sdO + c * CH128, &tmdO, q_full, c * 64, h, bb, q0);
            }
            for (int it = 0; it < niter; ++it) {
                const int st = it & 1;
                if (!mbar_wait(&st_empty[st], ((it >> 1) & 1) ^ 1)) {
                    atomicExch(p.status, 311);
                    break;
                }
                const int kvj = (jb + it) * 64;
                mbar_expect_tx(&st_full[st], 2 * C::SMALL);
                uint8_t* base = sStage + st * 2 * C::SMALL;
#pragma unroll
                for (int c = 0; c < C::NCH; ++c) {
                    tma_load_4d(base + c * CH64, &tmK, &st_full[st], c * 64, hk, bb, kvj);
                    tma_load_4d(base + C::SMALL + c * CH64, &tmV, &st_full[st], c * 64, hk, bb, kvj);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && niter > 0) {
            const uint32_t id_s = make_idesc_bf16(128, 64, 0, 0);
            const uint32_t id_g = make_idesc_bf16(128, D, 0, 1);
            const uint32_t q_base = smem_u32(sQ), do_base = smem_u32(sdO), ds_base = smem_u32(sdS);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicExch(p.status, 312);
            auto issue_scores = [&](int it) -> bool {
                const int st = it & 1;
                if (!mbar_wait(&st_full[st], (it >> 1) & 1)) return false;
                if (!mbar_wait(&sdp_empty[st], ((it >> 1) & 1) ^ 1)) return false;
                tc_fence_after();
                const uint32_t TM_S = TM_SC + st * 128, TM_DP = TM_S + 64;
                const uint32_t k_base = smem_u32(sStage + st * 2 * C::SMALL);
                const uint32_t v_base = k_base + C::SMALL;
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t oa = (k >> 2) * CH128 + (k & 3) * 32, ob = (k >> 2) * CH64 + (k & 3) * 32;
                    umma_bf16_ss(TM_S, make_smem_desc_sw128(q_base + oa, 16, 1024),
                                 make_smem_desc_sw128(k_base + ob, 16, 1024), id_s, k != 0);
                }
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t oa = (k >> 2) * CH128 + (k & 3) * 32, ob = (k >> 2) * CH64 + (k & 3) * 32;
                    umma_bf16_ss(TM_DP, make_smem_desc_sw128(do_base + oa, 16, 1024),
                                 make_smem_desc_sw128(v_base + ob, 16, 1024), id_s, k != 0);
                }
                umma_commit(&sdp_full[st]);
                return true;
            };
            if (ok && !issue_scores(0)) {
                atomicExch(p.status, 313);
                ok = false;
            }
            for (int it = 0; it < niter && ok; ++it) {
                const int st = it & 1;
                if (it + 1 < niter && !issue_scores(it + 1)) {      // next block's scores before this block's dQ
                    atomicExch(p.status, 315);
                    ok = false;
                    break;
                }
                if (!mbar_wait(ds_full, it & 1)) {
                    atomicExch(p.status, 314);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t k_base = smem_u32(sStage + st * 2 * C::SMALL);
#pragma unroll
                for (int k = 0; k < 4; ++k) {   // contraction over the 64 keys
                    umma_bf16_ss(TM_DQ, make_smem_desc_sw128(ds_base + k * 32, 16, 1024),
                                 make_smem_desc_sw128(k_base + k * 2048, CH64, 1024), id_g, (it | k) != 0);
                }
                umma_commit(&st_empty[st]);
                umma_commit(ds_empty);
            }
            umma_commit(acc_full);
        }
    } else if (warp >= 4) {
        // two warps per TMEM lane quarter (32 query rows): warps 4-7 take key columns 0-31 of the block, 8-11 the rest
        const int half = (warp - 4) >> 2;
        const int row = (warp & 3) * 32 + lane;
        const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
        const int q = q0 + row;
        const int qpos = q + off;
        const size_t sidx = ((size_t)bb * p.hq + h) * p.sq + q;
        const float lse2 = (q < p.sq) ? p.lse[sidx] * LOG2E : INFINITY;
        const float dl = (q < p.sq) ? p.delta[sidx] : 0.f;
        const float slope = p.slopes ? p.slopes[h] * LOG2E : 0.f;
        bool ok = true;
        for (int it = 0; it < niter; ++it) {
            const int kvj = (jb + it) * 64 + half * CPT;
            if (!mbar_wait_warp(&sdp_full[it & 1], (it >> 1) & 1)) {
                if (lane == 0) atomicExch(p.status, 316);
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t TM_S = TM_SC + (it & 1) * 128, TM_DP = TM_S + 64;
            float pt[CPT], ds[CPT];
            {
                uint32_t r[CPT], r2[CPT];
                tmem_ld_cols(TM_S + lane_base + half * CPT, r);
                tmem_ld_cols(TM_DP + lane_base + half * CPT, r2);
                tmem_wait_ld();
#pragma unroll
                for (int k = 0; k < CPT; ++k) {
                    pt[k] = __uint_as_float(r[k]);
                    ds[k] = __uint_as_float(r2[k]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sdp_empty[it & 1]);
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int kv = kvj + c;
                float t = pt[c] * p.scale_log2;
                if (p.slopes) t -= slope * fabsf((float)(qpos - kv));
                const bool dead = (kv >= p.sk) || (q >= p.sq) || (p.causal && kv > qpos) ||
                                  (p.window >= 0 && kv < qpos - p.window);
                const float pv = dead ? 0.f : exp2f(t - lse2);
                ds[c] = pv * (ds[c] - dl) * p.scale;
            }
            if (!mbar_wait_warp(ds_empty, (it & 1) ^ 1)) {
                if (lane == 0) atomicExch(p.status, 317);
                ok = false;
                break;
            }
            store_row_part(sdS, row, half, ds);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(ds_full);
        }
        if (niter > 0 && ok) {
            if (!mbar_wait_warp(acc_full, 0)) {
                if (lane == 0) atomicExch(p.status, 318);
                ok = false;
            }
            tc_fence_after();
        }
        ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld below is warp-collective
        const bool live = q < p.sq;
        if (ok && half == 0) {
            __nv_bfloat16* dqp = p.dq + (long long)(live ? q : 0) * p.dq_s[0] + bb * p.dq_s[1] + h * p.dq_s[2];
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t r[32];
                if (niter > 0) {
                    tmem_ld_cols(TM_DQ + lane_base + c * 32, r);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int k = 0; k < 32; ++k) r[k] = 0;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    uint4 qv;
                    qv.x = pack_bf16x2(__uint_as_float(r[u * 8 + 0]), __uint_as_float(r[u * 8 + 1]));
                    qv.y = pack_bf16x2(__uint_as_float(r[u * 8 + 2]), __uint_as_float(r[u * 8 + 3]));
                    qv.z = pack_bf16x2(__uint_as_float(r[u * 8 + 4]), __uint_as_float(r[u * 8 + 5]));
                    qv.w = pack_bf16x2(__uint_as_float(r[u * 8 + 6]), __uint_as_float(r[u * 8 + 7]));
                    if (live) reinterpret_cast<uint4*>(dqp + c * 32)[u] = qv;
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

template <int D>
int launch_bwd(const CUtensorMap (&t)[8], const BwdParams& p, cudaStream_t st) {
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(flash_bwd_dkv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, BCfg<D>::SMEM) != cudaSuccess ||
            cudaFuncSetAttribute(flash_bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, BCfg<D>::SMEM) != cudaSuccess)
            return NEOX_ERR_LAUNCH;
        attr = true;
    }
    dim3 g1((p.sk + 127) / 128, p.b * p.hkv);
    flash_bwd_dkv_kernel<D><<<g1, BWD_THREADS, BCfg<D>::SMEM, st>>>(t[0], t[1], t[2], t[3], p);
    dim3 g2((p.sq + 127) / 128, p.b * p.hq);
    flash_bwd_dq_kernel<D><<<g2, BWD_THREADS, BCfg<D>::SMEM, st>>>(t[4], t[5], t[6], t[7], p);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

}  // namespace

// delta_ws: fp32 scratch of b*hq*sq elements (row sums of dO*O), provided by the caller.
// dq / dk / dv are [s, b, h, d] views with element strides g_s = {dq_ss, dq_sb, dq_sh, dk_ss, ..., dv_sh}; rows must be
// 16-byte aligned (strides multiples of 8 elements).
extern "C" int neox_flash_bwd_strided(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                      const float* lse, void* dq, void* dk, void* dv, float* delta_ws, int sq, int sk,
                                      int b, int hq, int hkv, int d, long long q_ss, long long q_sb, long long q_sh,
                                      long long k_ss, long long k_sb, long long k_sh, long long v_ss, long long v_sb,
                                      long long v_sh, const long long* g_s, float scale, int causal, int window,
                                      const float* slopes, void* stream);

extern "C" int neox_flash_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                              const float* lse, void* dq, void* dk, void* dv, float* delta_ws, int sq, int sk, int b,
                              int hq, int hkv, int d, long long q_ss, long long q_sb, long long q_sh, long long k_ss,
                              long long k_sb, long long k_sh, long long v_ss, long long v_sb, long long v_sh,
                              float scale, int causal, int window, const float* slopes, void* stream) {
    const long long g_s[9] = {(long long)b * hq * d,  (long long)hq * d,  d, (long long)b * hkv * d, (long long)hkv * d, d,
                              (long long)b * hkv * d, (long long)hkv * d, d};
    return neox_flash_bwd_strided(q, k, v, out, dout, lse, dq, dk, dv, delta_ws, sq, sk, b, hq, hkv, d, q_ss, q_sb, q_sh,
                                  k_ss, k_sb, k_sh, v_ss, v_sb, v_sh, g_s, scale, causal, window, slopes, stream);
}

extern "C" int neox_flash_bwd_strided(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                      const float* lse, void* dq, void* dk, void* dv, float* delta_ws, int sq, int sk,
                                      int b, int hq, int hkv, int d, long long q_ss, long long q_sb, long long q_sh,
                                      long long k_ss, long long k_sb, long long k_sh, long long v_ss, long long v_sb,
                                      long long v_sh, const long long* g_s, float scale, int causal, int window,
                                      const float* slopes, void* stream) {
    if (d != 64 && d != 96 && d != 128) return NEOX_ERR_SHAPE;
    for (int i = 0; i < 9; ++i)
        if (g_s[i] % 8) return NEOX_ERR_ALIGN;
    if ((reinterpret_cast<uintptr_t>(dq) & 15) || (reinterpret_cast<uintptr_t>(dk) & 15) ||
        (reinterpret_cast<uintptr_t>(dv) & 15))
        return NEOX_ERR_ALIGN;
    if (sq <= 0 || sk <= 0 || b <= 0) return 0;
    if (hq % hkv) return NEOX_ERR_SHAPE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long rows = (long long)sq * b * hq;
    delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(out),
                                                             static_cast<const __nv_bfloat16*>(dout), delta_ws, sq, b,
                                                             hq, d);
    // dO is contiguous [sq, b, hq, d]
    const long long o_sh = d, o_sb = (long long)hq * d, o_ss = (long long)b * hq * d;
    CUtensorMap t[8];
    int rc = 0;
    // dkv kernel: Q and dO streamed in 64-row boxes, K and V resident 128-row boxes
    rc |= neox_make_tmap_bf16_4d(&t[0], q, d, hq, b, sq, q_sh, q_sb, q_ss, 64, 64);
    rc |= neox_make_tmap_bf16_4d(&t[1], k, d, hkv, b, sk, k_sh, k_sb, k_ss, 64, 128);
    rc |= neox_make_tmap_bf16_4d(&t[2], v, d, hkv, b, sk, v_sh, v_sb, v_ss, 64, 128);
    rc |= neox_make_tmap_bf16_4d(&t[3], dout, d, hq, b, sq, o_sh, o_sb, o_ss, 64, 64);
    // dq kernel: Q and dO resident 128-row boxes, K and V streamed in 64-row boxes
    rc |= neox_make_tmap_bf16_4d(&t[4], q, d, hq, b, sq, q_sh, q_sb, q_ss, 64, 128);
    rc |= neox_make_tmap_bf16_4d(&t[5], k, d, hkv, b, sk, k_sh, k_sb, k_ss, 64, 64);
    rc |= neox_make_tmap_bf16_4d(&t[6], v, d, hkv, b, sk, v_sh, v_sb, v_ss, 64, 64);
    rc |= neox_make_tmap_bf16_4d(&t[7], dout, d, hq, b, sq, o_sh, o_sb, o_ss, 64, 128);
    if (rc) return NEOX_ERR_TMAP;
    BwdParams p;
    p.sq = sq; p.sk = sk; p.b = b; p.hq = hq; p.hkv = hkv; p.d = d;
    p.scale = scale; p.scale_log2 = scale * LOG2E;
    p.causal = causal; p.window = window; p.slopes = slopes;
    p.lse = lse; p.delta = delta_ws;
    p.dq = static_cast<__nv_bfloat16*>(dq); p.dk = static_cast<__nv_bfloat16*>(dk); p.dv = static_cast<__nv_bfloat16*>(dv);
    for (int i = 0; i < 3; ++i) {
        p.dq_s[i] = g_s[i];
        p.dk_s[i] = g_s[3 + i];
        p.dv_s[i] = g_s[6 + i];
    }
    p.status = neox_status_word();
    if (!p.status) return NEOX_ERR_DRIVER;
    if (d == 64) return launch_bwd<64>(t, p, st);
    if (d == 96) return launch_bwd<96>(t, p, st);
    return launch_bwd<128>(t, p, st);
}
