// Flash attention forward for sm_100a, two query tiles per CTA (the default forward kernel).
//
// A CTA owns 256 query rows of one (batch, head): two 128-row tiles whose softmax warpgroups alternate, so that
// the tensor pipe always has a QK^T or a PV of the other tile in flight while one tile's exponentials are computed.
//
//   warp 0        TMA producer: both Q tiles once, then K and V tiles of 128 keys through two 2-stage rings
//                 (4-D tensor maps over the strided [s, b, h, d] views: the fused QKV projection is read in place);
//   warp 1        MMA issuer (one thread).  Per key block g:  PV_0(g), QK_0(g+1), PV_1(g), QK_1(g+1).
//                 S_i = Q_i K^T goes to a 128-column TMEM accumulator; O_i += P_i V accumulates in TMEM over all key
//                 blocks, with P_i read from TENSOR MEMORY (A operand of tcgen05.mma): the softmax warps store P as
//                 packed 16-bit pairs over the first 64 columns of S_i, no shared-memory round trip;
//   warps 4-7     softmax of tile 0, warps 8-11 softmax of tile 1: a thread owns one query row and holds its 128
//                 scores in registers (four tcgen05.ld 32x32b in flight, one wait; these warpgroups raise their
//                 register allowance with setmaxnreg, the others lower theirs): row maximum, exp2, row sum, pack,
//                 store; masks (causal, sliding window, key tail) and ALiBi generated in registers;
//   warps 12-15   correction: O_i is rescaled in tensor memory only when a row maximum of the warp's 32 rows grew by
//                 more than 2^8 since the last rescale (the stale maximum stays the exponent reference otherwise, which
//                 is exact after the final division by the row sum); final 1/l scaling and the 16-bit store of O.
//
// TMEM: S_0 | S_1 | O_0 | O_1, 128 columns each.  Head sizes 64 / 96 / 128, bf16 or fp16 operands, grouped-query
// attention (kv head = q head / (hq / hkv)), bottom-right aligned causal mask when sq < sk.
//
// Replaces the flash-attn 2 calls of megatron/model/transformer.py:627-744.  Every wait is bounded.
#include "sm100_ptx.cuh"
#include "neox_b200.h"
#include <cuda_fp16.h>
#include <math.h>

using namespace sm100;

namespace {

constexpr int BM = 128;                  // rows per query tile
constexpr int BN = 128;                  // keys per block
constexpr int CHUNK_BYTES = 128 * 128;   // one [128 rows x 64 x 16-bit] swizzled chunk
constexpr int THREADS = 512;
constexpr float RESCALE_THRESHOLD = 8.0f;   // log2 units

struct Fwd2Params {
    int sq, sk, b, hq, hkv;
    float scale_log2;      // softmax scale * log2(e)
    int causal, window;
    const float* slopes;   // ALiBi slopes per q head (nullable)
    void* out;             // [sq, b, hq, d] contiguous, 16-bit
    float* lse;            // [b, hq, sq]
    int* status;
};

template <int D>
struct Cfg2 {
    static constexpr int NCH = (D == 64) ? 1 : 2;
    static constexpr int TILE = NCH * CHUNK_BYTES;
    static constexpr int OFF_Q = 0;                    // 2 tiles
    static constexpr int OFF_K = 2 * TILE;             // 2 stages
    static constexpr int OFF_V = OFF_K + 2 * TILE;     // 2 stages
    static constexpr int OFF_MISC = OFF_V + 2 * TILE;
    static constexpr int MISC_BYTES = 4096;
    static constexpr int SMEM = OFF_MISC + MISC_BYTES + 1024;
};

__device__ __forceinline__ float max3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// tcgen05.wait::ld that also "redefines" the destination registers of the loads it completes, so the compiler cannot
// schedule a use of those registers above the wait.
__device__ __forceinline__ void tmem_wait_ld_dep(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                   "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                   "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

// Empty instruction that "redefines" 32 registers: placed after a wait, it keeps every use of them below the wait.
__device__ __forceinline__ void reg_fence(uint32_t (&r)[32]) {
    asm volatile(""
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                   "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                   "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

template <int N>
__device__ __forceinline__ void reg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// D[tmem] (+)= A[tmem] * B[smem], B descriptor given as halves.
__device__ __forceinline__ void umma_ts_lohi(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi,
                                             uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}

template <bool FP16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    if (FP16) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    return pack_bf16x2(lo, hi);
}

// kind::f16 instruction descriptor: operand format 0 = fp16, 1 = bf16; fp32 accumulate.
__device__ __forceinline__ uint32_t make_idesc_16(int M, int N, int a_mn, int b_mn, bool fp16) {
    uint32_t d = 0;
    d |= 1u << 4;
    d |= (fp16 ? 0u : 1u) << 7;
    d |= (fp16 ? 0u : 1u) << 10;
    d |= (uint32_t)(a_mn & 1) << 15;
    d |= (uint32_t)(b_mn & 1) << 16;
    d |= (uint32_t)(N >> 3) << 17;
    d |= (uint32_t)(M >> 4) << 24;
    return d;
}

template <int D, bool FP16>
__global__ void __launch_bounds__(THREADS, 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const Fwd2Params p) {
    using C = Cfg2<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem + C::OFF_Q;
    uint8_t* sK = smem + C::OFF_K;
    uint8_t* sV = smem + C::OFF_V;
    float* s_alpha = reinterpret_cast<float*>(smem + C::OFF_MISC);   // [2][128]
    float* s_l = s_alpha + 2 * 128;                                    // [2][128]
    volatile int* s_flag = reinterpret_cast<volatile int*>(s_l + 2 * 128);   // [2][4]
    uint64_t* bars = reinterpret_cast<uint64_t*>(const_cast<int*>(s_flag) + 8);
    uint64_t* q_full = bars;            // 1
    uint64_t* k_full = bars + 1;        // 2
    uint64_t* k_empty = bars + 3;       // 2
    uint64_t* v_full = bars + 5;        // 2
    uint64_t* v_empty = bars + 7;       // 2
    uint64_t* s_full = bars + 9;        // 2 (per tile)
    uint64_t* p_full = bars + 11;       // 2
    uint64_t* alpha_ready = bars + 13;  // 2
    uint64_t* o_scaled = bars + 15;     // 2
    uint64_t* pv_done = bars + 17;      // 2
    uint64_t* l_ready = bars + 19;      // 2
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_pair = gridDim.x - 1 - blockIdx.x;      // heavy (late) query tiles first
    const int bh = blockIdx.y;
    const int bb = bh / p.hq, h = bh % p.hq;
    const int hk = h / (p.hq / p.hkv);
    const int off = p.sk - p.sq;

    // key-block range of each tile, then the union the producer walks
    int jb[2], je[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int q0 = q_pair * 2 * BM + i * BM;
        int kv_end = p.sk, kv_begin = 0;
        if (p.causal) kv_end = min(p.sk, q0 + BM + off);
        if (p.window >= 0) kv_begin = max(0, q0 + off - p.window);
        jb[i] = kv_begin / BN;
        je[i] = (kv_end + BN - 1) / BN;
        if (q0 >= p.sq || je[i] <= jb[i]) { jb[i] = 0; je[i] = 0; }
    }
    const int n0 = je[0] - jb[0], n1 = je[1] - jb[1];
    int ub, ue;
    if (n0 > 0 && n1 > 0) { ub = min(jb[0], jb[1]); ue = max(je[0], je[1]); }
    else if (n0 > 0) { ub = jb[0]; ue = je[0]; }
    else { ub = jb[1]; ue = je[1]; }
    const int G = ue - ub;                                 // union blocks g = 0 .. G-1 (key block ub + g)
    const int a0 = (n0 > 0) ? jb[0] - ub : 0, e0 = (n0 > 0) ? je[0] - ub : 0;
    const int a1 = (n1 > 0) ? jb[1] - ub : 0, e1 = (n1 > 0) ? je[1] - ub : 0;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 4);
            mbar_init(&alpha_ready[i], 4);
            mbar_init(&o_scaled[i], 4);
            mbar_init(&pv_done[i], 1);
            mbar_init(&l_ready[i], 4);
        }
        fence_barrier_init();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // 512 threads start with 128 registers each; the softmax warpgroups hold a whole 128-score row per thread
    if (warp < 4) {
        reg_dec<48>();
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0 && G > 0) {
            mbar_expect_tx(q_full, ((n0 > 0) + (n1 > 0)) * C::TILE);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if ((i == 0 ? n0 : n1) == 0) continue;
#pragma unroll
                for (int c = 0; c < C::NCH; ++c)
                    tma_load_4d(sQ + i * C::TILE + c * CHUNK_BYTES, &tmQ, q_full, c * 64, h, bb,
                                q_pair * 2 * BM + i * BM);
            }
            for (int g = 0; g < G; ++g) {
                const int st = g & 1;
                const uint32_t ph = ((g >> 1) & 1) ^ 1;
                const int kv0 = (ub + g) * BN;
                if (!mbar_wait(&k_empty[st], ph)) { atomicExch(p.status, 231); break; }
                mbar_expect_tx(&k_full[st], C::TILE);
#pragma unroll
                for (int c = 0; c < C::NCH; ++c)
                    tma_load_4d(sK + st * C::TILE + c * CHUNK_BYTES, &tmK, &k_full[st], c * 64, hk, bb, kv0);
                if (!mbar_wait(&v_empty[st], ph)) { atomicExch(p.status, 232); break; }
                mbar_expect_tx(&v_full[st], C::TILE);
#pragma unroll
                for (int c = 0; c < C::NCH; ++c)
                    tma_load_4d(sV + st * C::TILE + c * CHUNK_BYTES, &tmV, &v_full[st], c * 64, hk, bb, kv0);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && G > 0) {
            const uint32_t idesc_qk = make_idesc_16(BM, BN, 0, 0, FP16);
            const uint32_t idesc_pv = make_idesc_16(BM, D, 0, 1, FP16);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicExch(p.status, 233);
            auto active = [&](int i, int g) { return i == 0 ? (g >= a0 && g < e0) : (g >= a1 && g < e1); };
            // Operand descriptors are formed with one 32-bit add per MMA (constant upper half; the lower half counts
            // 16-byte units): a single thread issues every MMA, so the instruction count per MMA is what limits it.
            const uint32_t hi = smem_desc_hi_sw128(1024);
            const uint32_t q_lo[2] = {smem_desc_lo(smem_u32(sQ), 16), smem_desc_lo(smem_u32(sQ + C::TILE), 16)};
            const uint32_t k_lo[2] = {smem_desc_lo(smem_u32(sK), 16), smem_desc_lo(smem_u32(sK + C::TILE), 16)};
            const uint32_t v_lo[2] = {smem_desc_lo(smem_u32(sV), CHUNK_BYTES),
                                      smem_desc_lo(smem_u32(sV + C::TILE), CHUNK_BYTES)};
            auto qk = [&](int i, int g) -> bool {
                const int st = g & 1;
                if (!mbar_wait(&k_full[st], (g >> 1) & 1)) return false;
                tc_fence_after();
                const uint32_t ql = q_lo[i], kl = k_lo[st], td = tmem_base + i * 128;
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t o = ((k >> 2) * CHUNK_BYTES + (k & 3) * 32) >> 4;
                    umma_ss_lohi<false, false>(td, ql + o, hi, kl + o, hi, idesc_qk, k != 0 ? 1u : 0u);
                }
                umma_commit(&s_full[i]);
                return true;
            };
            auto pv = [&](int i, int g) -> bool {
                const int st = g & 1;
                const int t = g - (i == 0 ? a0 : a1);
                if (!mbar_wait(&p_full[i], t & 1) || !mbar_wait(&o_scaled[i], t & 1) ||
                    !mbar_wait(&v_full[st], (g >> 1) & 1))
                    return false;
                tc_fence_after();
                    const uint32_t vl = v_lo[st], td = tmem_base + 256 + i * 128, ta = tmem_base + i * 128;
                umma_ts_lohi(td, ta, vl, hi, idesc_pv, t != 0 ? 1u : 0u);
#pragma unroll
                for (int k = 1; k < BN / 16; ++k) umma_ts_lohi(td, ta + k * 8, vl + k * 128, hi, idesc_pv, 1u);
                umma_commit(&pv_done[i]);
                    return true;
            };
            if (ok) {
                for (int i = 0; i < 2 && ok; ++i)
                    if (active(i, 0) && !qk(i, 0)) { atomicExch(p.status, 234); ok = false; }
                if (ok) umma_commit(&k_empty[0]);
            }
            for (int g = 0; g < G && ok; ++g) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (!ok) break;
                    if (active(i, g) && !pv(i, g)) { atomicExch(p.status, 235); ok = false; break; }
                    if (i == 1) umma_commit(&v_empty[g & 1]);
                    if (g + 1 < G && active(i, g + 1) && !qk(i, g + 1)) { atomicExch(p.status, 236); ok = false; break; }
                    if (i == 1 && g + 1 < G) umma_commit(&k_empty[(g + 1) & 1]);
                }
            }
        }
    }
    } else if (warp < 12) {
        // ------------------------------------------------------------ softmax of tile i
        reg_inc<192>();
        const int i = (warp - 4) >> 2;
        const int qtr = warp & 3;
        const int row = qtr * 32 + lane;
        const uint32_t lane_base = uint32_t(qtr * 32) << 16;
        const uint32_t TM_S = tmem_base + lane_base + i * 128;
        const int q0 = q_pair * 2 * BM + i * BM;
        const int qpos = q0 + row + off;             // key index of this row's diagonal
        const int n = (i == 0) ? n0 : n1;
        const int jfirst = jb[i];
        const float scale = p.scale_log2;
        // scores stay unscaled in registers, so the ALiBi slope is divided by the softmax scale
        const float slope_raw = p.slopes ? p.slopes[h] * 1.4426950408889634f / p.scale_log2 : 0.f;
        const bool alibi = p.slopes != nullptr;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int t = 0; t < n; ++t) {
            if (!mbar_wait_warp(&s_full[i], t & 1)) {
                if (lane == 0) atomicExch(p.status, 237);
                ok = false;
                break;
            }
            tc_fence_after();
            const int kvb = (jfirst + t) * BN;
            // columns [lo, hi) of this block are visible to this row
            int lo = 0, hi = min(BN, p.sk - kvb);
            if (p.causal) hi = min(hi, qpos - kvb + 1);
            if (p.window >= 0) lo = max(lo, qpos - p.window - kvb);
            const bool need_mask = __any_sync(0xffffffffu, lo > 0 || hi < BN);
            const unsigned span = (hi > lo) ? (unsigned)(hi - lo) : 0u;
            const int dpos = qpos - kvb;
            // ---- the whole score row into registers (four loads in flight, one wait); S_i is free afterwards
            uint32_t r0[32], r1[32], r2[32], r3[32];
            tmem_ld_32x32(TM_S, r0);
            tmem_ld_32x32(TM_S + 32, r1);
            tmem_ld_32x32(TM_S + 64, r2);
            tmem_ld_32x32(TM_S + 96, r3);
            tmem_wait_ld_dep(r0);
            reg_fence(r1);
            reg_fence(r2);
            reg_fence(r3);
            // ---- row maximum of the scaled (and biased, masked) scores
            float mx;
            if (alibi || need_mask) {
                auto fix = [&](uint32_t(&r)[32], int c0) {
                    float m = -INFINITY;
#pragma unroll
                    for (int k = 0; k < 32; ++k) {
                        const int col = c0 + k;
                        float x = __uint_as_float(r[k]);
                        if (alibi) x -= slope_raw * fabsf((float)(dpos - col));
                        if (need_mask && (unsigned)(col - lo) >= span) x = -INFINITY;
                        r[k] = __float_as_uint(x);
                        m = fmaxf(m, x);
                    }
                    return m;
                };
                mx = fmaxf(fmaxf(fix(r0, 0), fix(r1, 32)), fmaxf(fix(r2, 64), fix(r3, 96)));
            } else {
                auto rowmax = [&](uint32_t(&r)[32]) {     // 3-input maxima, four independent chains
                    float m4[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) m4[k] = fmaxf(__uint_as_float(r[2 * k]), __uint_as_float(r[2 * k + 1]));
#pragma unroll
                    for (int k = 0; k < 12; ++k)
                        m4[k & 3] = max3(m4[k & 3], __uint_as_float(r[8 + 2 * k]), __uint_as_float(r[9 + 2 * k]));
                    return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                };
                mx = fmaxf(fmaxf(rowmax(r0), rowmax(r1)), fmaxf(rowmax(r2), rowmax(r3)));
            }
            mx *= scale;      // scores are kept unscaled in registers; scale > 0
            // ---- running maximum; rescale only when some row of this warp moved by more than the threshold
            const float m_new = fmaxf(m_used, mx);
            const bool grow = (t == 0) || (m_new > m_used + RESCALE_THRESHOLD);
            const bool any = __any_sync(0xffffffffu, grow);
            if (any) {
                const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
                const float alpha = (m_used == -INFINITY) ? 0.f : ex2(m_used - m_ref);
                l *= alpha;
                s_alpha[i * 128 + row] = alpha;
                m_used = m_new;
            }
            if (lane == 0) s_flag[i * 4 + qtr] = (any && t > 0) ? 1 : 0;
            __syncwarp();
            if (lane == 0) mbar_arrive(&alpha_ready[i]);
            const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
            // ---- P = exp2(x * scale - m), row sum, 16-bit pack, store over the first 64 columns of S_i
            float s4[4] = {0.f, 0.f, 0.f, 0.f};
            auto expo = [&](uint32_t(&r)[32], int cc) {
                uint32_t pk[16];
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const float e0 = ex2(fmaf(__uint_as_float(r[2 * k]), scale, -m_sub));
                    const float e1 = ex2(fmaf(__uint_as_float(r[2 * k + 1]), scale, -m_sub));
                    s4[k & 3] += e0 + e1;
                    pk[k] = pack16<FP16>(e0, e1);
                }
                tmem_st_32x16(TM_S + cc * 16, pk);
            };
            expo(r0, 0);
            expo(r1, 1);
            expo(r2, 2);
            expo(r3, 3);
            l += (s4[0] + s4[1]) + (s4[2] + s4[3]);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[i]);
        }
        if (n > 0) {
            s_l[i * 128 + row] = l;
            if (ok && q0 + row < p.sq && p.lse) {
                const float lse = (l > 0.f) ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
                p.lse[((size_t)bb * p.hq + h) * p.sq + q0 + row] = lse;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&l_ready[i]);
        }
    } else {
        // ------------------------------------------------------------ correction + epilogue (both tiles)
        reg_dec<80>();
        const int qtr = warp & 3;
        const int row = qtr * 32 + lane;
        const uint32_t lane_base = uint32_t(qtr * 32) << 16;
        bool ok = true;
        for (int g = 0; g < G && ok; ++g) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int a = (i == 0) ? a0 : a1, e = (i == 0) ? e0 : e1;
                if (g < a || g >= e) continue;
                const int t = g - a;
                if (!mbar_wait_warp(&alpha_ready[i], t & 1)) {
                    if (lane == 0) atomicExch(p.status, 238);
                    ok = false;
                    break;
                }
                if (s_flag[i * 4 + qtr]) {
                    if (!mbar_wait_warp(&pv_done[i], (t - 1) & 1)) {
                        if (lane == 0) atomicExch(p.status, 239);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const float al = s_alpha[i * 128 + row];
                    const uint32_t TM_O = tmem_base + lane_base + 256 + i * 128;
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t r[32];
                        tmem_ld_32x32(TM_O + c * 32, r);
                        tmem_wait_ld_dep(r);
#pragma unroll
                        for (int k = 0; k < 32; ++k) r[k] = __float_as_uint(__uint_as_float(r[k]) * al);
                        tmem_st_32x32(TM_O + c * 32, r);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&o_scaled[i]);
            }
        }
        // ---- epilogue: O_i / l_i -> 16-bit, rows of the [sq, b, hq, d] output
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int n = (i == 0) ? n0 : n1;
            if (n == 0 || !ok) continue;
            if (!mbar_wait_warp(&pv_done[i], (n - 1) & 1) || !mbar_wait_warp(&l_ready[i], 0)) {
                if (lane == 0) atomicExch(p.status, 240);
                ok = false;
                continue;
            }
            tc_fence_after();
            const int q0 = q_pair * 2 * BM + i * BM;
            const float lsum = s_l[i * 128 + row];
            const float inv = (lsum > 0.f) ? 1.0f / lsum : 0.f;
            const uint32_t TM_O = tmem_base + lane_base + 256 + i * 128;
            uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + (((size_t)(q0 + row) * p.b + bb) * p.hq + h) * D;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(TM_O + c * 32, r);
                tmem_wait_ld_dep(r);
                if (q0 + row < p.sq) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        uint4 q;
                        q.x = pack16<FP16>(__uint_as_float(r[u * 8 + 0]) * inv, __uint_as_float(r[u * 8 + 1]) * inv);
                        q.y = pack16<FP16>(__uint_as_float(r[u * 8 + 2]) * inv, __uint_as_float(r[u * 8 + 3]) * inv);
                        q.z = pack16<FP16>(__uint_as_float(r[u * 8 + 4]) * inv, __uint_as_float(r[u * 8 + 5]) * inv);
                        q.w = pack16<FP16>(__uint_as_float(r[u * 8 + 6]) * inv, __uint_as_float(r[u * 8 + 7]) * inv);
                        reinterpret_cast<uint4*>(o + c * 32)[u] = q;
                    }
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

template <int D, bool FP16>
int launch_fwd2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const Fwd2Params& p,
                cudaStream_t st) {
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(flash_fwd2_kernel<D, FP16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg2<D>::SMEM) != cudaSuccess)
            return NEOX_ERR_LAUNCH;
        attr = true;
    }
    dim3 grid((p.sq + 2 * BM - 1) / (2 * BM), p.b * p.hq);
    flash_fwd2_kernel<D, FP16><<<grid, THREADS, Cfg2<D>::SMEM, st>>>(tq, tk, tv, p);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

}  // namespace

// dtype: 0 = bf16, 2 = fp16 (the numbering of the other entry points of this library).
extern "C" int neox_flash_fwd2(const void* q, const void* k, const void* v, void* out, float* lse, int sq, int sk,
                               int b, int hq, int hkv, int d, long long q_ss, long long q_sb, long long q_sh,
                               long long k_ss, long long k_sb, long long k_sh, long long v_ss, long long v_sb,
                               long long v_sh, float scale, int causal, int window, const float* slopes, int dtype,
                               void* stream) {
    if (d != 64 && d != 96 && d != 128) return NEOX_ERR_SHAPE;
    if (dtype != 0 && dtype != 2) return NEOX_ERR_SHAPE;
    if (sq <= 0 || sk <= 0 || b <= 0) return 0;
    if (hq % hkv) return NEOX_ERR_SHAPE;
    CUtensorMap tq, tk, tv;
    int rc = neox_make_tmap_bf16_4d(&tq, q, d, hq, b, sq, q_sh, q_sb, q_ss, 64, BM);
    if (rc) return rc;
    rc = neox_make_tmap_bf16_4d(&tk, k, d, hkv, b, sk, k_sh, k_sb, k_ss, 64, BN);
    if (rc) return rc;
    rc = neox_make_tmap_bf16_4d(&tv, v, d, hkv, b, sk, v_sh, v_sb, v_ss, 64, BN);
    if (rc) return rc;
    Fwd2Params p;
    p.sq = sq; p.sk = sk; p.b = b; p.hq = hq; p.hkv = hkv;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.causal = causal; p.window = window; p.slopes = slopes;
    p.out = out;
    p.lse = lse;
    p.status = neox_status_word();
    if (!p.status) return NEOX_ERR_DRIVER;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool h16 = dtype == 2;
    if (d == 64) return h16 ? launch_fwd2<64, true>(tq, tk, tv, p, st) : launch_fwd2<64, false>(tq, tk, tv, p, st);
    if (d == 96) return h16 ? launch_fwd2<96, true>(tq, tk, tv, p, st) : launch_fwd2<96, false>(tq, tk, tv, p, st);
    return h16 ? launch_fwd2<128, true>(tq, tk, tv, p, st) : launch_fwd2<128, false>(tq, tk, tv, p, st);
}
