// Flash attention forward for sm_100a: S = QK^T and O = PV on tcgen05 with accumulators in tensor memory.
//
// One CTA per (128-row query tile, batch, head).  Warp roles:
//   warp 0      TMA producer: Q once, then K/V tiles of 128 keys through a 2-stage ring (4-D tensor maps over
//               the strided [s, b, h, d] views, so the fused QKV projection output is read in place);
//   warp 1      MMA issuer: S_j = Q K_j^T into a double-buffered 128-column TMEM accumulator, and
//               O_j = P_j V_j into a second double buffer; QK^T of block j+1 is issued before P_j is awaited;
//   warps 4-11  softmax group, two warps per TMEM lane quarter: a thread owns one query row (tcgen05.ld 32x32b hands
//               each thread one accumulator row) and one 64-column half of the 128-key block; the two halves agree
//               on the running row maximum through a shared-memory mailbox (bounded wait), keep partial row sums,
//               apply scale, ALiBi, causal / sliding-window / tail masks, exp2, and write their half of P_j as bf16
//               into 128-byte-swizzled shared memory;
//   warps 12-19 accumulate group, two warps per lane quarter, each owning half of the head dimension:
//               O_acc = O_acc * alpha_j + O_j in registers (alpha_j handed over through shared memory), final 1/l
//               normalisation and bf16 store.
// Head sizes 64 / 96 / 128 (96 occupies one and a half 64-wide swizzle chunks; TMA zero-fills the rest and the
// MMAs only iterate over the real 96 columns).  Grouped-query attention: kv head = q head / (hq / hkv).
//
// Replaces the flash-attn 2 calls of megatron/model/transformer.py:627-744.  All waits are bounded.
#include "sm100_ptx.cuh"
#include "neox_b200.h"
#include <math.h>

using namespace sm100;

namespace {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int CHUNK_BYTES = 128 * 128;  // one [128 rows x 64 bf16] swizzled chunk
constexpr int SPARTS = 2;                // softmax warps per TMEM lane quarter (64 score columns per thread)
constexpr int APARTS = 2;                // accumulate warps per lane quarter (half of the head dimension each)
constexpr int FWD_THREADS = 128 + 128 * SPARTS + 128 * APARTS;

struct FwdParams {
    int sq, sk, b, hq, hkv, d;
    float scale_log2;  // softmax scale * log2(e)
    int causal, window;
    const float* slopes;  // ALiBi slopes per q head (nullable)
    __nv_bfloat16* out;   // [sq, b, hq, d] contiguous
    float* lse;           // [b, hq, sq]
    int* status;
};

template <int D>
struct Cfg {
    static constexpr int NCH = (D == 64) ? 1 : 2;  // 64-wide chunks per operand tile
    static constexpr int TILE = NCH * CHUNK_BYTES;
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = TILE;
    static constexpr int OFF_V = OFF_K + 2 * TILE;
    static constexpr int OFF_P = OFF_V + 2 * TILE;
    static constexpr int OFF_MISC = OFF_P + 2 * CHUNK_BYTES;
    static constexpr int MISC_BYTES = 8192;   // alpha ring, partial row sums, row-max mailboxes, barriers
    static constexpr int SMEM = OFF_MISC + MISC_BYTES + 1024;
};

template <int D>
__global__ void __launch_bounds__(FWD_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
    using C = Cfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem + C::OFF_Q;
    uint8_t* sK = smem + C::OFF_K;
    uint8_t* sV = smem + C::OFF_V;
    uint8_t* sP = smem + C::OFF_P;
    float* s_alpha = reinterpret_cast<float*>(smem + C::OFF_MISC);  // [4][128]
    float* s_l = s_alpha + 4 * 128;                                   // [SPARTS][128] partial row sums
    float* s_max = s_l + SPARTS * 128;                                // [2][SPARTS][128] row-max mailboxes
    volatile int* s_seq = reinterpret_cast<volatile int*>(s_max + 2 * SPARTS * 128);   // [4 quarters][SPARTS]
    uint64_t* bars = reinterpret_cast<uint64_t*>(const_cast<int*>(s_seq) + 4 * SPARTS + 8);
    uint64_t* q_full = bars;          // 1
    uint64_t* k_full = bars + 1;      // 2   K and V have separate rings: a K stage is free as soon as QK^T of its
    uint64_t* k_empty = bars + 3;     // 2   block has run, two iterations before the V stage of the same block, so
    uint64_t* v_full = bars + 5;      // 2   the next K tile is already in flight while the softmax of the current
    uint64_t* v_empty = bars + 7;     // 2   block runs and no TMA latency sits on the critical path
    uint64_t* s_full = bars + 9;      // 2
    uint64_t* s_empty = bars + 11;    // 2
    uint64_t* p_full = bars + 13;     // 1
    uint64_t* p_empty = bars + 14;    // 1
    uint64_t* o_full = bars + 15;     // 2
    uint64_t* o_empty = bars + 17;    // 2
    uint64_t* l_full = bars + 19;     // 1
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heavy (late) query tiles first so that causal work is balanced across the wave
    const int q_tile = gridDim.x - 1 - blockIdx.x;
    const int bh = blockIdx.y;
    const int bb = bh / p.hq, h = bh % p.hq;
    const int hk = h / (p.hq / p.hkv);
    const int q0 = q_tile * BM;
    const int off = p.sk - p.sq;  // bottom-right aligned causal mask

    int kv_end = p.sk;
    if (p.causal) kv_end = min(p.sk, q0 + BM + off);
    int kv_begin = 0;
    if (p.window >= 0) kv_begin = max(0, q0 + off - p.window);
    const int jb = kv_begin / BN;
    const int je = (kv_end + BN - 1) / BN;  // blocks [jb, je)
    const int nblk = max(je - jb, 0);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 4 * SPARTS);
            mbar_init(&o_full[i], 1);
            mbar_init(&o_empty[i], 4 * APARTS);
        }
        mbar_init(p_full, 4 * SPARTS);
        mbar_init(p_empty, 1);
        mbar_init(l_full, 4 * SPARTS);
        for (int i = 0; i < 4 * SPARTS; ++i) s_seq[i] = 0;
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
    const uint32_t TM_S = tmem_base;         // 2 x 128 columns
    const uint32_t TM_O = tmem_base + 256;   // 2 x 128 columns

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0 && nblk > 0) {
            mbar_expect_tx(q_full, C::TILE);
#pragma unroll
            for (int c = 0; c < C::NCH; ++c) tma_load_4d(sQ + c * CHUNK_BYTES, &tmQ, q_full, c * 64, h, bb, q0);
            for (int i = 0; i < nblk; ++i) {
                const int st = i & 1;
                const int kv0 = (jb + i) * BN;
                if (!mbar_wait(&k_empty[st], ((i >> 1) & 1) ^ 1)) {
                    atomicExch(p.status, 201);
                    break;
                }
                mbar_expect_tx(&k_full[st], C::TILE);
#pragma unroll
                for (int c = 0; c < C::NCH; ++c)
                    tma_load_4d(sK + st * C::TILE + c * CHUNK_BYTES, &tmK, &k_full[st], c * 64, hk, bb, kv0);
                if (!mbar_wait(&v_empty[st], ((i >> 1) & 1) ^ 1)) {
                    atomicExch(p.status, 211);
                    break;
                }
                mbar_expect_tx(&v_full[st], C::TILE);
#pragma unroll
                for (int c = 0; c < C::NCH; ++c)
                    tma_load_4d(sV + st * C::TILE + c * CHUNK_BYTES, &tmV, &v_full[st], c * 64, hk, bb, kv0);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && nblk > 0) {
            const uint32_t idesc_qk = make_idesc_bf16(BM, BN, 0, 0);
            const uint32_t idesc_pv = make_idesc_bf16(BM, D, 0, 1);
            const uint32_t q_base = smem_u32(sQ), p_base = smem_u32(sP);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicExch(p.status, 202);
            auto issue_qk = [&](int i) -> bool {
                const int st = i & 1;
                if (!mbar_wait(&k_full[st], (i >> 1) & 1)) return false;
                if (!mbar_wait(&s_empty[st], ((i >> 1) & 1) ^ 1)) return false;
                tc_fence_after();
                const uint32_t k_base = smem_u32(sK + st * C::TILE);
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t o = (k >> 2) * CHUNK_BYTES + (k & 3) * 32;
                    umma_bf16_ss(TM_S + st * 128, make_smem_desc_sw128(q_base + o, 16, 1024),
                                 make_smem_desc_sw128(k_base + o, 16, 1024), idesc_qk, k != 0);
                }
                umma_commit(&s_full[st]);
                umma_commit(&k_empty[st]);
                return true;
            };
            if (ok && !issue_qk(0)) {
                atomicExch(p.status, 203);
                ok = false;
            }
            for (int i = 0; i < nblk && ok; ++i) {
                const int st = i & 1;
                if (i + 1 < nblk && !issue_qk(i + 1)) {
                    atomicExch(p.status, 204);
                    break;
                }
                if (!mbar_wait(p_full, i & 1) || !mbar_wait(&o_empty[st], ((i >> 1) & 1) ^ 1) ||
                    !mbar_wait(&v_full[st], (i >> 1) & 1)) {
                    atomicExch(p.status, 205);
                    break;
                }
                tc_fence_after();
                const uint32_t v_base = smem_u32(sV + st * C::TILE);
#pragma unroll
                for (int k = 0; k < BN / 16; ++k) {
                    const uint32_t po = (k >> 2) * CHUNK_BYTES + (k & 3) * 32;
                    umma_bf16_ss(TM_O + st * 128, make_smem_desc_sw128(p_base + po, 16, 1024),
                                 make_smem_desc_sw128(v_base + k * 2048, CHUNK_BYTES, 1024), idesc_pv, k != 0);
                }
                umma_commit(&o_full[st]);
                umma_commit(&v_empty[st]);
                umma_commit(p_empty);
            }
        }
    } else if (warp < 4) {
        // warps 2 and 3 have no role
    } else if (warp < 4 + 4 * SPARTS) {
        // ------------------------------------------------------------ softmax group
        const int qtr = warp & 3;                 // TMEM lane quarter
        const int part = (warp - 4) >> 2;         // which 64-column half of the key block
        const int row = qtr * 32 + lane;
        const uint32_t lane_base = uint32_t(qtr * 32) << 16;
        const int qpos = q0 + row + off;  // key index of the diagonal for this row
        const float slope = p.slopes ? p.slopes[h] * 1.4426950408889634f : 0.f;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        // Bounded wait until the other half has published its value for sequence number `want`.
        auto wait_other = [&](int want) -> bool {
            int good = 1;
            if (lane == 0) {
                const long long t0 = clock64();
                while (s_seq[qtr * SPARTS + (part ^ 1)] < want) {
                    if (clock64() - t0 > SPIN_LIMIT_CYCLES) {
                        good = 0;
                        break;
                    }
                }
                __threadfence_block();
            }
            good = __shfl_sync(0xffffffffu, good, 0);
            return good != 0;
        };
        for (int i = 0; i < nblk; ++i) {
            const int st = i & 1;
            if (!mbar_wait_warp(&s_full[st], (i >> 1) & 1)) {
                if (lane == 0) atomicExch(p.status, 206);
                ok = false;
                break;
            }
            tc_fence_after();
            float t[64];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(TM_S + lane_base + st * 128 + part * 64 + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int k = 0; k < 32; ++k) t[c * 32 + k] = __uint_as_float(r[k]) * p.scale_log2;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[st]);
            const int kvb = (jb + i) * BN;            // first key of the block
            const int kv0 = kvb + part * 64;          // first key of this thread's half
            if (p.slopes) {
#pragma unroll
                for (int k = 0; k < 64; ++k) t[k] -= slope * fabsf((float)(qpos - (kv0 + k)));
            }
            const bool need_mask = (kvb + BN > p.sk) || (p.causal && kvb + BN - 1 > q0 + off) ||
                                   (p.window >= 0 && kvb < q0 + BM - 1 + off - p.window);
            if (need_mask) {
#pragma unroll
                for (int k = 0; k < 64; ++k) {
                    const int kv = kv0 + k;
                    const bool dead = (kv >= p.sk) || (p.causal && kv > qpos) || (p.window >= 0 && kv < qpos - p.window);
                    if (dead) t[k] = -INFINITY;
                }
            }
            float pm = -INFINITY;
#pragma unroll
            for (int k = 0; k < 64; ++k) pm = fmaxf(pm, t[k]);
            // exchange the block maximum with the warp that owns the other half of this row
            float* box = s_max + (i & 1) * SPARTS * 128;
            box[part * 128 + row] = pm;
            __syncwarp();
            if (lane == 0) {
                __threadfence_block();
                s_seq[qtr * SPARTS + part] = i + 1;
            }
            if (!wait_other(i + 1)) {
                if (lane == 0) atomicExch(p.status, 210);
                ok = false;
                break;
            }
            const float mx = fmaxf(m, fmaxf(pm, box[(part ^ 1) * 128 + row]));
            const float m_use = (mx == -INFINITY) ? 0.f : mx;
            const float alpha = exp2f(m - m_use);
            float sum = 0.f;
#pragma unroll
            for (int k = 0; k < 64; ++k) {
                t[k] = exp2f(t[k] - m_use);
                sum += t[k];
            }
            l = l * alpha + sum;
            m = mx;
            if (!mbar_wait_warp(p_empty, (i & 1) ^ 1)) {
                if (lane == 0) atomicExch(p.status, 207);
                ok = false;
                break;
            }
            // P (bf16) into the K-major 128-byte-swizzled layout the MMA reads: 16-byte unit u of row r lives at
            // r*128 + ((u ^ (r & 7)) << 4) inside its 64-column chunk; this thread's half IS chunk `part`.
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                uint4 q;
                q.x = pack_bf16x2(t[u * 8 + 0], t[u * 8 + 1]);
                q.y = pack_bf16x2(t[u * 8 + 2], t[u * 8 + 3]);
                q.z = pack_bf16x2(t[u * 8 + 4], t[u * 8 + 5]);
                q.w = pack_bf16x2(t[u * 8 + 6], t[u * 8 + 7]);
                *reinterpret_cast<uint4*>(sP + part * CHUNK_BYTES + row * 128 + ((u ^ (row & 7)) << 4)) = q;
            }
            if (part == 0) s_alpha[(i & 3) * 128 + row] = alpha;
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        s_l[part * 128 + row] = l;
        __syncwarp();
        if (lane == 0) {
            __threadfence_block();
            s_seq[qtr * SPARTS + part] = nblk + 1;
        }
        if (part == 0 && ok && wait_other(nblk + 1)) {
            const float lt = s_l[row] + s_l[128 + row];
            if (q0 + row < p.sq && p.lse) {
                const float lse = (lt > 0.f) ? (m + log2f(lt)) * 0.6931471805599453f : -INFINITY;
                p.lse[((size_t)bb * p.hq + h) * p.sq + q0 + row] = lse;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(l_full);
    } else {
        // ------------------------------------------------------------ accumulate group
        constexpr int DH = D / APARTS;            // head-dimension columns per thread: 32, 48 or 64
        const int qtr = warp & 3;
        const int part = (warp - 4 - 4 * SPARTS) >> 2;
        const int row = qtr * 32 + lane;
        const uint32_t lane_base = uint32_t(qtr * 32) << 16;
        float acc[DH];
#pragma unroll
        for (int k = 0; k < DH; ++k) acc[k] = 0.f;
        bool ok = true;
        for (int i = 0; i < nblk; ++i) {
            const int st = i & 1;
            if (!mbar_wait_warp(&o_full[st], (i >> 1) & 1)) {
                if (lane == 0) atomicExch(p.status, 208);
                ok = false;
                break;
            }
            tc_fence_after();
            const float a = s_alpha[(i & 3) * 128 + row];
            const uint32_t tcol = TM_O + lane_base + st * 128 + part * DH;
            {
                uint32_t r[32];
                tmem_ld_32x32(tcol, r);
                tmem_wait_ld();
#pragma unroll
                for (int k = 0; k < 32; ++k) acc[k] = acc[k] * a + __uint_as_float(r[k]);
            }
            if (DH == 48) {
                uint32_t r[16];
                tmem_ld_32x16(tcol + 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int k = 0; k < 16; ++k) acc[(32 + k) % DH] = acc[(32 + k) % DH] * a + __uint_as_float(r[k]);
            } else if (DH == 64) {
                uint32_t r[32];
                tmem_ld_32x32(tcol + 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int k = 0; k < 32; ++k) acc[(32 + k) % DH] = acc[(32 + k) % DH] * a + __uint_as_float(r[k]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_empty[st]);
        }
        if (ok && !mbar_wait_warp(l_full, 0)) {
            if (lane == 0) atomicExch(p.status, 209);
            ok = false;
        }
        if (ok && q0 + row < p.sq) {
            const float l = s_l[row] + s_l[128 + row];
            const float inv = (l > 0.f) ? 1.0f / l : 0.f;
            __nv_bfloat16* o = p.out + (((size_t)(q0 + row) * p.b + bb) * p.hq + h) * D + part * DH;
#pragma unroll
            for (int u = 0; u < DH / 8; ++u) {
                uint4 q;
                q.x = pack_bf16x2(acc[u * 8 + 0] * inv, acc[u * 8 + 1] * inv);
                q.y = pack_bf16x2(acc[u * 8 + 2] * inv, acc[u * 8 + 3] * inv);
                q.z = pack_bf16x2(acc[u * 8 + 4] * inv, acc[u * 8 + 5] * inv);
                q.w = pack_bf16x2(acc[u * 8 + 6] * inv, acc[u * 8 + 7] * inv);
                reinterpret_cast<uint4*>(o)[u] = q;
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
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p,
               cudaStream_t st) {
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(flash_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::SMEM) !=
            cudaSuccess)
            return NEOX_ERR_LAUNCH;
        attr = true;
    }
    dim3 grid((p.sq + BM - 1) / BM, p.b * p.hq);
    flash_fwd_kernel<D><<<grid, FWD_THREADS, Cfg<D>::SMEM, st>>>(tq, tk, tv, p);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

}  // namespace

extern "C" int neox_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int sq, int sk, int b,
                              int hq, int hkv, int d, long long q_ss, long long q_sb, long long q_sh, long long k_ss,
                              long long k_sb, long long k_sh, long long v_ss, long long v_sb, long long v_sh,
                              float scale, int causal, int window, const float* slopes, void* stream) {
    if (d != 64 && d != 96 && d != 128) return NEOX_ERR_SHAPE;
    if (sq <= 0 || sk <= 0 || b <= 0) return 0;
    if (hq % hkv) return NEOX_ERR_SHAPE;
    CUtensorMap tq, tk, tv;
    int rc = neox_make_tmap_bf16_4d(&tq, q, d, hq, b, sq, q_sh, q_sb, q_ss, 64, BM);
    if (rc) return rc;
    rc = neox_make_tmap_bf16_4d(&tk, k, d, hkv, b, sk, k_sh, k_sb, k_ss, 64, BN);
    if (rc) return rc;
    rc = neox_make_tmap_bf16_4d(&tv, v, d, hkv, b, sk, v_sh, v_sb, v_ss, 64, BN);
    if (rc) return rc;
    FwdParams p;
    p.sq = sq; p.sk = sk; p.b = b; p.hq = hq; p.hkv = hkv; p.d = d;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.causal = causal; p.window = window; p.slopes = slopes;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.lse = lse;
    p.status = neox_status_word();
    if (!p.status) return NEOX_ERR_DRIVER;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (d == 64) return launch_fwd<64>(tq, tk, tv, p, st);
    if (d == 96) return launch_fwd<96>(tq, tk, tv, p, st);
    return launch_fwd<128>(tq, tk, tv, p, st);
}
