// bf16 and fp8 GEMMs on CTA pairs (tcgen05.mma.cta_group::2): one 256 x 256 output tile per pair of SMs.
//
// The two CTAs of a (2,1,1) cluster each stage 128 rows of A and HALF of the B tile (128 of its 256 columns); one
// thread of the even ("leader") CTA issues 256 x 256 x 16 MMAs that read A and B from both CTAs' shared memory and
// write 128 accumulator rows into each CTA's tensor memory.  Against the one-CTA kernel (gemm_sm100.cu) every SM
// moves 32 KB instead of 48 KB of operands per 128 x 256 x 64 of work, which is the resource that kernel is bound
// by (L2 -> SM traffic), and the freed shared memory deepens the ring from 4 to 6 stages.  Measured interleaved with
// the one-CTA kernel on the 20B layer shapes: 1.05x - 1.20x.
//
// Protocol (all barriers sit at the same shared-memory offsets in both CTAs):
//   empty[s]   per CTA, count 1: the leader's MMA thread commits to both CTAs at once (multicast commit);
//   full[s]    leader only: one arrive + the bytes of BOTH CTAs' TMA loads (each CTA's producer thread issues its own
//              loads into its own shared memory, completion counted on the leader's barrier);
//   tfull[b]   per CTA, count 1: accumulator buffer b is complete (multicast commit);
//   tempty[b]  leader only, count 8: the four epilogue warps of each CTA have drained buffer b (the odd CTA's warps
//              arrive through the cluster address of the leader's barrier).
// Tensor memory is allocated and freed by warp 1 of both CTAs with the cta_group::2 forms.  A cluster barrier after
// barrier initialisation and another before the free keep either CTA from touching the other's shared memory
// outside its lifetime.  Every wait is bounded; on a time-out the thread records a code, leaves its loops and still
// takes part in the final cluster barrier and the free.
//
// Same epilogue and operand layouts as gemm_sm100.cu / gemm_fp8_sm100.cu (which stay the kernels for small problems
// and for the per-row destination table); the fp8 form stages 128 one-byte elements of K per stage row.  Replaces
// the cuBLAS calls behind F.linear in megatron/mpu/layers.py:578,777 of the reference.
#include "gemm_common.cuh"
#include "neox_b200.h"
#include <stdio.h>
#include <stdlib.h>

using namespace sm100;
using namespace gemm;

namespace {

constexpr int STAGES2 = 6;
constexpr int BN_HALF = BN / 2;                       // B columns staged by one CTA
constexpr int A2_STAGE_BYTES = BM * BK * 2;           // 16 KB: 128 rows x 128 bytes of K
constexpr int B2_STAGE_BYTES = BN_HALF * BK * 2;      // 16 KB
constexpr int SMEM2_BYTES = STAGES2 * (A2_STAGE_BYTES + B2_STAGE_BYTES) + 256 + 1024;
constexpr int GROUP_M2 = 8;                           // 256-row tile rows per L2 group

struct PairScales {
    const float* inv_scale_a;                         // fp8 only: device scalars multiplied into alpha; NULL = 1
    const float* inv_scale_b;
    int a_fmt, b_fmt;                                 // fp8 only: 0 = E4M3, 1 = E5M2
    int group_m;                                      // 256-row tile rows per L2 group
};

__device__ __forceinline__ void tile_coords2(int tile, int num_m, int num_n, int group_m, int& m_blk, int& n_blk) {
    const int per_group = group_m * num_n;
    const int group = tile / per_group;
    const int first_m = group * group_m;
    const int gsize = min(num_m - first_m, group_m);
    const int in_group = tile - group * per_group;
    m_blk = first_m + in_group % gsize;
    n_blk = in_group / gsize;
}

// F8: operands are one-byte floats; a stage row still holds 128 bytes of K (128 elements instead of 64), an MMA
// consumes 32 of them, and an MN-major swizzle row covers 128 elements of the MN dimension instead of 64.
template <bool F8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                 const PairScales x) {
    constexpr int BKE = F8 ? 128 : 64;                // elements of K per stage
    constexpr int MNC = F8 ? 128 : 64;                // elements per MN-major chunk
    constexpr int CHUNK_BYTES = MNC * BKE * (F8 ? 1 : 2);
    constexpr int KSTEPS = 4;                         // MMAs per stage: 32 bytes of K each

    extern __shared__ uint8_t smem_raw[];
    // the dynamic shared memory window starts at the same offset in both CTAs, so this rounding is identical too
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES2 * A2_STAGE_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES2 * (A2_STAGE_BYTES + B2_STAGE_BYTES));
    uint64_t* empty = full + STAGES2;
    uint64_t* tfull = empty + STAGES2;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const int pair = blockIdx.x >> 1;
    const int npairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES2; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 8);
        }
        fence_barrier_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    // both CTAs' barriers exist before anyone signals across the pair
    cluster_sync_all();
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_m = (p.M + 2 * BM - 1) / (2 * BM);
    const int num_n = (p.N + BN - 1) / BN;
    const int ntiles = num_m * num_n;
    const int nk = (p.K + BKE - 1) / BKE;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (one per CTA)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; tile < ntiles && ok; tile += npairs) {
                int m_blk, n_blk;
                tile_coords2(tile, num_m, num_n, x.group_m, m_blk, n_blk);
                const int m0 = m_blk * 2 * BM + (int)rank * BM;
                const int n0 = n_blk * BN + (int)rank * BN_HALF;
                for (int kb = 0; kb < nk; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1)) {
                        atomicExch(p.status, 121);
                        ok = false;
                        break;
                    }
                    if (rank == 0) mbar_expect_tx(&full[stage], 2 * (A2_STAGE_BYTES + B2_STAGE_BYTES));
                    uint8_t* a_dst = sA + stage * A2_STAGE_BYTES;
                    uint8_t* b_dst = sB + stage * B2_STAGE_BYTES;
                    if (!p.a_mn) {
                        tma_load_2d_pair(a_dst, &tmA, &full[stage], kb * BKE, m0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / MNC; ++j)
                            tma_load_2d_pair(a_dst + j * CHUNK_BYTES, &tmA, &full[stage], m0 + j * MNC, kb * BKE);
                    }
                    if (!p.b_mn) {
                        tma_load_2d_pair(b_dst, &tmB, &full[stage], kb * BKE, n0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN_HALF / MNC; ++j)
                            tma_load_2d_pair(b_dst + j * CHUNK_BYTES, &tmB, &full[stage], n0 + j * MNC, kb * BKE);
                    }
                    if (++stage == STAGES2) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = F8 ? make_idesc_f8(2 * BM, BN, p.a_mn, p.b_mn, x.a_fmt, x.b_fmt)
                                      : make_idesc_16(2 * BM, BN, p.a_mn, p.b_mn, p.h16);
            // operand descriptors: constant upper half; lower half = stage base + k-step offset (16-byte units).
            // K-major: the next 32 bytes of K lie 32 bytes along the swizzled row; MN-major: they are the next
            // 16 (bf16) or 32 (fp8) rows of 128 bytes, with chunks of the MN dimension CHUNK_BYTES apart.
            const uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA), p.a_mn ? CHUNK_BYTES : 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(sB), p.b_mn ? CHUNK_BYTES : 16);
            const uint32_t mn_step = ((F8 ? 32 : 16) * 128) >> 4;
            const uint32_t a_step = p.a_mn ? mn_step : 2;
            const uint32_t b_step = p.b_mn ? mn_step : 2;
            int stage = 0;
            uint32_t phase = 0;
            int buf = 0;
            uint32_t bphase = 0;
            bool ok = true;
            for (int tile = pair; tile < ntiles && ok; tile += npairs) {
                if (!mbar_wait(&tempty[buf], bphase ^ 1)) {
                    atomicExch(p.status, 122);
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < nk; ++kb) {
                    if (!mbar_wait(&full[stage], phase)) {
                        atomicExch(p.status, 123);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + stage * (A2_STAGE_BYTES >> 4);
                    const uint32_t b_lo = b_lo0 + stage * (B2_STAGE_BYTES >> 4);
#pragma unroll
                    for (int k = 0; k < KSTEPS; ++k)
                        umma_ss_lohi<true, F8>(tmem_d, a_lo + k * a_step, desc_hi, b_lo + k * b_step, desc_hi, idesc,
                                               (kb | k) != 0);
                    umma_commit_pair(&empty[stage], 3);
                    if (++stage == STAGES2) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit_pair(&tfull[buf], 3);
                buf ^= 1;
                if (buf == 0) bphase ^= 1;
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps (2..5), both CTAs
        GemmParams pe = p;
        if (F8) {
            if (x.inv_scale_a) pe.alpha *= __ldg(x.inv_scale_a);
            if (x.inv_scale_b) pe.alpha *= __ldg(x.inv_scale_b);
        }
        const int q = warp & 3;
        const uint32_t tempty_leader0 = cluster_map(smem_u32(&tempty[0]), 0);
        int buf = 0;
        uint32_t bphase = 0;
        for (int tile = pair; tile < ntiles; tile += npairs) {
            int m_blk, n_blk;
            tile_coords2(tile, num_m, num_n, x.group_m, m_blk, n_blk);
            if (!mbar_wait_warp(&tfull[buf], bphase)) {
                if (lane == 0) atomicExch(p.status, 124);
                break;
            }
            tc_fence_after();
            const int row = m_blk * 2 * BM + (int)rank * BM + q * 32 + lane;
            const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int col0 = n_blk * BN + c * 32;
                if (col0 >= p.N) break;  // warp-uniform
                uint32_t r[32];
                tmem_ld_32x32(taddr + c * 32, r);
                tmem_wait_ld();
                if (row < p.M) epilogue_chunk(r, row, col0, F8 ? pe : p);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader0 + buf * 8);
            buf ^= 1;
            if (buf == 0) bphase ^= 1;
        }
    }

    // no CTA leaves (or frees tensor memory) while its partner may still signal it or run MMAs into it
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

template <bool F8>
int launch_pair(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb, long long ldd,
                int a_mn, int b_mn, PairScales x, int d_fp32, const void* bias, const void* add, long long ldadd,
                int add_fp32, void* preact, long long ldpre, const void* aux, long long ldaux, int act, float alpha,
                cudaStream_t stream, int h16 = 0) {
    constexpr int BKE = F8 ? 128 : 64, MNC = F8 ? 128 : 64, PITCH = F8 ? 16 : 8;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % PITCH) || (ldb % PITCH))
        return NEOX_ERR_ALIGN;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;
    auto tmap = F8 ? neox_make_tmap_u8_2d : neox_make_tmap_bf16_2d;

    CUtensorMap tmA, tmB;
    int rc;
    if (!a_mn) rc = tmap(&tmA, A, K, M, lda, BKE, BM);
    else rc = tmap(&tmA, A, M, K, lda, MNC, BKE);
    if (rc) return rc;
    if (!b_mn) rc = tmap(&tmB, B, K, N, ldb, BKE, BN_HALF);
    else rc = tmap(&tmB, B, N, K, ldb, MNC, BKE);
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
    p.h16 = h16 ? 1 : 0;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    bool vec = al16(D) && (ldd % 8 == 0);
    if (bias) vec = vec && al16(bias);
    if (add) vec = vec && al16(add) && (ldadd % 8 == 0);
    if (preact) vec = vec && al16(preact) && (ldpre % 8 == 0);
    if (aux) vec = vec && al16(aux) && (ldaux % 8 == 0);
    p.vec_ok = vec ? 1 : 0;

    static int group_m = 0;
    if (!group_m) {
        const char* e = getenv("NEOX_PAIR_GROUP_M");
        group_m = e ? atoi(e) : GROUP_M2;
        if (group_m < 1) group_m = GROUP_M2;
    }
    x.group_m = group_m;
    static bool attr_set = false;     // one per instantiation
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_2cta_kernel<F8>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES) !=
            cudaSuccess)
            return NEOX_ERR_LAUNCH;
        attr_set = true;
    }
    const int num_m = (M + 2 * BM - 1) / (2 * BM), num_n = (N + BN - 1) / BN;
    int pairs = num_m * num_n;
    const int max_pairs = neox_sm_count() / 2;
    if (pairs > max_pairs) pairs = max_pairs;
    gemm_2cta_kernel<F8><<<2 * pairs, NUM_THREADS, SMEM2_BYTES, stream>>>(tmA, tmB, p, x);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

}  // namespace

// Same contract as neox_gemm_bf16 (no row table).
extern "C" int neox_gemm_bf16_2cta(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                                   long long ldb, long long ldd, int a_mn, int b_mn, int d_fp32, const void* bias,
                                   const void* add, long long ldadd, int add_fp32, void* preact, long long ldpre,
                                   const void* aux, long long ldaux, int act, float alpha, void* stream_) {
    return launch_pair<false>(A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, PairScales{nullptr, nullptr, 0, 0, 0}, d_fp32,
                              bias, add, ldadd, add_fp32, preact, ldpre, aux, ldaux, act, alpha,
                              static_cast<cudaStream_t>(stream_));
}

// Same with the 16-bit type chosen by h16 (0 = bf16, 1 = fp16).
extern "C" int neox_gemm_16_2cta(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                                 long long ldb, long long ldd, int a_mn, int b_mn, int d_fp32, const void* bias,
                                 const void* add, long long ldadd, int add_fp32, void* preact, long long ldpre,
                                 const void* aux, long long ldaux, int act, float alpha, int h16, void* stream_) {
    return launch_pair<false>(A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, PairScales{nullptr, nullptr, 0, 0, 0}, d_fp32,
                              bias, add, ldadd, add_fp32, preact, ldpre, aux, ldaux, act, alpha,
                              static_cast<cudaStream_t>(stream_), h16);
}

// Same contract as neox_gemm_fp8.
extern "C" int neox_gemm_fp8_2cta(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                                  long long ldb, long long ldd, int a_mn, int b_mn, int a_fmt, int b_fmt,
                                  const float* inv_scale_a, const float* inv_scale_b, int d_fp32, const void* bias,
                                  const void* add, long long ldadd, int add_fp32, void* preact, long long ldpre,
                                  const void* aux, long long ldaux, int act, float alpha, void* stream_) {
    if ((a_fmt | b_fmt) & ~1) return NEOX_ERR_SHAPE;
    return launch_pair<true>(A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn,
                             PairScales{inv_scale_a, inv_scale_b, a_fmt, b_fmt, 0}, d_fp32, bias, add, ldadd, add_fp32,
                             preact, ldpre, aux, ldaux, act, alpha, static_cast<cudaStream_t>(stream_));
}
