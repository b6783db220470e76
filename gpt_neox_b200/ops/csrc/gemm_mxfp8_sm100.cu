// MXFP8 GEMM on the block-scaled fp8 tensor cores of sm_100a (tcgen05.mma.kind::mxf8f6f4.block_scale):
//
//     D = epilogue( alpha * sum_k  (A_q[m, k] * 2^(sa[m, k / 32] - 127)) * (B_q[n, k] * 2^(sb[n, k / 32] - 127)) )
//
// A_q / B_q are FP8 bytes (E4M3 or E5M2 per operand); sa / sb are E8M0 bytes, one per 32 elements along K (the OCP
// MX format).  The hardware applies the scales inside the MMA: per 128 bytes of K (one pipeline stage = four
// K = 32 instructions) the issuing thread copies the stage's scale chunks from shared memory into tensor memory
// with tcgen05.cp (32 lanes x 128 bits, replicated to the four lane quarters) and passes their tensor-memory address
// plus a byte selector (which of the four K-blocks of the stage) to each MMA.
//
// Pipeline as in gemm_fp8_sm100.cu, with three differences:
//   * the scale chunks of a stage (512 bytes for the 128 rows of A, 1024 bytes for two 128-column chunks of B)
//     travel in the same stage, by plain bulk copies from the tiled layout that mxfp8.cu writes;
//   * the output tile is 128 x 192, so that two accumulators (384 columns) and the scale columns (2 x 12) fit in the
//     512 columns of tensor memory and the epilogue of one tile still overlaps the main loop of the next;
//   * a 192-wide tile starts in the middle of a 128-column scale chunk every other tile: the B scales are then read
//     two tensor-memory columns (64 values of n) further in.
// Both operands may be K-major or MN-major (scales are indexed by (row-or-column, K block) either way), so forward,
// data-gradient and weight-gradient GEMMs of a linear layer all run here without transposed copies.
//
// The reference has no block-scaled path (its fp8 is Transformer Engine's per-tensor delayed scaling,
// megatron/model/transformer_engine.py).  All barrier waits are bounded.
#include "gemm_common.cuh"
#include "neox_b200.h"

using namespace sm100;
using namespace gemm;

namespace {

constexpr int BNX = 192;                     // output columns per tile
constexpr int BKX = 128;                     // bytes (= elements) of K per stage
constexpr int STAGESX = 4;
constexpr int AX_STAGE = BM * BKX;           // 16 KB
constexpr int BX_STAGE = 2 * 128 * BKX;      // 32 KB: K-major uses 192 rows of it, MN-major two 128-wide chunks
constexpr int SFA_BYTES = 512, SFB_BYTES = 1024;
constexpr int SF_STAGE = SFA_BYTES + SFB_BYTES;
constexpr int SMEMX_BYTES = STAGESX * (AX_STAGE + BX_STAGE + SF_STAGE) + 256 + 1024;
constexpr int TM_SF = 2 * BNX;               // first scale column in tensor memory; two regions of 16 columns

struct MxParams {
    const unsigned char* sfa;                // tiled scale layouts (see mxfp8.cu)
    const unsigned char* sfb;
    long long sfa_mnb, sfb_mnb;              // chunks per row of chunks
    int a_fmt, b_fmt;
};

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// 32 rows x 16 bytes from shared memory (row pitch 16 bytes: un-swizzled K-major descriptor, 8-row groups 128 bytes
// apart) to 4 tensor-memory columns, lanes 0-31, replicated into lanes 32-63, 64-95 and 96-127.
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)(128 >> 4) << 32;         // stride between 8-row groups
    d |= (uint64_t)1 << 46;
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(d) : "memory");
}
// Instruction descriptor of the block-scaled kind: E8M0 scales, fp32 accumulate, M = 128.
__device__ __forceinline__ uint32_t make_idesc_mx(int N, int a_mn, int b_mn, int a_fmt, int b_fmt) {
    uint32_t d = 0;
    d |= (uint32_t)(a_fmt & 7) << 7;
    d |= (uint32_t)(b_fmt & 7) << 10;
    d |= (uint32_t)(a_mn & 1) << 15;
    d |= (uint32_t)(b_mn & 1) << 16;
    d |= (uint32_t)(N >> 3) << 17;
    d |= 1u << 23;                           // scale format E8M0
    d |= (uint32_t)(BM >> 4) << 24;
    return d;
}
__device__ __forceinline__ void umma_mx_ss(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                           uint32_t idesc, uint32_t sfa_taddr, uint32_t sfb_taddr, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %8, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], da, db, %5, [%6], [%7], p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(sfa_taddr), "r"(sfb_taddr),
        "r"(accumulate)
        : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                  const MxParams x) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGESX * AX_STAGE;
    uint8_t* sSF = sB + STAGESX * BX_STAGE;
    uint64_t* full = reinterpret_cast<uint64_t*>(sSF + STAGESX * SF_STAGE);
    uint64_t* empty = full + STAGESX;
    uint64_t* tfull = empty + STAGESX;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGESX; ++s) {
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
    const int num_n = (p.N + BNX - 1) / BNX;
    const int ntiles = num_m * num_n;
    const int nk = (p.K + BKX - 1) / BKX;
    const uint32_t b_bytes = p.b_mn ? 2 * 128 * BKX : BNX * BKX;

    if (warp == 0) {
        // ------------------------------------------------------------ producer: operands by TMA, scales by bulk copy
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // loop state in registers: this one thread must finish a k-block's bookkeeping well inside the ~500
            // clocks the tensor core spends on it
            const bool a_mn = p.a_mn != 0, b_mn = p.b_mn != 0;
            const uint32_t tx_bytes = AX_STAGE + b_bytes + SF_STAGE;
            const long long sfa_step = x.sfa_mnb * 512, sfb_step = x.sfb_mnb * 512;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                int m_blk, n_blk;
                tile_coords(tile, num_m, num_n, m_blk, n_blk);
                const int n0 = n_blk * BNX;
                const int m0 = m_blk * BM;
                const unsigned char* sfa = x.sfa + (long long)m_blk * 512;
                const unsigned char* sfb = x.sfb + (long long)(n0 >> 7) * 512;
                int k0 = 0;
                for (int kb = 0; kb < nk; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1)) {
                        atomicExch(p.status, 131);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[stage], tx_bytes);
                    uint8_t* a_dst = sA + stage * AX_STAGE;
                    uint8_t* b_dst = sB + stage * BX_STAGE;
                    uint8_t* sf_dst = sSF + stage * SF_STAGE;
                    if (!a_mn) tma_load_2d(a_dst, &tmA, &full[stage], k0, m0);
                    else tma_load_2d(a_dst, &tmA, &full[stage], m0, k0);
                    if (!b_mn) {
                        tma_load_2d(b_dst, &tmB, &full[stage], k0, n0);
                    } else {
                        tma_load_2d(b_dst, &tmB, &full[stage], n0, k0);
                        tma_load_2d(b_dst + 128 * BKX, &tmB, &full[stage], n0 + 128, k0);
                    }
                    bulk_load(sf_dst, sfa, SFA_BYTES, &full[stage]);
                    bulk_load(sf_dst + SFA_BYTES, sfb, SFB_BYTES, &full[stage]);
                    sfa += sfa_step;
                    sfb += sfb_step;
                    k0 += BKX;
                    if (++stage == STAGESX) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc0 = make_idesc_mx(BNX, p.a_mn, p.b_mn, x.a_fmt, x.b_fmt);
            const uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA), p.a_mn ? 128 * BKX : 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(sB), p.b_mn ? 128 * BKX : 16);
            const uint32_t a_step = (p.a_mn ? 32 * 128 : 32) >> 4;
            const uint32_t b_step = (p.b_mn ? 32 * 128 : 32) >> 4;
            const uint32_t sf_smem0 = smem_u32(sSF);
            uint32_t idesc_k[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) idesc_k[k] = idesc0 | ((uint32_t)k << 29) | ((uint32_t)k << 4);
            int stage = 0;
            uint32_t phase = 0;
            int buf = 0;
            uint32_t bphase = 0;
            uint32_t sfr = 0;                 // which of the two scale regions of tensor memory
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                int m_blk, n_blk;
                tile_coords(tile, num_m, num_n, m_blk, n_blk);
                // a 192-wide tile starts 0 or 64 columns into a 128-column scale chunk: 0 or 2 columns of 32 values
                const uint32_t sfb_col = (uint32_t)(((n_blk * BNX) & 127) >> 5);
                if (!mbar_wait(&tempty[buf], bphase ^ 1)) {
                    atomicExch(p.status, 132);
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BNX;
                for (int kb = 0; kb < nk; ++kb) {
                    if (!mbar_wait(&full[stage], phase)) {
                        atomicExch(p.status, 133);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sf_t = tmem_base + TM_SF + sfr * 16;
                    const uint32_t sf_s = sf_smem0 + stage * SF_STAGE;
                    tmem_cp_sf(sf_t, sf_s);                       // A scales: 4 columns
                    tmem_cp_sf(sf_t + 4, sf_s + SFA_BYTES);       // B scales: 2 chunks x 4 columns
                    tmem_cp_sf(sf_t + 8, sf_s + SFA_BYTES + 512);
                    const uint32_t a_lo = a_lo0 + stage * (AX_STAGE >> 4);
                    const uint32_t b_lo = b_lo0 + stage * (BX_STAGE >> 4);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_mx_ss(tmem_d, a_lo + k * a_step, desc_hi, b_lo + k * b_step, desc_hi,
                                   idesc_k[k], sf_t, sf_t + 4 + sfb_col,
                                   (kb | k) != 0);
                    umma_commit(&empty[stage]);
                    sfr ^= 1;
                    if (++stage == STAGESX) {
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
        const int q = warp & 3;
        int buf = 0;
        uint32_t bphase = 0;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
            int m_blk, n_blk;
            tile_coords(tile, num_m, num_n, m_blk, n_blk);
            if (!mbar_wait_warp(&tfull[buf], bphase)) {
                if (lane == 0) atomicExch(p.status, 134);
                break;
            }
            tc_fence_after();
            const int row = m_blk * BM + q * 32 + lane;
            const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * BNX;
#pragma unroll 1
            for (int c = 0; c < BNX / 32; ++c) {
                const int col0 = n_blk * BNX + c * 32;
                if (col0 >= p.N) break;  // warp-uniform
                uint32_t r[32];
                tmem_ld_32x32(taddr + c * 32, r);
                tmem_wait_ld();
                if (row < p.M) epilogue_chunk(r, row, col0, p);
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

}  // namespace

// A, B: fp8 bytes ([M, K] / [N, K] K-major, or [K, M] / [K, N] MN-major; row pitches lda / ldb in bytes).  sfa, sfb:
// E8M0 scales in the tiled layout of neox_mxfp8_quant_tiled with sfa_mnb / sfb_mnb chunks per chunk row; sfb_mnb must
// be at least ceil(N / 128) + 1 (a 192-wide tile reads the chunk after its last one) and both buffers must cover
// ceil(K / 128) chunk rows.  The rest as neox_gemm_fp8.
extern "C" int neox_gemm_mxfp8(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                               long long ldd, int a_mn, int b_mn, int a_fmt, int b_fmt, const void* sfa,
                               long long sfa_mnb, const void* sfb, long long sfb_mnb, int d_fp32, const void* bias,
                               const void* add, long long ldadd, int add_fp32, void* preact, long long ldpre,
                               const void* aux, long long ldaux, int act, float alpha, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 16) || (ldb % 16) ||
        (reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15))
        return NEOX_ERR_ALIGN;
    if ((a_fmt | b_fmt) & ~1) return NEOX_ERR_SHAPE;
    if (sfa_mnb < (M + 127) / 128 || sfb_mnb < (N + 127) / 128 + 1) return NEOX_ERR_SHAPE;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;

    CUtensorMap tmA, tmB;
    int rc;
    if (!a_mn) rc = neox_make_tmap_u8_2d(&tmA, A, K, M, lda, BKX, BM);
    else rc = neox_make_tmap_u8_2d(&tmA, A, M, K, lda, 128, BKX);
    if (rc) return rc;
    if (!b_mn) rc = neox_make_tmap_u8_2d(&tmB, B, K, N, ldb, BKX, BNX);
    else rc = neox_make_tmap_u8_2d(&tmB, B, N, K, ldb, 128, BKX);
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
    MxParams x{static_cast<const unsigned char*>(sfa), static_cast<const unsigned char*>(sfb), sfa_mnb, sfb_mnb, a_fmt,
               b_fmt};

    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEMX_BYTES) !=
            cudaSuccess)
            return NEOX_ERR_LAUNCH;
        attr_set = true;
    }
    const int num_m = (M + BM - 1) / BM, num_n = (N + BNX - 1) / BNX;
    int grid = num_m * num_n;
    const int sms = neox_sm_count();
    if (grid > sms) grid = sms;
    gemm_mxfp8_kernel<<<grid, NUM_THREADS, SMEMX_BYTES, stream>>>(tmA, tmB, p, x);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
