// Persistent, warp-specialised bf16 GEMM for sm_100a:  D = epilogue(alpha * op(A) * op(B)).
//
//   * operands are staged global -> shared by TMA (cp.async.bulk.tensor, 128-byte swizzle) through a
//     4-deep mbarrier ring; one producer thread issues the copies;
//   * one thread issues tcgen05.mma (128 x 256 x 16 per instruction, cta_group::1), accumulating in
//     tensor memory; two 256-column accumulators are double-buffered so that the epilogue of tile i
//     overlaps the main loop of tile i+1;
//   * four epilogue warps read the accumulator with tcgen05.ld and apply the fused epilogue
//     (alpha, bias, optional store of the pre-activation, GeLU / GeLU', residual or gradient
//     accumulate, bf16 or fp32 output).
//
// Both operands may be K-major (the contraction index is contiguous in memory) or MN-major (the
// output index is contiguous); the four combinations cover forward (X·Wᵀ), dgrad (dY·W) and wgrad
// (dYᵀ·X) of a linear layer without any transposition pass.  This replaces the cuBLAS calls behind
// F.linear in megatron/mpu/layers.py:578,777 of the reference.
//
// All barrier waits are bounded (see sm100_ptx.cuh); on a time-out the kernel records a code in the
// status word, leaves its loops, frees its tensor memory and returns.
#include "gemm_common.cuh"
#include "neox_b200.h"
#include <mutex>
#include <unordered_map>
#include <string.h>
#include <stdio.h>

using namespace sm100;

using namespace gemm;

namespace {

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const GemmParams p) {
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
    const int ntiles = p.group_mode ? __ldg(p.group_ntiles) : num_m * num_n;
    const int nk = (p.K + BK - 1) / BK;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const TileInfo t = tile_info(p, tile, num_m, num_n, nk);
                for (int kb = 0; kb < t.nk; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1)) {
                        atomicExch(p.status, 101);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[stage], A_STAGE_BYTES + B_STAGE_BYTES);
                    uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
                    uint8_t* b_dst = sB + stage * B_STAGE_BYTES;
                    if (!p.a_mn) {
                        tma_load_2d(a_dst, &tmA, &full[stage], kb * BK, t.a_m0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j)
                            tma_load_2d(a_dst + j * (64 * BK * 2), &tmA, &full[stage], t.a_m0 + j * 64,
                                        t.a_k0 + kb * BK);
                    }
                    if (!p.b_mn) {
                        tma_load_2d(b_dst, &tmB, &full[stage], kb * BK, t.b_n0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(b_dst + j * (64 * BK * 2), &tmB, &full[stage], t.b_n0 + j * 64,
                                        t.b_k0 + kb * BK);
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
            const uint32_t idesc = make_idesc_16(BM, BN, p.a_mn, p.b_mn, p.h16);
            // operand descriptors: constant upper half; lower half = stage base + k-step offset (16-byte units), so
            // the issuing thread spends one add per operand per MMA.  K-major: the next 16 elements of K are 32
            // bytes along the swizzled row; MN-major: the next 16 rows of 128 bytes, with 64-element chunks of the
            // MN dimension 64 * BK * 2 bytes apart.
            const uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA), p.a_mn ? 64 * BK * 2 : 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(sB), p.b_mn ? 64 * BK * 2 : 16);
            const uint32_t a_step = (p.a_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            const uint32_t b_step = (p.b_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            int stage = 0;
            uint32_t phase = 0;
            int buf = 0;
            uint32_t bphase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                if (!mbar_wait(&tempty[buf], bphase ^ 1)) {
                    atomicExch(p.status, 102);
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                const int nk_t = p.group_mode == 2 ? __ldg(p.groups + tile).y : nk;
                for (int kb = 0; kb < nk_t; ++kb) {
                    if (!mbar_wait(&full[stage], phase)) {
                        atomicExch(p.status, 103);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + stage * (A_STAGE_BYTES >> 4);
                    const uint32_t b_lo = b_lo0 + stage * (B_STAGE_BYTES >> 4);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_ss_lohi<false, false>(tmem_d, a_lo + k * a_step, desc_hi, b_lo + k * b_step, desc_hi, idesc,
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
        const int q = warp & 3;  // tensor-memory lane quarter this warp may read
        int buf = 0;
        uint32_t bphase = 0;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
            const TileInfo t = tile_info(p, tile, num_m, num_n, nk);
            if (!mbar_wait_warp(&tfull[buf], bphase)) {
                if (lane == 0) atomicExch(p.status, 104);
                break;
            }
            tc_fence_after();
            const int row = t.row0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int col0 = t.n0 + c * 32;
                if (col0 >= p.N) break;  // warp-uniform
                uint32_t r[32];
                tmem_ld_32x32(taddr + c * 32, r);
                tmem_wait_ld();
                if (row < t.row_end) epilogue_chunk(r, row, col0, p);
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

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

struct MapKey {
    const void* ptr;
    unsigned long long d0, d1, ld;
    unsigned b0, b1;
    unsigned esize;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && ld == o.ld && b0 == o.b0 && b1 == o.b1 && esize == o.esize;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.ptr);
        h = h * 1000003u ^ k.d0;
        h = h * 1000003u ^ k.d1;
        h = h * 1000003u ^ k.ld;
        h = h * 1000003u ^ (size_t(k.b0) << 16 | k.b1);
        h = h * 1000003u ^ k.esize;
        return h;
    }
};

std::mutex g_map_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

}  // namespace

// Build (or fetch from a cache) the 2-D tensor map of a row-major [d1, d0] view of 1-byte (esize 1) or bf16
// (esize 2) elements with a row pitch of `ld` elements and a [b1, b0] box, 128-byte swizzled.
static int make_tmap_2d(CUtensorMap* out, const void* ptr, unsigned long long d0, unsigned long long d1,
                        unsigned long long ld, unsigned b0, unsigned b1, unsigned esize) {
    MapKey key{ptr, d0, d1, ld, b0, b1, esize};
    {
        std::lock_guard<std::mutex> g(g_map_mu);
        auto it = g_maps.find(key);
        if (it != g_maps.end()) {
            *out = it->second;
            return 0;
        }
    }
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return NEOX_ERR_DRIVER;
    cuuint64_t dims[2] = {d0, d1};
    cuuint64_t strides[1] = {ld * esize};
    cuuint32_t box[2] = {b0, b1};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, esize == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                     const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return NEOX_ERR_TMAP;
    std::lock_guard<std::mutex> g(g_map_mu);
    if (g_maps.size() > 8192) g_maps.clear();
    g_maps.emplace(key, *out);
    return 0;
}

int neox_make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, unsigned long long d0, unsigned long long d1,
                           unsigned long long ld, unsigned b0, unsigned b1) {
    return make_tmap_2d(out, ptr, d0, d1, ld, b0, b1, 2);
}

int neox_make_tmap_u8_2d(CUtensorMap* out, const void* ptr, unsigned long long d0, unsigned long long d1,
                         unsigned long long ld, unsigned b0, unsigned b1) {
    return make_tmap_2d(out, ptr, d0, d1, ld, b0, b1, 1);
}

// 4-D bf16 tensor map over a strided [d3, d2, d1, d0] view (d0 contiguous; strides in elements), box
// [b3, 1, 1, b0], 128-byte swizzled.  Used by the attention kernels to read [s, b, h, d] views in place.
int neox_make_tmap_bf16_4d(CUtensorMap* out, const void* ptr, unsigned long long d0, unsigned long long d1,
                           unsigned long long d2, unsigned long long d3, long long s1, long long s2, long long s3,
                           unsigned b0, unsigned b3) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return NEOX_ERR_DRIVER;
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (s1 % 8) || (s2 % 8) || (s3 % 8)) return NEOX_ERR_ALIGN;
    cuuint64_t dims[4] = {d0, d1, d2, d3};
    cuuint64_t strides[3] = {(cuuint64_t)s1 * 2, (cuuint64_t)s2 * 2, (cuuint64_t)s3 * 2};
    cuuint32_t box[4] = {b0, 1, 1, b3};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    // a size-1 dimension may carry any stride; the encoder wants strides that are positive multiples of 16
    for (int i = 0; i < 3; ++i)
        if (strides[i] == 0) strides[i] = 16;
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : NEOX_ERR_TMAP;
}

extern "C" int neox_gemm_bf16_rowmap(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                                     long long ldb, long long ldd, int a_mn, int b_mn, int d_fp32, const void* bias,
                                     const void* add, long long ldadd, int add_fp32, void* preact, long long ldpre,
                                     const void* aux, long long ldaux, int act, float alpha, const void* row_ptrs,
                                     void* stream_);

extern "C" int neox_gemm_16(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                            long long ldd, int a_mn, int b_mn, int d_fp32, const void* bias, const void* add,
                            long long ldadd, int add_fp32, void* preact, long long ldpre, const void* aux,
                            long long ldaux, int act, float alpha, const void* row_ptrs, int h16, void* stream_);

extern "C" int neox_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                              long long ldb, long long ldd, int a_mn, int b_mn, int d_fp32, const void* bias,
                              const void* add, long long ldadd, int add_fp32, void* preact, long long ldpre,
                              const void* aux, long long ldaux, int act, float alpha, void* stream_) {
    return neox_gemm_bf16_rowmap(A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, d_fp32, bias, add, ldadd, add_fp32, preact,
                                 ldpre, aux, ldaux, act, alpha, nullptr, stream_);
}

// row_ptrs (device array of M addresses, or NULL): destination of every output row (16-bit output; each address
// 16-byte aligned and valid for N elements).  With it D may be NULL.
extern "C" int neox_gemm_bf16_rowmap(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                                     long long ldb, long long ldd, int a_mn, int b_mn, int d_fp32, const void* bias,
                                     const void* add, long long ldadd, int add_fp32, void* preact, long long ldpre,
                                     const void* aux, long long ldaux, int act, float alpha, const void* row_ptrs,
                                     void* stream_) {
    return neox_gemm_16(A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, d_fp32, bias, add, ldadd, add_fp32, preact, ldpre,
                        aux, ldaux, act, alpha, row_ptrs, 0, stream_);
}

// The general entry point: h16 = 0 for bf16, 1 for fp16 (operands and every 16-bit epilogue tensor share the type).
extern "C" int neox_gemm_16(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                            long long ldd, int a_mn, int b_mn, int d_fp32, const void* bias, const void* add,
                            long long ldadd, int add_fp32, void* preact, long long ldpre, const void* aux,
                            long long ldaux, int act, float alpha, const void* row_ptrs, int h16, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (row_ptrs && d_fp32) return NEOX_ERR_SHAPE;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    // TMA constraints: 16-byte aligned base, row pitch a multiple of 16 bytes.
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8))
        return NEOX_ERR_ALIGN;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;

    CUtensorMap tmA, tmB;
    int rc;
    if (!a_mn) rc = neox_make_tmap_bf16_2d(&tmA, A, K, M, lda, BK, BM);
    else rc = neox_make_tmap_bf16_2d(&tmA, A, M, K, lda, 64, BK);
    if (rc) return rc;
    if (!b_mn) rc = neox_make_tmap_bf16_2d(&tmB, B, K, N, ldb, BK, BN);
    else rc = neox_make_tmap_bf16_2d(&tmB, B, N, K, ldb, 64, BK);
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
    p.row_ptrs = static_cast<const unsigned long long*>(row_ptrs);
    p.h16 = h16 ? 1 : 0;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    bool vec = row_ptrs ? (N % 8 == 0) : (al16(D) && (ldd % 8 == 0));
    if (bias) vec = vec && al16(bias);
    if (add) vec = vec && al16(add) && (ldadd % 8 == 0);
    if (preact) vec = vec && al16(preact) && (ldpre % 8 == 0);
    if (aux) vec = vec && al16(aux) && (ldaux % 8 == 0);
    p.vec_ok = vec ? 1 : 0;

    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             SMEM_BYTES);
        if (e != cudaSuccess) return NEOX_ERR_LAUNCH;
        attr_set = true;
    }
    const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN;
    int grid = num_m * num_n;
    const int sms = neox_sm_count();
    if (grid > sms) grid = sms;
    gemm_bf16_tcgen05_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// ------------------------------------------------------------------------------------------------------------
// Grouped GEMM for mixture-of-experts layers: all experts in one launch of the kernel above.
//
// The rows routed to expert e form one contiguous segment of the activation matrix; segment e starts at
// sum_{i<e} round_up(count_i, pad) (pad = 64 keeps every segment on a contraction-block boundary, which the weight
// gradient needs; the padding rows must hold zeros).  The tile table is built ON THE DEVICE from the per-expert
// counts, so routing never needs a host synchronisation.  Counterpart of the grouped / block-sparse expert GEMMs
// of the MegaBlocks library that the reference calls (megatron/model/moe_mlp.py of the reference: `gg.ops.gmm`).
__global__ void __launch_bounds__(256) moe_tile_table_kernel(const long long* __restrict__ counts, int E, int pad,
                                                             int mode, int num_m, int num_n, int b_stride,
                                                             int m_total, int max_tiles, int4* __restrict__ table,
                                                             int* __restrict__ ntiles) {
    extern __shared__ int sh[];   // [E] segment starts, [E] first tile of each expert
    int* seg = sh;
    int* first = sh + E;
    if (threadIdx.x == 0) {
        int row = 0, tile = 0;
        for (int e = 0; e < E; ++e) {
            const int c = (int)counts[e];
            seg[e] = row;
            first[e] = tile;
            row += (c + pad - 1) / pad * pad;
            if (mode == 1) tile += ((c + pad - 1) / pad * pad + BM - 1) / BM * num_n;
            else tile += c > 0 ? num_m * num_n : 0;
        }
        if (mode == 1 && row < m_total) {
            // rows behind the last segment (the matrix has a static, generous row count): their inputs are zero,
            // so running them through expert 0 stores zeros -- no row of the output is left uninitialised
            const int mb_n = (m_total - row + BM - 1) / BM;
            for (int nb = 0; nb < num_n; ++nb)
                for (int mb = 0; mb < mb_n; ++mb, ++tile)
                    if (tile < max_tiles) table[tile] = make_int4(row + mb * BM, m_total, 0, nb);
        }
        *ntiles = tile < max_tiles ? tile : max_tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int c = (int)counts[e];
        int t = first[e];
        if (mode == 1) {
            // the padding rows of a segment are computed too (their inputs are zero), so that every row a later
            // contraction-grouped GEMM reads holds a finite value
            const int cp = (c + pad - 1) / pad * pad;
            const int mb_n = (cp + BM - 1) / BM;
            for (int nb = 0; nb < num_n; ++nb)
                for (int mb = 0; mb < mb_n; ++mb, ++t)
                    if (t < max_tiles) table[t] = make_int4(seg[e] + mb * BM, seg[e] + cp, e * b_stride, nb);
        } else if (c > 0) {
            for (int nb = 0; nb < num_n; ++nb)
                for (int mb = 0; mb < num_m; ++mb, ++t)
                    if (t < max_tiles) table[t] = make_int4(seg[e], (c + BK - 1) / BK, e, (mb << 16) | nb);
        }
    }
}

// mode 1: D[rows of segment e, :] = act(alpha * A[rows, :] @ op(B_e)) (+ add), A [m_total, K] K-major, B the stacked
//         expert matrices: [E * N, K] K-major (b_mn = 0) or [E * K, N] MN-major (b_mn = 1; K % 64 == 0).
//         M = m_total (rows of A and D).
// mode 2: D[e * M + m, n] = sum over the rows r of segment e of A[r, m] * B[r, n] (+ add): A [m_total, M] and
//         B [m_total, N] both MN-major (a_mn = b_mn = 1), D the stacked [E * M, N]; `K` = m_total.
// `table` holds max_tiles int4 entries, `ntiles` one int; both are written by this call (on `stream`).
extern "C" int neox_gemm_grouped_16(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                                    long long ldb, long long ldd, int b_mn, int d_fp32, const void* add,
                                    long long ldadd, int add_fp32, void* preact, long long ldpre, const void* aux,
                                    long long ldaux, int act, float alpha, const long long* counts, int E, int pad,
                                    int mode, void* table, int max_tiles, int* ntiles, int h16, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (M <= 0 || N <= 0 || K <= 0 || E <= 0 || max_tiles <= 0) return 0;
    if (mode != 1 && mode != 2) return NEOX_ERR_SHAPE;
    if (E > 4096 || pad < 1) return NEOX_ERR_SHAPE;
    if (mode == 1 && b_mn && (K % BK)) return NEOX_ERR_SHAPE;   // an expert's contraction rows end on a block edge
    if (mode == 2 && (pad % BK)) return NEOX_ERR_SHAPE;         // segments start and end on contraction blocks
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8))
        return NEOX_ERR_ALIGN;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;

    CUtensorMap tmA, tmB;
    int rc;
    const int a_mn = mode == 2;
    if (mode == 1) {
        rc = neox_make_tmap_bf16_2d(&tmA, A, K, M, lda, BK, BM);
        if (rc) return rc;
        if (!b_mn) rc = neox_make_tmap_bf16_2d(&tmB, B, K, (unsigned long long)E * N, ldb, BK, BN);
        else rc = neox_make_tmap_bf16_2d(&tmB, B, N, (unsigned long long)E * K, ldb, 64, BK);
    } else {
        b_mn = 1;
        rc = neox_make_tmap_bf16_2d(&tmA, A, M, K, lda, 64, BK);
        if (rc) return rc;
        rc = neox_make_tmap_bf16_2d(&tmB, B, N, K, ldb, 64, BK);
    }
    if (rc) return rc;

    const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN;
    if (mode == 2 && (num_m > 0x7fff || num_n > 0xffff)) return NEOX_ERR_SHAPE;
    moe_tile_table_kernel<<<1, 256, 2 * E * sizeof(int), stream>>>(counts, E, pad, mode, num_m, num_n,
                                                                    b_mn ? K : N, M, max_tiles,
                                                                    static_cast<int4*>(table), ntiles);
    if (cudaGetLastError() != cudaSuccess) return NEOX_ERR_LAUNCH;

    GemmParams p;
    p.M = M; p.N = N; p.K = K;
    p.a_mn = a_mn; p.b_mn = b_mn;
    p.D = D; p.ldd = ldd; p.d_fp32 = d_fp32;
    p.bias = nullptr;
    p.add = add; p.ldadd = ldadd; p.add_fp32 = add_fp32;
    p.preact = static_cast<__nv_bfloat16*>(preact); p.ldpre = ldpre;
    p.aux = static_cast<const __nv_bfloat16*>(aux); p.ldaux = ldaux;
    p.act = act; p.alpha = alpha;
    p.status = status;
    p.row_ptrs = nullptr;
    p.h16 = h16 ? 1 : 0;
    p.groups = static_cast<const int4*>(table);
    p.group_ntiles = ntiles;
    p.group_mode = mode;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    bool vec = al16(D) && (ldd % 8 == 0);
    if (add) vec = vec && al16(add) && (ldadd % 8 == 0);
    if (preact) vec = vec && al16(preact) && (ldpre % 8 == 0);
    if (aux) vec = vec && al16(aux) && (ldaux % 8 == 0);
    p.vec_ok = vec ? 1 : 0;

    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_BYTES);
    if (e != cudaSuccess) return NEOX_ERR_LAUNCH;
    int grid = max_tiles;
    const int sms = neox_sm_count();
    if (grid > sms) grid = sms;
    gemm_bf16_tcgen05_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
