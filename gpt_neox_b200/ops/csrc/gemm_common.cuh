// Shared pieces of the tcgen05 GEMM kernels (plain and communication-fused): tile constants, the parameter
// block, the L2-friendly tile order and the fused epilogue applied to 32 accumulator columns of one row.
#pragma once
#include "sm100_ptx.cuh"

namespace gemm {
using namespace sm100;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 16;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 256 + 1024;

struct GemmParams {
    int M, N, K;
    int a_mn, b_mn;
    void* D;
    long long ldd;
    int d_fp32;
    const __nv_bfloat16* bias;
    const void* add;
    long long ldadd;
    int add_fp32;
    __nv_bfloat16* preact;
    long long ldpre;
    const __nv_bfloat16* aux;
    long long ldaux;
    int act;
    float alpha;
    int vec_ok;
    int* status;
    // optional per-row destination table (bf16 output only): row r is stored at address row_ptrs[r] instead of
    // D + r * ldd -- the rows of one GEMM can then land in different buffers, including peers' memory
    const unsigned long long* row_ptrs;
    int h16 = 0;   // 16-bit storage type of the operands, D, bias, add, preact, aux: 0 = bf16, 1 = fp16
    // grouped GEMM (one launch for all experts of a mixture-of-experts layer): a device-built table with one int4
    // per output tile, and a device word with the number of valid entries.
    //   mode 1, rows grouped (forward, dgrad): {first row of A / D, end row of the segment, offset of this expert
    //           in B (rows of a K-major B, contraction rows of an MN-major B), column block}
    //   mode 2, contraction grouped (wgrad): {first contraction row, number of 64-row contraction blocks, expert
    //           (output rows e * M ...), row block << 16 | column block}
    const int4* groups = nullptr;
    const int* group_ntiles = nullptr;
    int group_mode = 0;
};

// Where one output tile reads and writes: plain tiles come from tile_coords, grouped ones from the table.
struct TileInfo {
    int a_m0;      // row coordinate of A's tile (MN index)
    int a_k0;      // contraction offset of an MN-major A
    int b_n0;      // row coordinate of B's tile (MN index, plus the expert's row offset for a K-major B)
    int b_k0;      // contraction offset of an MN-major B
    int n0;        // first output column
    int nk;        // contraction blocks of BK
    int row0;      // output row of accumulator lane 0
    int row_end;   // rows at or beyond it are not stored
};

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_blk, int& n_blk) {
    const int per_group = GROUP_M * num_n;
    const int group = tile / per_group;
    const int first_m = group * GROUP_M;
    const int gsize = min(num_m - first_m, GROUP_M);
    const int in_group = tile - group * per_group;
    m_blk = first_m + in_group % gsize;
    n_blk = in_group / gsize;
}

__device__ __forceinline__ TileInfo tile_info(const GemmParams& p, int tile, int num_m, int num_n, int nk_all) {
    TileInfo t;
    if (p.group_mode == 0) {
        int m_blk, n_blk;
        tile_coords(tile, num_m, num_n, m_blk, n_blk);
        t.a_m0 = m_blk * BM; t.a_k0 = 0; t.b_n0 = n_blk * BN; t.b_k0 = 0; t.n0 = n_blk * BN; t.nk = nk_all;
        t.row0 = m_blk * BM; t.row_end = p.M;
    } else if (p.group_mode == 1) {
        const int4 g = __ldg(p.groups + tile);
        t.a_m0 = g.x; t.a_k0 = 0; t.n0 = g.w * BN; t.nk = nk_all;
        t.b_n0 = p.b_mn ? t.n0 : g.z + t.n0;
        t.b_k0 = p.b_mn ? g.z : 0;
        t.row0 = g.x; t.row_end = g.y;
    } else {
        const int4 g = __ldg(p.groups + tile);
        const int m_blk = g.w >> 16, n_blk = g.w & 0xffff;
        t.a_m0 = m_blk * BM; t.a_k0 = g.x; t.b_n0 = n_blk * BN; t.b_k0 = g.x; t.n0 = n_blk * BN; t.nk = g.y;
        t.row0 = g.z * p.M + m_blk * BM; t.row_end = g.z * p.M + p.M;
    }
    return t;
}

// Apply the fused epilogue to 32 consecutive columns of one output row (H16: fp16 storage, else bf16).
template <bool H16>
__device__ __forceinline__ void epilogue_chunk_t(const uint32_t (&r)[32], int row, int col0, const GemmParams& p) {
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
    const bool full = p.vec_ok && (col0 + 32 <= p.N);
    if (full) {
        if (p.bias) {
            const uint4* b4 = reinterpret_cast<const uint4*>(p.bias + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint4 b = __ldg(b4 + j);
                uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    v[j * 8 + t * 2] += lo_16<H16>(w[t]);
                    v[j * 8 + t * 2 + 1] += hi_16<H16>(w[t]);
                }
            }
        }
        if (p.preact) {
            uint4* o = reinterpret_cast<uint4*>(p.preact + (long long)row * p.ldpre + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint4 q;
                q.x = pack_16x2<H16>(v[j * 8 + 0], v[j * 8 + 1]);
                q.y = pack_16x2<H16>(v[j * 8 + 2], v[j * 8 + 3]);
                q.z = pack_16x2<H16>(v[j * 8 + 4], v[j * 8 + 5]);
                q.w = pack_16x2<H16>(v[j * 8 + 6], v[j * 8 + 7]);
                o[j] = q;
            }
        }
        if (p.act == 1) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
        } else if (p.act == 2) {
            const uint4* a4 = reinterpret_cast<const uint4*>(p.aux + (long long)row * p.ldaux + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint4 a = __ldg(a4 + j);
                uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    v[j * 8 + t * 2] *= dgelu_tanh(lo_16<H16>(w[t]));
                    v[j * 8 + t * 2 + 1] *= dgelu_tanh(hi_16<H16>(w[t]));
                }
            }
        }
        // fp32 accumulate into the output itself (weight gradients into the main-gradient buffer): every element is
        // owned by one thread, so a vector reduction at the L2 does the read-modify-write and the SM never waits
        // for the old value
        const bool inplace = p.d_fp32 && p.add_fp32 && p.add == p.D && p.ldadd == p.ldd;
        if (p.add && !inplace) {
            if (p.add_fp32) {
                const float4* a4 = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.add) +
                                                                   (long long)row * p.ldadd + col0);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float4 a = a4[j];
                    v[j * 4 + 0] += a.x;
                    v[j * 4 + 1] += a.y;
                    v[j * 4 + 2] += a.z;
                    v[j * 4 + 3] += a.w;
                }
            } else {
                const uint4* a4 = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.add) +
                                                                 (long long)row * p.ldadd + col0);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint4 a = a4[j];
                    uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        v[j * 8 + t * 2] += lo_16<H16>(w[t]);
                        v[j * 8 + t * 2 + 1] += hi_16<H16>(w[t]);
                    }
                }
            }
        }
        if (p.d_fp32) {
            float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.D) + (long long)row * p.ldd + col0);
            if (inplace) {
#pragma unroll
                for (int j = 0; j < 8; ++j) atomicAdd(o + j, make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]));
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
            }
        } else {
            __nv_bfloat16* drow = p.row_ptrs ? reinterpret_cast<__nv_bfloat16*>(p.row_ptrs[row])
                                             : reinterpret_cast<__nv_bfloat16*>(p.D) + (long long)row * p.ldd;
            uint4* o = reinterpret_cast<uint4*>(drow + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint4 q;
                q.x = pack_16x2<H16>(v[j * 8 + 0], v[j * 8 + 1]);
                q.y = pack_16x2<H16>(v[j * 8 + 2], v[j * 8 + 3]);
                q.z = pack_16x2<H16>(v[j * 8 + 4], v[j * 8 + 5]);
                q.w = pack_16x2<H16>(v[j * 8 + 6], v[j * 8 + 7]);
                o[j] = q;
            }
        }
    } else {
        // ragged / unaligned edge: element-wise with bounds checks
        for (int i = 0; i < 32; ++i) {
            const int col = col0 + i;
            if (col >= p.N) break;
            float x = v[i];
            if (p.bias) x += ld_16<H16>(p.bias, col);
            if (p.preact) st_16<H16>(p.preact, (long long)row * p.ldpre + col, x);
            if (p.act == 1) x = gelu_tanh(x);
            else if (p.act == 2) x *= dgelu_tanh(ld_16<H16>(p.aux, (long long)row * p.ldaux + col));
            if (p.add) {
                if (p.add_fp32) x += reinterpret_cast<const float*>(p.add)[(long long)row * p.ldadd + col];
                else x += ld_16<H16>(p.add, (long long)row * p.ldadd + col);
            }
            if (p.d_fp32) reinterpret_cast<float*>(p.D)[(long long)row * p.ldd + col] = x;
            else if (p.row_ptrs) st_16<H16>(reinterpret_cast<void*>(p.row_ptrs[row]), col, x);
            else st_16<H16>(p.D, (long long)row * p.ldd + col, x);
        }
    }
}

__device__ __forceinline__ void epilogue_chunk(const uint32_t (&r)[32], int row, int col0, const GemmParams& p) {
    if (p.h16) epilogue_chunk_t<true>(r, row, col0, p);
    else epilogue_chunk_t<false>(r, row, col0, p);
}

}  // namespace gemm
