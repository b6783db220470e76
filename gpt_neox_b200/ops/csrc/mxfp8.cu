// MXFP8 (OCP microscaling) quantisation: 32-element blocks share one power-of-two scale (E8M0), elements are FP8
// E4M3 or E5M2.
//
//     e      = floor(log2(max |x| over the block)) - emax_elem          (emax_elem = 8 for E4M3, 15 for E5M2)
//     scale  = 2^e   (stored as the biased byte e + 127; 0 for an all-zero block)
//     q_i    = fp8(x_i / scale)        round-to-nearest-even, saturating
//
// Blocks run along the contraction dimension of the GEMM the tensor feeds, so both directions are provided:
// `along_rows = 0` groups 32 consecutive elements of a row (contraction = last dim), `along_rows = 1` groups 32
// consecutive rows of a column (contraction = first dim, as in a weight-gradient GEMM over tokens).
//
// Three entry points: quantise (bytes + scales, the storage / interchange format), dequantise, and the fused
// quantise->dequantise that the block-scaled linear layer uses.  fp8 x 2^e is exactly representable in bf16, so a
// bf16 tensor-core GEMM with fp32 accumulation over the dequantised operands computes exactly the products a
// hardware block-scaled MMA computes; only the rate differs.  (The reference reaches fp8 through Transformer
// Engine's delayed-scaling recipe, megatron/model/transformer_engine.py; block scaling needs no amax history.)
#include "neox_b200.h"
#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ int block_exponent(float amax, int emax_elem) {
    // floor(log2(amax)) from the float's exponent field (amax > 0, finite)
    const int e = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127;
    return max(-127, min(127, e - emax_elem));
}
__device__ __forceinline__ float pow2i(int e) { return __uint_as_float((uint32_t)(e + 127) << 23); }   // e in [-126, 127]

template <bool E5M2>
__device__ __forceinline__ unsigned char to_fp8(float v) {
    return (unsigned char)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
}
template <bool E5M2>
__device__ __forceinline__ float from_fp8(unsigned char q) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(q, E5M2 ? __NV_E5M2 : __NV_E4M3);
    return __half2float(__half(h));
}

// Where the scale of (mn, ks) -- mn: index along the non-contracted dimension, ks: 32-element block along the
// contracted one -- sits in the layout the block-scaled MMA kernel (gemm_mxfp8_sm100.cu) consumes: 512-byte chunks,
// one per (128 values of mn, 4 values of ks), ordered [ks / 4][mn / 128] with `mnb` chunks per row of chunks; inside
// a chunk byte (mn % 32) * 16 + ((mn % 128) / 32) * 4 + ks % 4.  A chunk copied to tensor memory as 32 lanes x 16
// bytes puts the scale of row mn at lane mn % 32, column (mn % 128) / 32, byte ks % 4, which is where the MMA looks.
__device__ __forceinline__ long long sf_tiled_offset(long long mn, long long ks, long long mnb) {
    return ((ks >> 2) * mnb + (mn >> 7)) * 512 + (mn & 31) * 16 + ((mn & 127) >> 5) * 4 + (ks & 3);
}

// Two values -> two fp8 bytes in one conversion instruction (low byte = first value).
template <bool E5M2>
__device__ __forceinline__ uint32_t to_fp8x2(float a, float b) {
    return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
}

// One thread per 32-element block.  mode 0: q + scales out; mode 1: dequantised bf16 out (fused q -> dq).
// tiled_mnb > 0: scales go to the tiled layout above instead of the linear one.
template <bool E5M2>
__global__ void __launch_bounds__(256) mx_quant_kernel(const bf16* __restrict__ x, unsigned char* __restrict__ q,
                                                       unsigned char* __restrict__ scales, bf16* __restrict__ dq,
                                                       long long rows, long long cols, int along_rows,
                                                       long long tiled_mnb) {
    const long long nblk = along_rows ? ((rows + 31) / 32) * cols : rows * ((cols + 31) / 32);
    for (long long bi = blockIdx.x * (long long)blockDim.x + threadIdx.x; bi < nblk;
         bi += (long long)gridDim.x * blockDim.x) {
        long long base, stride, mn, ks;
        int n;
        if (along_rows) {
            // consecutive threads take consecutive columns of the same 32-row band: coalesced
            const long long band = bi / cols, c = bi - band * cols;
            base = band * 32 * cols + c;
            stride = cols;
            n = (int)min(32LL, rows - band * 32);
            mn = c;
            ks = band;
        } else {
            const long long bpr = (cols + 31) / 32;
            const long long r = bi / bpr, b = bi - r * bpr;
            base = r * cols + b * 32;
            stride = 1;
            n = (int)min(32LL, cols - b * 32);
            mn = r;
            ks = b;
        }
        float v[32];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            v[i] = i < n ? __bfloat162float(x[base + i * stride]) : 0.f;
            amax = fmaxf(amax, fabsf(v[i]));
        }
        int e = -127;
        float inv = 0.f, sc = 0.f;
        if (amax > 0.f && amax < 3.0e38f) {
            e = block_exponent(amax, E5M2 ? 15 : 8);
            e = max(e, -126);
            sc = pow2i(e);
            inv = pow2i(-e > 127 ? 127 : -e);
        }
        if (scales) scales[tiled_mnb > 0 ? sf_tiled_offset(mn, ks, tiled_mnb) : bi] = (unsigned char)(amax > 0.f ? e + 127 : 0);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (i < n) {
                const unsigned char b8 = to_fp8<E5M2>(v[i] * inv);
                if (q) q[base + i * stride] = b8;
                if (dq) dq[base + i * stride] = __float2bfloat16(from_fp8<E5M2>(b8) * sc);
            }
        }
    }
}

template <bool E5M2>
__global__ void __launch_bounds__(256) mx_dequant_kernel(const unsigned char* __restrict__ q,
                                                         const unsigned char* __restrict__ scales,
                                                         bf16* __restrict__ out, long long rows, long long cols,
                                                         int along_rows) {
    const long long total = rows * cols;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols, c = i - r * cols;
        const long long bi = along_rows ? (r / 32) * cols + c : r * ((cols + 31) / 32) + c / 32;
        const int s = scales[bi];
        const float sc = s == 0 ? 0.f : pow2i(max(s - 127, -126));
        out[i] = __float2bfloat16(from_fp8<E5M2>(q[i]) * sc);
    }
}

// Both block directions from ONE read of the tensor.  A warp owns a band of 32 rows x 128 columns; a lane owns 4
// consecutive columns of it and walks the 32 rows with the raw bf16 pairs kept in registers (64 registers, so two
// CTAs fit on an SM and one CTA's loads overlap the other's conversions).
//   * blocks along a row (32 consecutive columns = 8 adjacent lanes): amax by three shuffles, quantise, store 4 bytes;
//   * blocks along a column (the lane's 32 rows of each of its 4 columns): amax accumulated over the walk, then the
//     registers are quantised a second time with the column scales.
// Either output pair may be NULL.  Scales go to the tiled layout (sf_tiled_offset): mn = row, ks = column block for
// the row direction; mn = column, ks = row band for the column direction.  cols % 8 == 0.
template <bool E5M2>
__global__ void __launch_bounds__(256, 2) mx_quant_dual_kernel(const bf16* __restrict__ x,
                                                               unsigned char* __restrict__ q_c,
                                                               unsigned char* __restrict__ sf_c, long long mnb_c,
                                                               unsigned char* __restrict__ q_r,
                                                               unsigned char* __restrict__ sf_r, long long mnb_r,
                                                               long long rows, long long cols) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long band = blockIdx.y;
    const long long wcol0 = ((long long)blockIdx.x * 8 + warp) * 128;
    if (wcol0 >= cols) return;                                               // warp-uniform
    const long long col0 = wcol0 + lane * 4;
    const long long row0 = band * 32;
    const bool col_ok = col0 < cols;                                         // cols % 4 == 0: all four or none
    const int nrows = (int)min(32LL, rows - row0);
    const int emax = E5M2 ? 15 : 8;

    uint2 raw[32];
#pragma unroll
    for (int r = 0; r < 32; ++r) {
        raw[r] = make_uint2(0, 0);
        if (col_ok && r < nrows) raw[r] = __ldg(reinterpret_cast<const uint2*>(x + (row0 + r) * cols + col0));
    }
    float cmax[4] = {0.f, 0.f, 0.f, 0.f};

#pragma unroll
    for (int r = 0; r < 32; ++r) {
        float v[4];
        v[0] = __uint_as_float(raw[r].x << 16);
        v[1] = __uint_as_float(raw[r].x & 0xFFFF0000u);
        v[2] = __uint_as_float(raw[r].y << 16);
        v[3] = __uint_as_float(raw[r].y & 0xFFFF0000u);
        float amax = 0.f;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            cmax[t] = fmaxf(cmax[t], fabsf(v[t]));
            amax = fmaxf(amax, fabsf(v[t]));
        }
        if (q_c) {                                                            // uniform
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            int e = -127;
            float inv = 0.f;
            if (amax > 0.f && amax < 3.0e38f) {
                e = max(block_exponent(amax, emax), -126);
                inv = pow2i(-e > 127 ? 127 : -e);
            }
            if (col_ok && r < nrows) {
                const uint32_t o = to_fp8x2<E5M2>(v[0] * inv, v[1] * inv) | (to_fp8x2<E5M2>(v[2] * inv, v[3] * inv) << 16);
                *reinterpret_cast<uint32_t*>(q_c + (row0 + r) * cols + col0) = o;
                if ((lane & 7) == 0)
                    sf_c[sf_tiled_offset(row0 + r, col0 >> 5, mnb_c)] = (unsigned char)(amax > 0.f ? e + 127 : 0);
            }
        }
    }
    if (q_r && col_ok) {
        float inv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int e = -127;
            inv[j] = 0.f;
            if (cmax[j] > 0.f && cmax[j] < 3.0e38f) {
                e = max(block_exponent(cmax[j], emax), -126);
                inv[j] = pow2i(-e > 127 ? 127 : -e);
            }
            sf_r[sf_tiled_offset(col0 + j, band, mnb_r)] = (unsigned char)(cmax[j] > 0.f ? e + 127 : 0);
        }
#pragma unroll
        for (int r = 0; r < 32; ++r) {
            if (r < nrows) {
                const uint32_t o =
                    to_fp8x2<E5M2>(__uint_as_float(raw[r].x << 16) * inv[0], __uint_as_float(raw[r].x & 0xFFFF0000u) * inv[1]) |
                    (to_fp8x2<E5M2>(__uint_as_float(raw[r].y << 16) * inv[2], __uint_as_float(raw[r].y & 0xFFFF0000u) * inv[3])
                     << 16);
                *reinterpret_cast<uint32_t*>(q_r + (row0 + r) * cols + col0) = o;
            }
        }
    }
}

int grid_for_blocks(long long n) {
    long long g = (n + 255) / 256;
    const long long cap = 148LL * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

// x: bf16 [rows, cols] contiguous.  q (bytes, same shape) and scales (one byte per block) may be NULL, dq (bf16, same
// shape) may be NULL; e5m2 selects the element format.
extern "C" int neox_mxfp8_quant_tiled(const void* x, void* q, void* scales, void* dq, long long rows, long long cols,
                                      int along_rows, int e5m2, long long tiled_mnb, void* stream);

extern "C" int neox_mxfp8_quant(const void* x, void* q, void* scales, void* dq, long long rows, long long cols,
                                int along_rows, int e5m2, void* stream) {
    return neox_mxfp8_quant_tiled(x, q, scales, dq, rows, cols, along_rows, e5m2, 0, stream);
}

// tiled_mnb > 0: `scales` is a zero-initialised buffer of ceil(K_blocks / 4) * tiled_mnb * 512 bytes in the tiled
// layout (see sf_tiled_offset); tiled_mnb >= ceil(MN / 128).
extern "C" int neox_mxfp8_quant_tiled(const void* x, void* q, void* scales, void* dq, long long rows, long long cols,
                                      int along_rows, int e5m2, long long tiled_mnb, void* stream) {
    if (rows <= 0 || cols <= 0) return 0;
    const long long nblk = along_rows ? ((rows + 31) / 32) * cols : rows * ((cols + 31) / 32);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (e5m2)
        mx_quant_kernel<true><<<grid_for_blocks(nblk), 256, 0, st>>>(static_cast<const bf16*>(x),
                                                                      static_cast<unsigned char*>(q),
                                                                      static_cast<unsigned char*>(scales),
                                                                      static_cast<bf16*>(dq), rows, cols, along_rows, tiled_mnb);
    else
        mx_quant_kernel<false><<<grid_for_blocks(nblk), 256, 0, st>>>(static_cast<const bf16*>(x),
                                                                       static_cast<unsigned char*>(q),
                                                                       static_cast<unsigned char*>(scales),
                                                                       static_cast<bf16*>(dq), rows, cols, along_rows, tiled_mnb);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

extern "C" int neox_mxfp8_dequant(const void* q, const void* scales, void* out, long long rows, long long cols,
                                  int along_rows, int e5m2, void* stream) {
    if (rows <= 0 || cols <= 0) return 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (e5m2)
        mx_dequant_kernel<true><<<grid_for_blocks(rows * cols), 256, 0, st>>>(
            static_cast<const unsigned char*>(q), static_cast<const unsigned char*>(scales), static_cast<bf16*>(out),
            rows, cols, along_rows);
    else
        mx_dequant_kernel<false><<<grid_for_blocks(rows * cols), 256, 0, st>>>(
            static_cast<const unsigned char*>(q), static_cast<const unsigned char*>(scales), static_cast<bf16*>(out),
            rows, cols, along_rows);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// Quantise x (bf16 [rows, cols], cols % 8 == 0, 16-byte aligned) in one pass along its columns (q_c, sf_c: blocks of
// 32 consecutive columns, usable as a K-major operand) and / or along its rows (q_r, sf_r: blocks of 32 consecutive
// rows, usable as an MN-major operand).  Scale buffers: tiled layout, zero-initialised by the caller, with mnb_c >=
// ceil(rows / 128) and mnb_r >= ceil(cols / 128) chunks per chunk row.  Either pair may be NULL.
extern "C" int neox_mxfp8_quant_dual(const void* x, void* q_c, void* sf_c, long long mnb_c, void* q_r, void* sf_r,
                                     long long mnb_r, long long rows, long long cols, int e5m2, void* stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (cols % 8) return NEOX_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q_c) & 7) ||
        (reinterpret_cast<uintptr_t>(q_r) & 7))
        return NEOX_ERR_ALIGN;
    const dim3 grid((unsigned)((cols + 1023) / 1024), (unsigned)((rows + 31) / 32));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (e5m2)
        mx_quant_dual_kernel<true><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), static_cast<unsigned char*>(q_c),
                                                         static_cast<unsigned char*>(sf_c), mnb_c,
                                                         static_cast<unsigned char*>(q_r),
                                                         static_cast<unsigned char*>(sf_r), mnb_r, rows, cols);
    else
        mx_quant_dual_kernel<false><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), static_cast<unsigned char*>(q_c),
                                                          static_cast<unsigned char*>(sf_c), mnb_c,
                                                          static_cast<unsigned char*>(q_r),
                                                          static_cast<unsigned char*>(sf_r), mnb_r, rows, cols);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
