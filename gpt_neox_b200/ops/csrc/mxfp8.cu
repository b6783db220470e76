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

// One thread per 32-element block.  mode 0: q + scales out; mode 1: dequantised bf16 out (fused q -> dq).
template <bool E5M2>
__global__ void __launch_bounds__(256) mx_quant_kernel(const bf16* __restrict__ x, unsigned char* __restrict__ q,
                                                       unsigned char* __restrict__ scales, bf16* __restrict__ dq,
                                                       long long rows, long long cols, int along_rows) {
    const long long nblk = along_rows ? ((rows + 31) / 32) * cols : rows * ((cols + 31) / 32);
    for (long long bi = blockIdx.x * (long long)blockDim.x + threadIdx.x; bi < nblk;
         bi += (long long)gridDim.x * blockDim.x) {
        long long base, stride;
        int n;
        if (along_rows) {
            // consecutive threads take consecutive columns of the same 32-row band: coalesced
            const long long band = bi / cols, c = bi - band * cols;
            base = band * 32 * cols + c;
            stride = cols;
            n = (int)min(32LL, rows - band * 32);
        } else {
            const long long bpr = (cols + 31) / 32;
            const long long r = bi / bpr, b = bi - r * bpr;
            base = r * cols + b * 32;
            stride = 1;
            n = (int)min(32LL, cols - b * 32);
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
        if (scales) scales[bi] = (unsigned char)(amax > 0.f ? e + 127 : 0);
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

int grid_for_blocks(long long n) {
    long long g = (n + 255) / 256;
    const long long cap = 148LL * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

// x: bf16 [rows, cols] contiguous.  q (bytes, same shape) and scales (one byte per block) may be NULL, dq (bf16, same
// shape) may be NULL; e5m2 selects the element format.
extern "C" int neox_mxfp8_quant(const void* x, void* q, void* scales, void* dq, long long rows, long long cols,
                                int along_rows, int e5m2, void* stream) {
    if (rows <= 0 || cols <= 0) return 0;
    const long long nblk = along_rows ? ((rows + 31) / 32) * cols : rows * ((cols + 31) / 32);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (e5m2)
        mx_quant_kernel<true><<<grid_for_blocks(nblk), 256, 0, st>>>(static_cast<const bf16*>(x),
                                                                      static_cast<unsigned char*>(q),
                                                                      static_cast<unsigned char*>(scales),
                                                                      static_cast<bf16*>(dq), rows, cols, along_rows);
    else
        mx_quant_kernel<false><<<grid_for_blocks(nblk), 256, 0, st>>>(static_cast<const bf16*>(x),
                                                                       static_cast<unsigned char*>(q),
                                                                       static_cast<unsigned char*>(scales),
                                                                       static_cast<bf16*>(dq), rows, cols, along_rows);
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
