// C ABI shared by every kernel file in this library.  All entry points are `extern "C"`, take raw
// device pointers plus a CUDA stream handle, launch asynchronously on that stream and return 0 on
// success or one of the NEOX_ERR_* codes below.  Python binds them through ctypes
// (gpt_neox_b200/ops/native.py).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#define NEOX_ERR_ALIGN 1    // pointer or pitch violates an alignment requirement
#define NEOX_ERR_TMAP 2     // cuTensorMapEncodeTiled rejected the descriptor
#define NEOX_ERR_DRIVER 3   // a driver entry point / allocation was unavailable
#define NEOX_ERR_LAUNCH 4   // the kernel launch itself failed
#define NEOX_ERR_SHAPE 5    // unsupported shape for this kernel
#define NEOX_ERR_TOO_LARGE 6  // request exceeds a compiled-in maximum

// Per-device 32-bit status word in global memory.  Kernels store a non-zero code there when a
// bounded wait gives up; the host reads and clears it with neox_read_status().
int* neox_status_word();
int neox_sm_count();
int neox_make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, unsigned long long d0, unsigned long long d1,
                           unsigned long long ld, unsigned b0, unsigned b1);

int neox_make_tmap_u8_2d(CUtensorMap* out, const void* ptr, unsigned long long d0, unsigned long long d1,
                         unsigned long long ld, unsigned b0, unsigned b1);
int neox_make_tmap_bf16_4d(CUtensorMap* out, const void* ptr, unsigned long long d0, unsigned long long d1,
                           unsigned long long d2, unsigned long long d3, long long s1, long long s2, long long s3,
                           unsigned b0, unsigned b3);

extern "C" {
int neox_read_status();  // synchronises the device; returns and clears the status word
int neox_norm_bwd_blocks(int rows);  // CTAs (= partial rows of scratch) the norm backward kernels use
}
