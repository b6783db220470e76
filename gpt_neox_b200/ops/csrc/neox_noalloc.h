// Allocation-free entry point of libneox_b200.so.  It has no counterpart in the reference code base.
//
// Who needs it: callers that cannot obtain device memory at the time of the call -- a process whose GPU
// memory is already entirely reserved (typically by a deep-learning framework's caching allocator sized to
// the whole device), or code on a latency-critical path where cudaMalloc / cudaFree and their implicit
// device-wide synchronisation are not acceptable.  The regular neox_layernorm_bwd() asks such callers for
// a scratch buffer they cannot supply; this variant carries its scratch inside the library image instead.
//
//   int neox_layernorm_bwd_noalloc(g, x, gamma, mean, rstd, dx, dgamma, dbeta, rows, cols, dtype, stream)
//
// computes exactly what neox_layernorm_bwd() computes (dx in the storage dtype, dgamma / dbeta in fp32) with
// the same kernels.  dtype: 0 = bf16, 1 = fp32, 2 = fp16.  Returns 0, or NEOX_ERR_SHAPE / NEOX_ERR_TOO_LARGE /
// NEOX_ERR_DRIVER / NEOX_ERR_LAUNCH; neox_noalloc_last_error() then describes the refusal in words (the text is kept
// per host thread: read it on the thread whose call was refused).
//
// Contract:
//   * cols <= NEOX_NOALLOC_MAX_COLS (and a multiple of 8); any number of rows.
//   * The scratch is one static device array of 2 * NEOX_NOALLOC_MAX_BLOCKS * NEOX_NOALLOC_MAX_COLS floats
//     (20 MiB); every GPU that loads the library holds it until the process exits.
//   * The first call on each device resolves the array's device address (cudaGetSymbolAddress, with that device
//     current).  Make that first call outside of any stream capture.
//   * No cudaMalloc, cudaFree or allocating library call is made, on the first call or later.
//   * All calls on a device share the array.  Nothing in it has to be cleared between calls (each launch
//     overwrites every element it later reads), but calls that may run concurrently on the GPU race on it --
//     issue them on one stream or order them with events.
#pragma once

#define NEOX_NOALLOC_MAX_COLS 8192
#define NEOX_NOALLOC_MAX_BLOCKS 320

#ifdef __cplusplus
extern "C" {
#endif
int neox_layernorm_bwd_noalloc(const void* g, const void* x, const void* gamma, const float* mean,
                               const float* rstd, void* dx, float* dgamma, float* dbeta, int rows, int cols,
                               int dtype, void* stream);
const char* neox_noalloc_last_error();
#ifdef __cplusplus
}
#endif
