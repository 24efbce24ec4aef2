// Allocation-free entry point of libtt_b200.  It has no counterpart in the reference
// framework; it exists for hosts that cannot allocate device memory at call time.
//
// Who needs it: a process that handed all free device memory to another allocator up front
// (so a late cudaMalloc simply fails), or code running on a path where cudaMalloc's implicit
// device-wide synchronisation is not acceptable, such as a latency-critical loop or a host
// callback.  Those callers still own their inputs and outputs; what they cannot provide is the
// temporary buffer a two-stage reduction needs.
//
//   tt_colsum_noalloc : out[c] (+)= sum over rows of x[r, c]
//
// Same result as tt_colsum (bias-gradient column sums), but the partial sums live in a
// file-scope device array of fixed size inside the library instead of a caller-provided
// scratch buffer.  Limits and rules:
//   * C <= TT_COLSUM_NOALLOC_MAX_C (a multiple of 8, like tt_colsum); larger C is rejected with
//     an error, nothing is launched.  rows is unbounded.
//   * the array (TT_COLSUM_NOALLOC_CHUNKS x TT_COLSUM_NOALLOC_MAX_C floats = 4 MiB) is part of
//     the library image: every GPU that loads the library holds it until the process exits.
//   * the first call on a device looks up the array's device address (once per device, with that
//     device current) and so should happen before any stream capture begins on that device.
//   * all calls on a device share the array and it keeps the previous call's partial sums.  Stage
//     one overwrites every element stage two reads, so nothing has to be cleared between calls,
//     but two calls whose kernels overlap on the GPU (different streams without ordering) race
//     on it: keep calls on one stream or order them with events.
//   * the function calls no cudaMalloc / cudaFree and no allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define TT_COLSUM_NOALLOC_MAX_C 16384
#define TT_COLSUM_NOALLOC_CHUNKS 64

#ifdef __cplusplus
extern "C" {
#endif

// x: bf16 [rows, C] with row stride ldx (elements, multiple of 8, 16-byte aligned base).
// out: fp32 (out_fp32 != 0) or bf16 [C].  accumulate != 0 adds to out instead of overwriting.
// Returns 0 on success, negative on error (message via tt_last_error()).
int tt_colsum_noalloc(const void* x, long long ldx, void* out, int out_fp32, int accumulate, int rows,
                      int C, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
