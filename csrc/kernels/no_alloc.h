// Allocation-free entry point.  This has no counterpart in the reference.
//
// Who needs it: the memory-scaling sweeps and the "max sequence length before out-of-memory" probes
// deliberately run a trainer with the device almost full, and the health checks that run right after
// an out-of-memory error (is the gradient still finite? how large is it?) run with the device
// completely full.  In both situations cudaMalloc -- and therefore torch.empty or any other
// allocating call -- fails or evicts the caching allocator's blocks, so the regular
// cpb_sumsq(), which wants a caller-allocated partial-sum buffer and ticket, cannot be fed.
// cpb_sumsq_noalloc() computes the same sum of squares of an fp32 vector using a small scratch
// area that is compiled into the library as a __device__ array, so the call allocates nothing.
//
//   * Scratch: CPB_NOALLOC_SCRATCH_BYTES (4352) bytes per GPU, held by every GPU that loads the
//     library until the process exits.
//   * Limit: n <= CPB_SUMSQ_NOALLOC_MAX_N elements; larger inputs are rejected with an error (the
//     return code is negative and cpb_last_error() names the limit), nothing is launched.
//   * Set-up: the first call on a device looks up the device address of the scratch array (once per
//     device, with that device current).  Make that first call outside any stream capture.
//   * Sharing: every call on a device uses the same scratch area, and the area keeps the previous
//     call's partial sums.  The entry point clears the one word that must start at zero (the
//     completion ticket) on the caller's stream before each launch.  Two calls whose kernels overlap on
//     the GPU (different streams, no ordering between them) race on the scratch area and return
//     garbage; order them on one stream or with events.
//   * It never calls cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define CPB_NOALLOC_SCRATCH_BYTES 4352
#define CPB_SUMSQ_NOALLOC_MAX_N 2147483647L

#ifdef __cplusplus
extern "C" {
#endif

// out[0] = sum_i g[i]^2 (fp32) for a device vector of n floats.  Returns 0, or a negative code with the
// reason available from cpb_last_error().
int cpb_sumsq_noalloc(const float* g, long n, float* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
