// Host-side helpers shared by the launchers: last-error string, tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda, so the library also loads on a machine
// without a GPU driver), device properties cache.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

namespace cpb {

// error codes returned by every extern "C" launcher
enum : int { CPB_OK = 0, CPB_ERR_ARG = -1, CPB_ERR_CUDA = -2, CPB_ERR_DRIVER = -3, CPB_ERR_LIMIT = -4 };

char* last_error_buf();                     // thread-local, 512 bytes
int set_error(int code, const char* fmt, ...);
int sm_count();                             // SMs of the current device
int check_launch(const char* what);         // cudaGetLastError -> code

// Encode a tiled tensor map for a bf16/fp32 tensor.  dims/strides are innermost-first; strides in
// bytes for dims 1..rank-1 (dim 0 is contiguous).  swizzle: 0 none, 1 = 128-byte.
int encode_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, int swizzle128);

#define CPB_CUDA_OK(expr)                                                              \
  do {                                                                                 \
    cudaError_t _e = (expr);                                                           \
    if (_e != cudaSuccess) return cpb::set_error(cpb::CPB_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

}  // namespace cpb
