// Sum of squares of an fp32 vector without any allocation: the scratch area (per-block partial sums and
// the completion ticket) is a file-scope __device__ array.  See no_alloc.h for who needs this and for
// the rules of use.
#include "no_alloc.h"

#include "common.cuh"
#include "host_utils.h"

namespace cpb {

constexpr int NA_MAX_BLOCKS = 1024;                       // partial sums: 4096 bytes
constexpr int NA_TICKET_OFFSET = NA_MAX_BLOCKS * 4;       // one 32-bit ticket after them

// Held by every GPU that loads the library.  In host code this name is only a stand-in for the symbol:
// the device address is obtained with cudaGetSymbolAddress below and passed to the kernel.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CPB_NOALLOC_SCRATCH_BYTES];

__global__ void sumsq_noalloc_kernel(const float* __restrict__ g, size_t n, unsigned char* scratch, float* __restrict__ out) {
  float* partial = reinterpret_cast<float*>(scratch);
  unsigned int* ticket = reinterpret_cast<unsigned int*>(scratch + NA_TICKET_OFFSET);
  __shared__ float red[32];
  __shared__ bool last;
  float s = 0.f;
  const size_t n4 = n >> 2;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(g)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0)
    for (size_t i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x) s += g[i] * g[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) {
      partial[blockIdx.x] = t;
      __threadfence();
      last = (atomicAdd(ticket, 1u) == gridDim.x - 1);
    }
  }
  __syncthreads();
  if (last) {
    float t = 0.f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) t += reinterpret_cast<volatile float*>(partial)[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = t;
    __syncthreads();
    if (threadIdx.x < 32) {
      float u = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) u += __shfl_xor_sync(0xffffffffu, u, o);
      if (threadIdx.x == 0) out[0] = u;
    }
  }
}

}  // namespace cpb

using namespace cpb;

extern "C" int cpb_sumsq_noalloc(const float* g, long n, float* out, cudaStream_t stream) {
  if (n < 0 || n > CPB_SUMSQ_NOALLOC_MAX_N)
    return set_error(CPB_ERR_LIMIT, "sumsq_noalloc: n=%ld is outside [0, %ld], the size this allocation-free entry point supports", n, CPB_SUMSQ_NOALLOC_MAX_N);
  if (g == nullptr || out == nullptr) return set_error(CPB_ERR_ARG, "sumsq_noalloc: null pointer");
  if ((reinterpret_cast<uintptr_t>(g) & 15) != 0) return set_error(CPB_ERR_ARG, "sumsq_noalloc: input must be 16-byte aligned");
  // One-time set-up per device, with that device current: the device address of the scratch array.
  static unsigned char* scratch_of_device[64] = {nullptr};
  int dev = -1;
  CPB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(CPB_ERR_LIMIT, "sumsq_noalloc: device index %d not supported", dev);
  if (scratch_of_device[dev] == nullptr) {
    unsigned char* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return set_error(CPB_ERR_CUDA, "sumsq_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
    scratch_of_device[dev] = p;
  }
  unsigned char* scratch = scratch_of_device[dev];
  // The ticket must start at zero; the partial sums are overwritten before they are read.
  CPB_CUDA_OK(cudaMemsetAsync(scratch + NA_TICKET_OFFSET, 0, sizeof(unsigned int), stream));
  long blocks = (n / 4 + 255) / 256;
  if (blocks < 1) blocks = 1;
  const long cap = (long)sm_count() * 4;
  if (blocks > cap) blocks = cap;
  if (blocks > NA_MAX_BLOCKS) blocks = NA_MAX_BLOCKS;
  sumsq_noalloc_kernel<<<(int)blocks, 256, 0, stream>>>(g, (size_t)n, scratch, out);
  return check_launch("sumsq_noalloc");
}
