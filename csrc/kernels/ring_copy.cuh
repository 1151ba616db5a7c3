// Copy role shared by the ring kernels: a few CTAs of the attention kernel (or a stand-alone launch)
// pull K/V blocks from their owners' arenas into this GPU's position-ordered buffer with plain
// 16-byte peer loads, chunk by chunk, and bump ready[chunk] once per CTA when a chunk has landed, so
// consumers (the TMA loader warps of the compute CTAs) can start on a chunk as soon as all copy CTAs
// have finished it: they wait for ready[chunk] >= calls_so_far * n_copy_ctas.
#pragma once
#include "common.cuh"

namespace cpb {

struct CopySeg {
  const uint4* src;     // peer (or local) source
  uint4* dst;           // local destination
  long n16;             // 16-byte vectors
  int chunk;            // readiness counter to bump when every segment of this chunk is done
  int pad;
};

__device__ __forceinline__ void ring_copy_arrive(int* ready, int chunk) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(ready + chunk, 1);
  }
}

__device__ __forceinline__ void ring_copy_cta(const CopySeg* __restrict__ segs, int n_segs, int n_ctas, int cta, int* ready) {
  int cur = -1;
  for (int s = 0; s < n_segs; ++s) {
    const CopySeg seg = segs[s];
    if (seg.chunk != cur) {
      if (cur >= 0) ring_copy_arrive(ready, cur);
      cur = seg.chunk;
    }
    const long stride = (long)n_ctas * blockDim.x;
    // eight independent peer loads in flight per thread (the tail of a segment included) before the first store
    constexpr int U = 8;
    for (long i = (long)cta * blockDim.x + threadIdx.x; i < seg.n16; i += U * stride) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i + u * stride < seg.n16) v[u] = seg.src[i + u * stride];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i + u * stride < seg.n16) seg.dst[i + u * stride] = v[u];
    }
  }
  if (cur >= 0) ring_copy_arrive(ready, cur);
}

}  // namespace cpb
