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
    long i = (long)cta * blockDim.x + threadIdx.x;
    // four independent loads in flight per thread
    for (; i + 3 * stride < seg.n16; i += 4 * stride) {
      const uint4 a = seg.src[i], b = seg.src[i + stride], c = seg.src[i + 2 * stride], d = seg.src[i + 3 * stride];
      seg.dst[i] = a; seg.dst[i + stride] = b; seg.dst[i + 2 * stride] = c; seg.dst[i + 3 * stride] = d;
    }
    for (; i < seg.n16; i += stride) seg.dst[i] = seg.src[i];
  }
  if (cur >= 0) ring_copy_arrive(ready, cur);
}

}  // namespace cpb
