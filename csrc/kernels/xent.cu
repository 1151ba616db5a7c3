// Softmax cross-entropy over a chunk of fp32 logits, forward and backward in one launch.
//
// The language-model head never materialises [tokens, vocab] for the whole sequence: the host loops
// over row chunks, runs the lm_head GEMM into an fp32 chunk buffer, and this kernel turns the chunk
// into per-row losses and bf16 dlogits = (softmax - onehot) * grad_scale in place of a separate
// backward pass; two more GEMMs then produce dX and accumulate dW.  Replaces the reference's
// materialised logits + sparse_cross_entropy_loss (Scripts/Blutrain/bluscriptCP.cpp:452-459,1712).
//
// One CTA per row: pass 1 computes max and sum(exp) online, pass 2 re-reads the row (L2 resident) and
// writes dlogits.  Rows whose target is negative are ignored (zero gradient, no loss).
#include "common.cuh"
#include "host_utils.h"

namespace cpb {

__global__ void __launch_bounds__(512)
xent_kernel(const float* __restrict__ logits, const int64_t* __restrict__ targets, __nv_bfloat16* __restrict__ dlogits,
            float* __restrict__ loss_sum, float* __restrict__ row_loss, int rows, int V, int Vcols, long ld_logits, long ld_dlogits,
            float grad_scale, int* status) {
  __shared__ float red_m[16], red_s[16];
  __shared__ float s_max, s_sum;
  const int row = blockIdx.x;
  if (row >= rows) return;
  const float* x = logits + (size_t)row * ld_logits;
  const int64_t tgt = targets[row];
  if (tgt >= V) report(status, ST_BAD_INDEX, 1200, (int)tgt);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float m = -INFINITY, s = 0.f;
  const int V4 = V >> 2;
  for (int i = threadIdx.x; i < V4; i += blockDim.x) {
    const float4 v = ((const float4*)x)[i];
    const float mx = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
    if (mx > m) { s *= __expf(m - mx); m = mx; }
    s += __expf(v.x - m) + __expf(v.y - m) + __expf(v.z - m) + __expf(v.w - m);
  }
  for (int i = (V4 << 2) + threadIdx.x; i < V; i += blockDim.x) {
    const float v = x[i];
    if (v > m) { s *= __expf(m - v); m = v; }
    s += __expf(v - m);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mn));
    m = mn;
  }
  if (lane == 0) { red_m[warp] = m; red_s[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    m = lane < nw ? red_m[lane] : -INFINITY;
    s = lane < nw ? red_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      const float mn = fmaxf(m, m2);
      s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mn));
      m = mn;
    }
    if (lane == 0) { s_max = m; s_sum = s; }
  }
  __syncthreads();
  m = s_max; s = s_sum;
  const bool ignore = tgt < 0 || tgt >= V;
  if (threadIdx.x == 0) {
    const float l = ignore ? 0.f : (m + __logf(s) - x[tgt]);
    if (row_loss) row_loss[row] = l;
    if (loss_sum && !ignore) atomicAdd(loss_sum, l);
  }
  if (dlogits == nullptr) return;
  __nv_bfloat16* d = dlogits + (size_t)row * ld_dlogits;
  const float inv = ignore ? 0.f : grad_scale / s;
  const int VC4 = Vcols >> 2;       // Vcols (>= V, multiple of 4): padded width; padding columns get zero gradient
  for (int i = threadIdx.x; i < VC4; i += blockDim.x) {
    const float4 v = ((const float4*)x)[i];
    const int c = i << 2;
    float p0 = c < V ? __expf(v.x - m) * inv : 0.f, p1 = c + 1 < V ? __expf(v.y - m) * inv : 0.f;
    float p2 = c + 2 < V ? __expf(v.z - m) * inv : 0.f, p3 = c + 3 < V ? __expf(v.w - m) * inv : 0.f;
    if (!ignore && tgt >= c && tgt < c + 4) {
      if (tgt == c) p0 -= grad_scale; else if (tgt == c + 1) p1 -= grad_scale; else if (tgt == c + 2) p2 -= grad_scale; else p3 -= grad_scale;
    }
    *(uint2*)(d + c) = make_uint2(pack_bf16(p0, p1), pack_bf16(p2, p3));
  }
}

}  // namespace cpb

using namespace cpb;

// logits fp32 [rows, Vcols] (row stride ld_logits, multiple of 4) of which the first V columns are real vocabulary;
// dlogits bf16 [rows, Vcols] (row stride multiple of 4) or null; loss_sum (fp32 scalar, +=) and row_loss [rows] optional.
extern "C" int cpb_xent(const float* logits, const int64_t* targets, void* dlogits, float* loss_sum, float* row_loss,
                        int rows, int V, int Vcols, long ld_logits, long ld_dlogits, float grad_scale, int* status, cudaStream_t stream) {
  if (rows <= 0) return CPB_OK;
  if (Vcols < V || (Vcols % 4)) return set_error(CPB_ERR_ARG, "xent: Vcols must be >= V and a multiple of 4");
  if ((ld_logits % 4) || (dlogits && (ld_dlogits % 4))) return set_error(CPB_ERR_ARG, "xent: row strides must be multiples of 4");
  xent_kernel<<<rows, 512, 0, stream>>>(logits, targets, (__nv_bfloat16*)dlogits, loss_sum, row_loss, rows, V, Vcols, ld_logits, ld_dlogits, grad_scale, status);
  return check_launch("xent");
}
