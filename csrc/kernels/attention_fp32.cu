// fp32-accurate attention for parity runs (ATTN_FP32=1): plain CUDA-core arithmetic, exact expf, no bf16 rounding of
// the probabilities, fp32 outputs and gradients.  One warp per query row; the lanes own head_dim/32 consecutive
// dimensions each, every score is a warp-wide dot product, the softmax is the online form, and masking uses the same
// global-position rule as the tensor-core kernels (query position q_pos[i], key position k_off + j).
// It is a measuring stick, not a fast path: the reference keeps a scalar fp32 kernel for the same purpose
// (context_parallel/AttentionForward.cu:126-376, selected by ATTN_FP32 in context_parallel/FusedSDPAOp.h:134-163).
//
// Layouts as in attention_fwd.cu: q [B,Tq,Hq,D], k/v [B,Tk,Hkv,D] bf16 with element strides (head, token, batch);
// out / dq / dk / dv fp32 contiguous [B,T,H,D]; lse [B,Hq,Tq] natural log.
#include "common.cuh"
#include "host_utils.h"

namespace cpb {

struct Fp32Params {
  const __nv_bfloat16 *q, *k, *v;
  int B, Tq, Tk, Hq, Hkv, causal, k_off;
  long q_sh, q_st, q_sb, k_sh, k_st, k_sb;
  float scale;
  const int* q_pos;
};

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int D>
__global__ void attn_fp32_fwd_kernel(Fp32Params p, float* __restrict__ out, float* __restrict__ lse) {
  constexpr int E = D / 32;
  const int lane = threadIdx.x & 31;
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= (long)p.B * p.Hq * p.Tq) return;
  const int i = (int)(row % p.Tq), h = (int)((row / p.Tq) % p.Hq), b = (int)(row / ((long)p.Tq * p.Hq));
  const int hk = h / (p.Hq / p.Hkv);
  const int qpos = p.q_pos ? p.q_pos[i] : i;
  const int jmax = p.causal ? min(p.Tk - 1, qpos - p.k_off) : p.Tk - 1;
  float qv[E], acc[E];
  const __nv_bfloat16* qr = p.q + b * p.q_sb + (long)i * p.q_st + h * p.q_sh + lane * E;
#pragma unroll
  for (int e = 0; e < E; ++e) { qv[e] = __bfloat162float(qr[e]); acc[e] = 0.f; }
  float m = -INFINITY, l = 0.f;
  for (int j = 0; j <= jmax; ++j) {
    const __nv_bfloat16* kr = p.k + b * p.k_sb + (long)j * p.k_st + hk * p.k_sh + lane * E;
    const __nv_bfloat16* vr = p.v + b * p.k_sb + (long)j * p.k_st + hk * p.k_sh + lane * E;
    float d = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) d += qv[e] * __bfloat162float(kr[e]);
    const float s = warp_sum_f(d) * p.scale;
    const float mn = fmaxf(m, s);
    const float alpha = expf(m - mn), pj = expf(s - mn);       // expf(-inf) = 0 on the first key
    l = l * alpha + pj;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = acc[e] * alpha + pj * __bfloat162float(vr[e]);
    m = mn;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  float* o = out + (((long)b * p.Tq + i) * p.Hq + h) * D + lane * E;
#pragma unroll
  for (int e = 0; e < E; ++e) o[e] = acc[e] * inv;
  if (lane == 0) lse[((long)b * p.Hq + h) * p.Tq + i] = l > 0.f ? m + logf(l) : -INFINITY;
}

// dq written, dk/dv accumulated with fp32 atomics (the caller zeroes them).
template <int D>
__global__ void attn_fp32_bwd_kernel(Fp32Params p, const float* __restrict__ out, const float* __restrict__ lse,
                                     const float* __restrict__ dout, float* __restrict__ dq, float* __restrict__ dk,
                                     float* __restrict__ dv) {
  constexpr int E = D / 32;
  const int lane = threadIdx.x & 31;
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= (long)p.B * p.Hq * p.Tq) return;
  const int i = (int)(row % p.Tq), h = (int)((row / p.Tq) % p.Hq), b = (int)(row / ((long)p.Tq * p.Hq));
  const int hk = h / (p.Hq / p.Hkv);
  const int qpos = p.q_pos ? p.q_pos[i] : i;
  const int jmax = p.causal ? min(p.Tk - 1, qpos - p.k_off) : p.Tk - 1;
  const long orow = (((long)b * p.Tq + i) * p.Hq + h) * D + lane * E;
  float qv[E], dov[E], dqv[E];
  const __nv_bfloat16* qr = p.q + b * p.q_sb + (long)i * p.q_st + h * p.q_sh + lane * E;
  float dsum = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    qv[e] = __bfloat162float(qr[e]); dov[e] = dout[orow + e]; dqv[e] = 0.f;
    dsum += dov[e] * out[orow + e];
  }
  const float delta = warp_sum_f(dsum);
  const float L = lse[((long)b * p.Hq + h) * p.Tq + i];
  for (int j = 0; j <= jmax; ++j) {
    const long koff = b * p.k_sb + (long)j * p.k_st + hk * p.k_sh + lane * E;
    float kv[E], vv[E], d = 0.f, dp = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      kv[e] = __bfloat162float(p.k[koff + e]); vv[e] = __bfloat162float(p.v[koff + e]);
      d += qv[e] * kv[e]; dp += dov[e] * vv[e];
    }
    const float s = warp_sum_f(d) * p.scale;
    const float pj = expf(s - L);
    const float ds = pj * (warp_sum_f(dp) - delta) * p.scale;
    float* dkr = dk + (((long)b * p.Tk + j) * p.Hkv + hk) * D + lane * E;
    float* dvr = dv + (((long)b * p.Tk + j) * p.Hkv + hk) * D + lane * E;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      dqv[e] += ds * kv[e];
      atomicAdd(dkr + e, ds * qv[e]);
      atomicAdd(dvr + e, pj * dov[e]);
    }
  }
#pragma unroll
  for (int e = 0; e < E; ++e) dq[orow + e] = dqv[e];
}

static int fill(Fp32Params& p, const void* q, const void* k, const void* v, int B, int Tq, int Tk, int Hq, int Hkv, int D, long q_sh,
                long q_st, long q_sb, long k_sh, long k_st, long k_sb, float scale, int causal, int k_off, const int* q_pos) {
  if (D != 32 && D != 64 && D != 128) return set_error(CPB_ERR_ARG, "attn_fp32: head_dim %d not in {32,64,128}", D);
  if (Hq % Hkv || B <= 0 || Tq <= 0 || Tk <= 0) return set_error(CPB_ERR_ARG, "attn_fp32: bad shape");
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.k_off = k_off;
  p.q_sh = q_sh; p.q_st = q_st; p.q_sb = q_sb; p.k_sh = k_sh; p.k_st = k_st; p.k_sb = k_sb; p.scale = scale; p.q_pos = q_pos;
  return CPB_OK;
}

}  // namespace cpb

using namespace cpb;

extern "C" int cpb_attn_fp32_fwd(const void* q, const void* k, const void* v, float* out, float* lse, int B, int Tq, int Tk,
                                 int Hq, int Hkv, int D, long q_sh, long q_st, long q_sb, long k_sh, long k_st, long k_sb,
                                 float scale, int causal, int k_off, const int* q_pos, cudaStream_t stream) {
  Fp32Params p;
  int rc = fill(p, q, k, v, B, Tq, Tk, Hq, Hkv, D, q_sh, q_st, q_sb, k_sh, k_st, k_sb, scale, causal, k_off, q_pos);
  if (rc) return rc;
  const long rows = (long)B * Hq * Tq;
  const int grid = (int)((rows + 3) / 4);
  if (D == 32) attn_fp32_fwd_kernel<32><<<grid, 128, 0, stream>>>(p, out, lse);
  else if (D == 64) attn_fp32_fwd_kernel<64><<<grid, 128, 0, stream>>>(p, out, lse);
  else attn_fp32_fwd_kernel<128><<<grid, 128, 0, stream>>>(p, out, lse);
  return check_launch("attn_fp32_fwd");
}

extern "C" int cpb_attn_fp32_bwd(const void* q, const void* k, const void* v, const float* out, const float* lse,
                                 const float* dout, float* dq, float* dk, float* dv, int B, int Tq, int Tk, int Hq, int Hkv,
                                 int D, long q_sh, long q_st, long q_sb, long k_sh, long k_st, long k_sb, float scale,
                                 int causal, int k_off, const int* q_pos, cudaStream_t stream) {
  Fp32Params p;
  int rc = fill(p, q, k, v, B, Tq, Tk, Hq, Hkv, D, q_sh, q_st, q_sb, k_sh, k_st, k_sb, scale, causal, k_off, q_pos);
  if (rc) return rc;
  const long rows = (long)B * Hq * Tq;
  const int grid = (int)((rows + 3) / 4);
  if (D == 32) attn_fp32_bwd_kernel<32><<<grid, 128, 0, stream>>>(p, out, lse, dout, dq, dk, dv);
  else if (D == 64) attn_fp32_bwd_kernel<64><<<grid, 128, 0, stream>>>(p, out, lse, dout, dq, dk, dv);
  else attn_fp32_bwd_kernel<128><<<grid, 128, 0, stream>>>(p, out, lse, dout, dq, dk, dv);
  return check_launch("attn_fp32_bwd");
}
