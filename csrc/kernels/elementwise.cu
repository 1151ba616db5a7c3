// Memory-bound kernels: RMSNorm / LayerNorm (with fused residual add), SwiGLU / GELU backward,
// bias gradient, embedding, QK-norm + RoPE on a packed QKV buffer, RoPE cache builders
// (YaRN / LongRoPE), HeadTail gather, K/V pack, LSE merge, gradient-norm + AdamW.
//
// They replace the reference's external tensor-library kernels (rms_norm, layer_norm, gelu,
// swiglu, embedding, rope_forward_cuda, AdamW, clip_grad_norm_) and its own headtail / kv-pack
// kernels (context_parallel/headtail_kernel.cu:26-105, context_parallel/KVPackKernel.cu:13-37),
// and fold the SDPA merge (context_parallel/SDPAMerger.h:108-121) into one launch.
// Everything is bf16 in / bf16 out with fp32 statistics, 16-byte vector accesses, one warp per row
// for the row reductions.
#include "common.cuh"
#include "host_utils.h"

namespace cpb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  f[0] = bf16_lo(u.x); f[1] = bf16_hi(u.x); f[2] = bf16_lo(u.y); f[3] = bf16_hi(u.y);
  f[4] = bf16_lo(u.z); f[5] = bf16_hi(u.z); f[6] = bf16_lo(u.w); f[7] = bf16_hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}

// eight consecutive fp32 parameters (vector c of a row) as two 16-byte loads; `fill` when the parameter is absent
__device__ __forceinline__ void load8f(const float* __restrict__ p, int c, float fill, float (&f)[8]) {
  if (p == nullptr) {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = fill;
    return;
  }
  const float4 a = __ldg((const float4*)p + 2 * c), b = __ldg((const float4*)p + 2 * c + 1);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// ============================================================================ norm forward
// One warp per row; d % 8 == 0; MAXV = max 16-byte vectors per lane (d <= 256*MAXV).
// If `res` != null: x_new = x + res is written to `xout` and normalised.
// LAYER = true -> LayerNorm (mean/var, optional bias); false -> RMSNorm.
template <bool LAYER, int MAXV>
__global__ void norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                const float* __restrict__ w, const float* __restrict__ b,
                                __nv_bfloat16* __restrict__ xout, __nv_bfloat16* __restrict__ y,
                                float* __restrict__ stats, int rows, int d, float eps) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int nvec = d >> 3;
  const uint4* xr = (const uint4*)(x + (size_t)row * d);
  const uint4* rr = res ? (const uint4*)(res + (size_t)row * d) : nullptr;
  // every load of the row is issued before the first use; the row then stays in registers as bf16 (the rounded x + res,
  // exactly what later kernels re-read)
  uint4 px[MAXV], pr[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + i * 32;
    if (c < nvec) {
      px[i] = xr[c];
      if (rr) pr[i] = rr[c];
    }
  }
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + i * 32;
    if (c < nvec) {
      float v[8];
      unpack8(px[i], v);
      if (rr) {
        float r8[8];
        unpack8(pr[i], r8);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] += r8[j];
        px[i] = pack8(v);
        ((uint4*)(xout + (size_t)row * d))[c] = px[i];
        unpack8(px[i], v);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s += v[j]; ss += v[j] * v[j]; }
    }
  }
  s = warp_sum(s); ss = warp_sum(ss);
  float mean = 0.f, rstd;
  if (LAYER) {
    mean = s / d;
    float var = fmaxf(ss / d - mean * mean, 0.f);
    rstd = rsqrtf(var + eps);
  } else {
    rstd = rsqrtf(ss / d + eps);
  }
  if (stats && lane == 0) { stats[2 * (size_t)row] = mean; stats[2 * (size_t)row + 1] = rstd; }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + i * 32;
    if (c < nvec) {
      float v[8], o[8], g[8], bb[8];
      unpack8(px[i], v);
      load8f(w, c, 1.f, g);
      if (LAYER) load8f(b, c, 0.f, bb);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[j] - mean) * rstd * g[j] + (LAYER ? bb[j] : 0.f);
      ((uint4*)(y + (size_t)row * d))[c] = pack8(o);
    }
  }
}

// ============================================================================ norm backward
// dx = rstd * (g*dy - xhat * mean(g*dy*xhat) [- mean(g*dy)])  (+ dres_in) ; dw += sum dy*xhat ; db += sum dy
// Each block handles `rows_per_block` rows with one warp per row in a loop and reduces dw/db through
// shared memory before one atomicAdd per column per block.
template <bool LAYER, int MAXV>
__global__ void __launch_bounds__(256, 2)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                const __nv_bfloat16* __restrict__ dres, const float* __restrict__ w,
                const float* __restrict__ stats, __nv_bfloat16* __restrict__ dx,
                float* __restrict__ dw, float* __restrict__ db, int rows, int d, int rows_per_block) {
  extern __shared__ float sm[];          // [2][d]: the block's partial dw, db
  float* sdw = sm;
  float* sdb = sm + d;
  for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) sm[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int nvec = d >> 3;
  const int rot = lane >> 2;             // shared-memory adds start at element `rot` of every vector: conflict-free banks
  const int r0 = blockIdx.x * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  for (int row = r0 + warp; row < r1; row += nwarps) {
    const float mean = LAYER ? stats[2 * (size_t)row] : 0.f;
    const float rstd = stats[2 * (size_t)row + 1];
    // the row stays in registers as it was loaded (bf16, 4 registers per 8 elements); every load is issued before the
    // first use, and the weight-gradient partials go to shared memory row by row, so that two blocks fit on an SM and
    // enough bytes are in flight to cover the memory latency
    uint4 px[MAXV], pd[MAXV], pr[MAXV];
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        px[i] = ((const uint4*)(x + (size_t)row * d))[c];
        pd[i] = ((const uint4*)(dy + (size_t)row * d))[c];
        if (dres) pr[i] = ((const uint4*)(dres + (size_t)row * d))[c];
      }
    }
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float xv[8], dv[8], wv[8];
        unpack8(px[i], xv); unpack8(pd[i], dv);
        load8f(w, c, 1.f, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd, g = dv[j] * wv[j];
          s1 += g * xh;
          s2 += g;
          xv[j] = dv[j] * xh;
        }
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int j = (jj + rot) & 7;
          if (dw) atomicAdd(&sdw[c * 8 + j], xv[j]);
          if (LAYER && db) atomicAdd(&sdb[c * 8 + j], dv[j]);
        }
      }
    }
    s1 = warp_sum(s1) / d;
    s2 = LAYER ? warp_sum(s2) / d : 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float xv[8], dv[8], wv[8], r8[8], o[8];
        unpack8(px[i], xv); unpack8(pd[i], dv);
        load8f(w, c, 1.f, wv);
        if (dres) unpack8(pr[i], r8);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd, g = dv[j] * wv[j];
          o[j] = rstd * (g - xh * s1 - s2);
          if (dres) o[j] += r8[j];
        }
        ((uint4*)(dx + (size_t)row * d))[c] = pack8(o);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    if (dw) atomicAdd(&dw[i], sdw[i]);
    if (LAYER && db) atomicAdd(&db[i], sdb[i]);
  }
}

// ============================================================================ activations (backward)
// gu: [rows, 2F] = [gate | up]; dact: [rows, F]; dgu: [rows, 2F]
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* __restrict__ dgu, size_t rows, int F) {
  const size_t nvec = rows * (size_t)(F >> 3);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / (F >> 3);
    const int c = (int)(i % (F >> 3)) * 8;
    float g[8], u[8], da[8], dg[8], du[8];
    uint4 ug = *(const uint4*)(gu + row * 2 * F + c);
    uint4 uu = *(const uint4*)(gu + row * 2 * F + F + c);
    uint4 ud = *(const uint4*)(dact + row * F + c);
    unpack8(ug, g); unpack8(uu, u); unpack8(ud, da);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float s = 1.f / (1.f + __expf(-g[j]));
      float silu = g[j] * s;
      dg[j] = da[j] * u[j] * (s + silu * (1.f - s));
      du[j] = da[j] * silu;
    }
    *(uint4*)(dgu + row * 2 * F + c) = pack8(dg);
    *(uint4*)(dgu + row * 2 * F + F + c) = pack8(du);
  }
}

// forward (standalone, used when the GEMM epilogue fusion is not): act = silu(g)*u
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, size_t rows, int F) {
  const size_t nvec = rows * (size_t)(F >> 3);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / (F >> 3);
    const int c = (int)(i % (F >> 3)) * 8;
    float g[8], u[8], o[8];
    uint4 ug = *(const uint4*)(gu + row * 2 * F + c);
    uint4 uu = *(const uint4*)(gu + row * 2 * F + F + c);
    unpack8(ug, g); unpack8(uu, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    *(uint4*)(act + row * F + c) = pack8(o);
  }
}

__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  float e = __expf(2.f * u);
  float t = 1.f - 2.f / (e + 1.f);
  float du = k0 * (1.f + 3.f * k1 * x * x);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}
__device__ __forceinline__ float gelu_tanh_val(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  float e = __expf(2.f * u);
  float t = 1.f - 2.f / (e + 1.f);
  return 0.5f * x * (1.f + t);
}
// mode 0: y = gelu(x) ; mode 1: y = dy * gelu'(x)
__global__ void gelu_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                            __nv_bfloat16* __restrict__ y, size_t n8, int mode) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float xv[8], o[8];
    uint4 ux = ((const uint4*)x)[i];
    unpack8(ux, xv);
    if (mode == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = gelu_tanh_val(xv[j]);
    } else {
      float dv[8];
      uint4 ud = ((const uint4*)dy)[i];
      unpack8(ud, dv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = dv[j] * gelu_tanh_grad(xv[j]);
    }
    ((uint4*)y)[i] = pack8(o);
  }
}

// y = a + b (bf16), 8 elements per thread
__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ y, size_t n8) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float av[8], bv[8];
    uint4 ua = ((const uint4*)a)[i], ub = ((const uint4*)b)[i];
    unpack8(ua, av); unpack8(ub, bv);
#pragma unroll
    for (int j = 0; j < 8; ++j) av[j] += bv[j];
    ((uint4*)y)[i] = pack8(av);
  }
}

// db[n] += sum_rows dy[row, n]; grid (ceil(N/64), row_blocks); block 256 = 8 row-lanes x 32 col-pairs
__global__ void bias_grad_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ db, int rows, int N, int rows_per_block) {
  __shared__ float red[8][64];
  const int cp = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int col = blockIdx.x * 64 + cp * 2;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float a0 = 0.f, a1 = 0.f;
  if (col < N) {
    for (int r = r0 + rl; r < r1; r += 8) {
      uint32_t u = *(const uint32_t*)(dy + (size_t)r * N + col);
      a0 += bf16_lo(u); a1 += bf16_hi(u);
    }
  }
  red[rl][cp * 2] = a0; red[rl][cp * 2 + 1] = a1;
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += red[i][threadIdx.x];
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (c < N) atomicAdd(&db[c], s);
  }
}

// ============================================================================ embedding
// out[row, :] = wte[idx[row], :] (+ wpe[pos[row], :])
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ idx, const int64_t* __restrict__ pos,
                                     const __nv_bfloat16* __restrict__ wte, const __nv_bfloat16* __restrict__ wpe,
                                     __nv_bfloat16* __restrict__ out, size_t rows, int d, int pos_period) {
  const int nvec = d >> 3;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < rows * nvec; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / nvec;
    const int c = (int)(i % nvec);
    uint4 u = ((const uint4*)(wte + (size_t)idx[row] * d))[c];
    if (wpe) {
      float a[8], b[8];
      uint4 up = ((const uint4*)(wpe + (size_t)pos[row % pos_period] * d))[c];
      unpack8(u, a); unpack8(up, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
      u = pack8(a);
    }
    ((uint4*)(out + row * d))[c] = u;
  }
}
// dwte[idx[row], :] += dout[row, :] ; dwpe[pos[row], :] += dout[row, :]   (fp32 atomics)
__global__ void embedding_bwd_kernel(const int64_t* __restrict__ idx, const int64_t* __restrict__ pos,
                                     const __nv_bfloat16* __restrict__ dout, float* __restrict__ dwte,
                                     float* __restrict__ dwpe, size_t rows, int d, int pos_period) {
  const int nvec = d >> 3;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < rows * nvec; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / nvec;
    const int c = (int)(i % nvec) * 8;
    float g[8];
    uint4 u = *(const uint4*)(dout + row * d + c);
    unpack8(u, g);
    float* wt = dwte + (size_t)idx[row] * d + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(wt + j, g[j]);
    if (dwpe) {
      float* wp = dwpe + (size_t)pos[row % pos_period] * d + c;
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(wp + j, g[j]);
    }
  }
}

// ============================================================================ QK-norm + RoPE
// Packed QKV [rows = B*T, (Hq + 2*Hkv) * D] bf16.  For every q and k head vector: optional RMS-norm with gain
// gamma_q / gamma_k, then NeoX rotation by cache row pos[t] (element e pairs with e + D/2); v is copied.
// A head vector is handled by D/8 adjacent lanes, each holding 8 consecutive elements (one 16-byte access), so a warp
// covers 4 (D = 64) or 2 (D = 128) vectors at a time; the lanes of the first half of the vector exchange values with
// the lanes of the second half by shuffle, and the sum of squares is reduced inside the lane group.
// Output: out (same packed shape, may alias in).  rstd (optional) [rows, Hq+Hkv] fp32.
template <int D>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = D / 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void load8_f32(const float* p, float (&v)[8]) {
  const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// One warp per token row: the row's cos / sin values (this lane's 8 positions inside a half) and its position are
// loaded once and reused for every q and k head of the row; without that reuse each head re-reads its 2 * D floats of the
// cache row, as many bytes as the packed QKV itself.  The heads of the row are swept 32 * 8 / D at a time, U sweeps' loads
// issued before the first use.
template <int D>
__global__ void __launch_bounds__(256, 3) qk_norm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                        const float* __restrict__ gq, const float* __restrict__ gk,
                                        const float* __restrict__ cache, const int64_t* __restrict__ pos,
                                        float* __restrict__ rstd, size_t rows, int T, int Hq, int Hkv, float eps,
                                        int cache_len, int* status) {
  constexpr int GL = D / 8, VPW = 32 / GL, half = D / 2, U = 4;
  const int H = Hq + 2 * Hkv;
  const int lane = threadIdx.x & 31;
  const int gl = lane % GL;                         // lane inside its vector's group
  const int hv = lane / GL;                         // which of the VPW heads of a sweep this lane works on
  const bool second = gl >= GL / 2;                 // this lane holds elements of the second half
  const int e0 = gl * 8;                            // first element this lane holds
  const int eh = (gl % (GL / 2)) * 8;               // the same position inside a half (index into cos / sin)
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  float gqv[8], gkv[8];
  if (gq) load8_f32(gq + e0, gqv);
  if (gk) load8_f32(gk + e0, gkv);
  for (size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
    float c[8], sn[8];
    bool have_cs = false;
    if (cache) {
      const int64_t p = pos[row % T];
      if (p >= 0 && p < cache_len) {
        const float* cr = cache + (size_t)p * D;
        load8_f32(cr + eh, c); load8_f32(cr + half + eh, sn);
        have_cs = true;
      } else {
        report(status, ST_BAD_INDEX, 400, (int)p);
      }
    }
    const __nv_bfloat16* irow = in + row * (size_t)H * D;
    __nv_bfloat16* orow = out + row * (size_t)H * D;
    for (int h0 = 0; h0 < H; h0 += VPW * U) {
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int h = h0 + u * VPW + hv;
        raw[u] = h < H ? *(const uint4*)(irow + (size_t)h * D + e0) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int h = h0 + u * VPW + hv;
        const bool live = h < H;
        const bool rot = live && h < Hq + Hkv;          // uniform inside a lane group
        const bool isq = h < Hq;
        float x[8];
        unpack8(raw[u], x);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
        ss = group_sum<D>(ss);
        if (rot && (isq ? gq != nullptr : gk != nullptr)) {
          const float r = rsqrtf(ss / D + eps);
          if (rstd && gl == 0) rstd[row * (size_t)(Hq + Hkv) + h] = r;
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] = x[i] * r * (isq ? gqv[i] : gkv[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float other = __shfl_xor_sync(0xffffffffu, x[i], GL / 2);      // the paired element of the other half
          if (rot && have_cs) x[i] = second ? other * sn[i] + x[i] * c[i] : x[i] * c[i] - other * sn[i];
        }
        if (live) *(uint4*)(orow + (size_t)h * D + e0) = pack8(x);
      }
    }
  }
}

// Backward of the above on the packed gradient: din = d(in); dgq / dgk (fp32, +=) accumulate the gain gradients.
// `in` is the ORIGINAL (pre-norm, pre-rotation) packed QKV.  Same row-per-warp sweep as the forward kernel.
template <int D>
__global__ void __launch_bounds__(256, 2) qk_norm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ dout,
                                        __nv_bfloat16* __restrict__ din, const float* __restrict__ gq,
                                        const float* __restrict__ gk, const float* __restrict__ cache,
                                        const int64_t* __restrict__ pos, float* __restrict__ dgq, float* __restrict__ dgk,
                                        size_t rows, int T, int Hq, int Hkv, float eps, int cache_len) {
  constexpr int GL = D / 8, VPW = 32 / GL, half = D / 2, U = 2;
  __shared__ float sg[2][D];
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) (&sg[0][0])[i] = 0.f;
  __syncthreads();
  const int H = Hq + 2 * Hkv;
  const int lane = threadIdx.x & 31;
  const int gl = lane % GL, hv = lane / GL;
  const bool second = gl >= GL / 2;
  const int e0 = gl * 8, eh = (gl % (GL / 2)) * 8;
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  float accq[8], acck[8], gqv[8], gkv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) accq[i] = acck[i] = 0.f;
  if (gq) load8_f32(gq + e0, gqv);
  if (gk) load8_f32(gk + e0, gkv);
  for (size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
    float c[8], sn[8];
    bool have_cs = false;
    if (cache) {
      const int64_t p = pos[row % T];
      if (p >= 0 && p < cache_len) {
        const float* cr = cache + (size_t)p * D;
        load8_f32(cr + eh, c); load8_f32(cr + half + eh, sn);
        have_cs = true;
      }
    }
    const size_t rbase = row * (size_t)H * D;
    for (int h0 = 0; h0 < H; h0 += VPW * U) {
      uint4 rawd[U], rawx[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int h = h0 + u * VPW + hv;
        const bool live = h < H;
        const bool normed = live && h < Hq + Hkv && (h < Hq ? gq != nullptr : gk != nullptr);
        rawd[u] = live ? *(const uint4*)(dout + rbase + (size_t)h * D + e0) : make_uint4(0, 0, 0, 0);
        rawx[u] = normed ? *(const uint4*)(in + rbase + (size_t)h * D + e0) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int h = h0 + u * VPW + hv;
        const bool live = h < H;
        const bool rot = live && h < Hq + Hkv;
        const bool isq = h < Hq;
        const bool normed = rot && (isq ? gq != nullptr : gk != nullptr);
        float d[8], xh[8];
        unpack8(rawd[u], d);
        unpack8(rawx[u], xh);
        // every shuffle below is executed by the whole warp: lane groups of one warp may hold different kinds of heads
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float other = __shfl_xor_sync(0xffffffffu, d[i], GL / 2);
          if (rot && have_cs) d[i] = second ? d[i] * c[i] - other * sn[i] : d[i] * c[i] + other * sn[i];   // transpose of the rotation
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += xh[i] * xh[i];
        ss = group_sum<D>(ss);
        const float r = rsqrtf(ss / D + eps);
        float dot = 0.f;
        if (normed) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            xh[i] *= r;
            if (isq) accq[i] += d[i] * xh[i]; else acck[i] += d[i] * xh[i];
            d[i] *= isq ? gqv[i] : gkv[i];
            dot += d[i] * xh[i];
          }
        }
        dot = group_sum<D>(dot) / D;
        if (normed) {
#pragma unroll
          for (int i = 0; i < 8; ++i) d[i] = r * (d[i] - xh[i] * dot);
        }
        if (live) *(uint4*)(din + rbase + (size_t)h * D + e0) = pack8(d);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) { atomicAdd(&sg[0][e0 + i], accq[i]); atomicAdd(&sg[1][e0 + i], acck[i]); }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    if (dgq) atomicAdd(&dgq[i], sg[0][i]);
    if (dgk) atomicAdd(&dgk[i], sg[1][i]);
  }
}

// ============================================================================ RoPE caches
// cache[p, i] = cos(p * f_i) * m ; cache[p, i + half] = sin(p * f_i) * m, with f_i from `inv_freq` (YaRN:
// ramp-blended on the host; LongRoPE: base_freq, divided by lambda_i when p >= n_hat).
__global__ void rope_cache_kernel(float* __restrict__ cache, const float* __restrict__ inv_freq,
                                  const float* __restrict__ lambda, const int64_t* __restrict__ positions,
                                  int64_t seq_len, int half, int64_t n_hat, float mscale) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < (size_t)seq_len * half; i += (size_t)gridDim.x * blockDim.x) {
    const int64_t r = (int64_t)(i / half);
    const int d = (int)(i % half);
    const int64_t p = positions ? positions[r] : r;
    float f = inv_freq[d];
    float ang = (float)p * f;
    if (lambda && p >= n_hat) ang = (float)p * f / lambda[d];
    float s, c;
    sincosf(ang, &s, &c);
    cache[(size_t)r * 2 * half + d] = c * mscale;
    cache[(size_t)r * 2 * half + d + half] = s * mscale;
  }
}
// out[r, :] = cache[labels[r], :]   (CREAM / PoSE / RandPos relabelling)
__global__ void gather_rows_f32_kernel(const float* __restrict__ src, const int64_t* __restrict__ index,
                                       float* __restrict__ out, int64_t rows, int width, int64_t src_rows, int* status) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < (size_t)rows * width; i += (size_t)gridDim.x * blockDim.x) {
    const int64_t r = (int64_t)(i / width);
    const int64_t s = index[r];
    if (s < 0 || s >= src_rows) { report(status, ST_BAD_INDEX, 410, (int)s); continue; }
    out[i] = src[(size_t)s * width + (i % width)];
  }
}

// ============================================================================ sequence permutations
// Generic gather along the sequence axis of a [outer, T_src, inner_bytes] tensor:
//   out[o, j, :] = in[o, index[j], :]       (16-byte vectors when inner_bytes % 16 == 0)
// index = HeadTail permutation -> loadbalance; inverse -> unloadbalance; local positions -> shard.
template <typename V>
__global__ void gather_seq_kernel(const V* __restrict__ in, V* __restrict__ out, const int64_t* __restrict__ index,
                                  int64_t outer, int64_t t_src, int64_t t_dst, int64_t inner, int* status) {
  const size_t total = (size_t)outer * t_dst * inner;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int64_t c = (int64_t)(i % inner);
    const int64_t j = (int64_t)((i / inner) % t_dst);
    const int64_t o = (int64_t)(i / (inner * t_dst));
    const int64_t s = index[j];
    if (s < 0 || s >= t_src) { report(status, ST_BAD_INDEX, 420, (int)s); continue; }
    out[i] = in[((size_t)o * t_src + s) * inner + c];
  }
}

// K,V (strided [B,T,H,D] views) -> contiguous [2][B,T,H,D] buffer
__global__ void kv_pack_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                               __nv_bfloat16* __restrict__ out, size_t rows, int hd, size_t k_row_stride, size_t v_row_stride) {
  const int nvec = hd >> 3;
  const size_t total = rows * nvec;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < 2 * total; i += (size_t)gridDim.x * blockDim.x) {
    const int which = i >= total;
    const size_t j = which ? i - total : i;
    const size_t row = j / nvec;
    const int c = (int)(j % nvec);
    const __nv_bfloat16* src = which ? v + row * v_row_stride : k + row * k_row_stride;
    ((uint4*)(out + (size_t)which * rows * hd + row * hd))[c] = ((const uint4*)src)[c];
  }
}

// ============================================================================ LSE merge
// out, blk: [B,T,H,D] bf16 ; lse, blk_lse: [B,H,T] fp32.  Rows t in [t_begin, T) are merged (t_begin = T/2
// reproduces the reference's `partial` second-half update).  One warp per (b,t,h) row.
__global__ void lse_merge_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                                 const __nv_bfloat16* __restrict__ blk, const float* __restrict__ blk_lse,
                                 int B, int T, int H, int D, int t_begin, int blk_T, int blk_t_offset) {
  const int lane = threadIdx.x & 31;
  const size_t nrow = (size_t)B * (T - t_begin) * H;
  for (size_t w = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5); w < nrow; w += (size_t)gridDim.x * (blockDim.x >> 5)) {
    const int h = (int)(w % H);
    const int t = (int)((w / H) % (T - t_begin)) + t_begin;
    const int b = (int)(w / ((size_t)H * (T - t_begin)));
    const int tb = t - blk_t_offset;          // row inside the block result
    const float l0 = lse[((size_t)b * H + h) * T + t];
    const float l1 = blk_lse[((size_t)b * H + h) * blk_T + tb];
    float wgt, lnew;
    if (l1 == -INFINITY) { wgt = 0.f; lnew = l0; }
    else if (l0 == -INFINITY) { wgt = 1.f; lnew = l1; }
    else {
      const float dlt = l1 - l0;
      wgt = 1.f / (1.f + __expf(-dlt));
      const float mx = fmaxf(l0, l1);
      lnew = mx + log1pf(__expf(-fabsf(dlt)));
    }
    __nv_bfloat16* o = out + (((size_t)b * T + t) * H + h) * D;
    const __nv_bfloat16* s = blk + (((size_t)b * blk_T + tb) * H + h) * D;
    for (int e = lane; e < D; e += 32) {
      const float ov = __bfloat162float(o[e]), sv = __bfloat162float(s[e]);
      o[e] = __float2bfloat16(ov - wgt * (ov - sv));
    }
    if (lane == 0) lse[((size_t)b * H + h) * T + t] = lnew;
  }
}

// ============================================================================ optimiser
// partial[blockIdx.x] = sum g^2 over the block's grid-stride range ; the last block (ticket) folds the
// partials into out[0] = total sum of squares (not sqrt) so the next kernel can consume it.
__global__ void sumsq_kernel(const float* __restrict__ g, size_t n, float* __restrict__ partial,
                             unsigned int* __restrict__ ticket, float* __restrict__ out) {
  __shared__ float red[32];
  __shared__ bool last;
  float s = 0.f;
  const size_t n4 = n >> 2;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    float4 v = ((const float4*)g)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0)
    for (size_t i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x) s += g[i] * g[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) {
      partial[blockIdx.x] = t;
      __threadfence();
      last = (atomicAdd(ticket, 1u) == gridDim.x - 1);
    }
  }
  __syncthreads();
  if (last) {
    float t = 0.f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) t += ((volatile float*)partial)[i];
    t = warp_sum(t);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = t;
    __syncthreads();
    if (threadIdx.x < 32) {
      float u = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
      u = warp_sum(u);
      if (threadIdx.x == 0) { out[0] = u; *ticket = 0; }
    }
  }
}

// AdamW on flat fp32 master / moment buffers, writing the bf16 compute copy in the same pass.
//   gscale = grad_prescale * min(1, clip / (sqrt(sumsq)*grad_prescale + 1e-6))   (sumsq read on device, no host sync)
// If sumsq is not finite the step is skipped (NaN/Inf guard) and flag[0] is set.
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ p16, size_t n, float lr, float b1,
                             float b2, float eps, float wd, float bc1, float bc2, float grad_prescale, float clip,
                             const float* __restrict__ sumsq, int* __restrict__ flag) {
  float gs = grad_prescale;
  if (sumsq) {
    const float ssq = sumsq[0];
    if (!isfinite(ssq)) { if (flag && blockIdx.x == 0 && threadIdx.x == 0) flag[0] = 1; return; }
    const float norm = sqrtf(ssq) * grad_prescale;
    if (clip > 0.f) gs *= fminf(1.f, clip / (norm + 1e-6f));
  }
  const float inv_bc2_sqrt = rsqrtf(bc2);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float gi = g[i] * gs;
    float pi = p[i] * (1.f - lr * wd);
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    pi -= (lr / bc1) * mi / (sqrtf(vi) * inv_bc2_sqrt + eps);
    p[i] = pi; m[i] = mi; v[i] = vi;
    if (p16) p16[i] = __float2bfloat16(pi);
  }
}

// AdamW over this rank's shard of a sharded optimiser state.  master/m/v/g are shard-contiguous; every segment
// (blockIdx.y) maps a run of shard elements to the flat parameter index it updates, so the refreshed compute copy is
// written at its flat position: bf16 for matrices (decay != 0, flat index < n_decay) and fp32 for vectors.
struct AdamSeg {
  long shard_begin;     // first element inside the shard buffers
  long flat_begin;      // flat parameter index of that element
  long n;
  long decay;           // 1: weight decay applies and the compute copy is bf16; 0: no decay, fp32 copy
};
__global__ void adamw_sharded_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                     float* __restrict__ v, __nv_bfloat16* __restrict__ p16, float* __restrict__ p32,
                                     long n_decay, const AdamSeg* __restrict__ segs, float lr, float b1, float b2,
                                     float eps, float wd, float bc1, float bc2, float grad_prescale, float clip,
                                     const float* __restrict__ sumsq, int* __restrict__ flag) {
  float gs = grad_prescale;
  if (sumsq) {
    const float ssq = sumsq[0];
    if (!isfinite(ssq)) { if (flag && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) flag[0] = 1; return; }
    const float norm = sqrtf(ssq) * grad_prescale;
    if (clip > 0.f) gs *= fminf(1.f, clip / (norm + 1e-6f));
  }
  const AdamSeg sg = segs[blockIdx.y];
  const float decay = sg.decay ? (1.f - lr * wd) : 1.f;
  const float inv_bc2_sqrt = rsqrtf(bc2);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < sg.n; i += (long)gridDim.x * blockDim.x) {
    const long s = sg.shard_begin + i, f = sg.flat_begin + i;
    const float gi = g[s] * gs;
    float pi = p[s] * decay;
    const float mi = b1 * m[s] + (1.f - b1) * gi;
    const float vi = b2 * v[s] + (1.f - b2) * gi * gi;
    pi -= (lr / bc1) * mi / (sqrtf(vi) * inv_bc2_sqrt + eps);
    p[s] = pi; m[s] = mi; v[s] = vi;
    if (sg.decay) p16[f] = __float2bfloat16(pi);
    else p32[f - n_decay] = pi;
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n, float scale) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(in[i] * scale);
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, size_t n, float scale, int accumulate) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(in[i]) * scale;
    out[i] = accumulate ? out[i] + v : v;
  }
}

static inline int grid_for(size_t work, int block, int per_sm = 8) {
  size_t g = (work + block - 1) / block;
  size_t cap = (size_t)sm_count() * per_sm;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace cpb

using namespace cpb;

#define NORM_DISPATCH(KERN, LAYER, ...)                                              \
  do {                                                                               \
    const int nv = (d / 8 + 31) / 32;                                                \
    if (nv <= 1) KERN<LAYER, 1> __VA_ARGS__;                                         \
    else if (nv <= 2) KERN<LAYER, 2> __VA_ARGS__;                                    \
    else if (nv <= 4) KERN<LAYER, 4> __VA_ARGS__;                                    \
    else if (nv <= 8) KERN<LAYER, 8> __VA_ARGS__;                                    \
    else if (nv <= 16) KERN<LAYER, 16> __VA_ARGS__;                                  \
    else return set_error(CPB_ERR_LIMIT, "norm: d=%d exceeds 4096", d);              \
  } while (0)

// x (+res) -> xout (only when res != null), y ; stats [rows,2] (mean, rstd) optional
extern "C" int cpb_norm_fwd(const void* x, const void* res, const float* w, const float* b, void* xout, void* y,
                            float* stats, int rows, int d, float eps, int layer, cudaStream_t stream) {
  if (d % 8) return set_error(CPB_ERR_ARG, "norm: d=%d must be a multiple of 8", d);
  if (rows <= 0) return CPB_OK;
  const int wpb = 8;
  dim3 grid((rows + wpb - 1) / wpb), block(wpb * 32);
  if (layer) NORM_DISPATCH(norm_fwd_kernel, true, <<<grid, block, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, w, b, (__nv_bfloat16*)xout, (__nv_bfloat16*)y, stats, rows, d, eps));
  else NORM_DISPATCH(norm_fwd_kernel, false, <<<grid, block, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, w, b, (__nv_bfloat16*)xout, (__nv_bfloat16*)y, stats, rows, d, eps));
  return check_launch("norm_fwd");
}

// dw / db are fp32 and accumulated into (+=).
extern "C" int cpb_norm_bwd(const void* x, const void* dy, const void* dres, const float* w, const float* stats,
                            void* dx, float* dw, float* db, int rows, int d, int layer, cudaStream_t stream) {
  if (d % 8) return set_error(CPB_ERR_ARG, "norm: d=%d must be a multiple of 8", d);
  if (rows <= 0) return CPB_OK;
  int blocks = sm_count() * 2;
  int rpb = (rows + blocks - 1) / blocks;
  if (rpb < 8) rpb = 8;
  blocks = (rows + rpb - 1) / rpb;
  const size_t smem = 2 * (size_t)d * sizeof(float);
  if (layer) NORM_DISPATCH(norm_bwd_kernel, true, <<<blocks, 256, smem, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)dres, w, stats, (__nv_bfloat16*)dx, dw, db, rows, d, rpb));
  else NORM_DISPATCH(norm_bwd_kernel, false, <<<blocks, 256, smem, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)dres, w, stats, (__nv_bfloat16*)dx, dw, db, rows, d, rpb));
  return check_launch("norm_bwd");
}

extern "C" int cpb_swiglu_fwd(const void* gu, void* act, long rows, int F, cudaStream_t stream) {
  if (F % 8) return set_error(CPB_ERR_ARG, "swiglu: F must be a multiple of 8");
  if (rows <= 0) return CPB_OK;
  swiglu_fwd_kernel<<<grid_for((size_t)rows * (F / 8), 256), 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)act, (size_t)rows, F);
  return check_launch("swiglu_fwd");
}
extern "C" int cpb_swiglu_bwd(const void* gu, const void* dact, void* dgu, long rows, int F, cudaStream_t stream) {
  if (F % 8) return set_error(CPB_ERR_ARG, "swiglu: F must be a multiple of 8");
  if (rows <= 0) return CPB_OK;
  swiglu_bwd_kernel<<<grid_for((size_t)rows * (F / 8), 256), 256, 0, stream>>>((const __nv_bfloat16*)gu, (const __nv_bfloat16*)dact, (__nv_bfloat16*)dgu, (size_t)rows, F);
  return check_launch("swiglu_bwd");
}
extern "C" int cpb_gelu(const void* x, const void* dy, void* y, long n, int mode, cudaStream_t stream) {
  if (n % 8) return set_error(CPB_ERR_ARG, "gelu: n must be a multiple of 8");
  if (n <= 0) return CPB_OK;
  gelu_kernel<<<grid_for((size_t)n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (__nv_bfloat16*)y, (size_t)n / 8, mode);
  return check_launch("gelu");
}
extern "C" int cpb_add_bf16(const void* a, const void* b, void* y, long n, cudaStream_t stream) {
  if (n % 8) return set_error(CPB_ERR_ARG, "add: n must be a multiple of 8");
  if (n <= 0) return CPB_OK;
  add_kernel<<<grid_for((size_t)n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, (size_t)n / 8);
  return check_launch("add");
}
extern "C" int cpb_bias_grad(const void* dy, float* db, int rows, int N, cudaStream_t stream) {
  if (N % 2) return set_error(CPB_ERR_ARG, "bias_grad: N must be even");
  if (rows <= 0) return CPB_OK;
  int rb = sm_count() * 4 / ((N + 63) / 64);
  if (rb < 1) rb = 1;
  int rpb = (rows + rb - 1) / rb;
  if (rpb < 64) rpb = 64;
  rb = (rows + rpb - 1) / rpb;
  bias_grad_kernel<<<dim3((N + 63) / 64, rb), 256, 0, stream>>>((const __nv_bfloat16*)dy, db, rows, N, rpb);
  return check_launch("bias_grad");
}
extern "C" int cpb_embedding_fwd(const int64_t* idx, const int64_t* pos, const void* wte, const void* wpe, void* out,
                                 long rows, int d, int pos_period, cudaStream_t stream) {
  if (d % 8) return set_error(CPB_ERR_ARG, "embedding: d must be a multiple of 8");
  if (rows <= 0) return CPB_OK;
  embedding_fwd_kernel<<<grid_for((size_t)rows * (d / 8), 256), 256, 0, stream>>>(idx, pos, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, (__nv_bfloat16*)out, (size_t)rows, d, pos_period);
  return check_launch("embedding_fwd");
}
extern "C" int cpb_embedding_bwd(const int64_t* idx, const int64_t* pos, const void* dout, float* dwte, float* dwpe,
                                 long rows, int d, int pos_period, cudaStream_t stream) {
  if (d % 8) return set_error(CPB_ERR_ARG, "embedding: d must be a multiple of 8");
  if (rows <= 0) return CPB_OK;
  embedding_bwd_kernel<<<grid_for((size_t)rows * (d / 8), 256), 256, 0, stream>>>(idx, pos, (const __nv_bfloat16*)dout, dwte, dwpe, (size_t)rows, d, pos_period);
  return check_launch("embedding_bwd");
}

extern "C" int cpb_qk_norm_rope_fwd(const void* in, void* out, const float* gq, const float* gk, const float* cache,
                                    const int64_t* pos, float* rstd, long rows, int T, int Hq, int Hkv, int D,
                                    float eps, int cache_len, int* status, cudaStream_t stream) {
  if (rows <= 0) return CPB_OK;
  const int grid = grid_for((size_t)rows, 8);      // one warp per token row, eight warps per block
  if (D == 64) qk_norm_rope_fwd_kernel<64><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, gq, gk, cache, pos, rstd, (size_t)rows, T, Hq, Hkv, eps, cache_len, status);
  else if (D == 128) qk_norm_rope_fwd_kernel<128><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, gq, gk, cache, pos, rstd, (size_t)rows, T, Hq, Hkv, eps, cache_len, status);
  else return set_error(CPB_ERR_ARG, "qk_norm_rope: head_dim %d not in {64,128}", D);
  return check_launch("qk_norm_rope_fwd");
}
extern "C" int cpb_qk_norm_rope_bwd(const void* in, const void* dout, void* din, const float* gq, const float* gk,
                                    const float* cache, const int64_t* pos, float* dgq, float* dgk, long rows, int T,
                                    int Hq, int Hkv, int D, float eps, int cache_len, cudaStream_t stream) {
  if (rows <= 0) return CPB_OK;
  const int grid = grid_for((size_t)rows, 8, 4);
  if (D == 64) qk_norm_rope_bwd_kernel<64><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)in, (const __nv_bfloat16*)dout, (__nv_bfloat16*)din, gq, gk, cache, pos, dgq, dgk, (size_t)rows, T, Hq, Hkv, eps, cache_len);
  else if (D == 128) qk_norm_rope_bwd_kernel<128><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)in, (const __nv_bfloat16*)dout, (__nv_bfloat16*)din, gq, gk, cache, pos, dgq, dgk, (size_t)rows, T, Hq, Hkv, eps, cache_len);
  else return set_error(CPB_ERR_ARG, "qk_norm_rope: head_dim %d not in {64,128}", D);
  return check_launch("qk_norm_rope_bwd");
}

extern "C" int cpb_rope_cache(float* cache, const float* inv_freq, const float* lambda, const int64_t* positions,
                              long seq_len, int half, long n_hat, float mscale, cudaStream_t stream) {
  if (seq_len <= 0) return CPB_OK;
  rope_cache_kernel<<<grid_for((size_t)seq_len * half, 256), 256, 0, stream>>>(cache, inv_freq, lambda, positions, seq_len, half, n_hat, mscale);
  return check_launch("rope_cache");
}
extern "C" int cpb_gather_rows_f32(const float* src, const int64_t* index, float* out, long rows, int width,
                                   long src_rows, int* status, cudaStream_t stream) {
  if (rows <= 0) return CPB_OK;
  gather_rows_f32_kernel<<<grid_for((size_t)rows * width, 256), 256, 0, stream>>>(src, index, out, rows, width, src_rows, status);
  return check_launch("gather_rows_f32");
}
// in/out: [outer, T, inner_bytes] raw bytes
extern "C" int cpb_gather_seq(const void* in, void* out, const int64_t* index, long outer, long t_src, long t_dst,
                              long inner_bytes, int* status, cudaStream_t stream) {
  if (outer * t_dst * inner_bytes <= 0) return CPB_OK;
  const bool vec16 = (inner_bytes % 16 == 0) && (((uintptr_t)in | (uintptr_t)out) % 16 == 0);
  if (vec16) {
    const long inner = inner_bytes / 16;
    gather_seq_kernel<uint4><<<grid_for((size_t)outer * t_dst * inner, 256), 256, 0, stream>>>((const uint4*)in, (uint4*)out, index, outer, t_src, t_dst, inner, status);
  } else if (inner_bytes % 8 == 0 && (((uintptr_t)in | (uintptr_t)out) % 8 == 0)) {
    const long inner = inner_bytes / 8;
    gather_seq_kernel<uint2><<<grid_for((size_t)outer * t_dst * inner, 256), 256, 0, stream>>>((const uint2*)in, (uint2*)out, index, outer, t_src, t_dst, inner, status);
  } else {
    gather_seq_kernel<uint8_t><<<grid_for((size_t)outer * t_dst * inner_bytes, 256), 256, 0, stream>>>((const uint8_t*)in, (uint8_t*)out, index, outer, t_src, t_dst, inner_bytes, status);
  }
  return check_launch("gather_seq");
}
extern "C" int cpb_kv_pack(const void* k, const void* v, void* out, long rows, int hd, long k_row_stride,
                           long v_row_stride, cudaStream_t stream) {
  if (hd % 8 || k_row_stride % 8 || v_row_stride % 8) return set_error(CPB_ERR_ARG, "kv_pack: sizes must be multiples of 8 elements");
  if (rows <= 0) return CPB_OK;
  kv_pack_kernel<<<grid_for((size_t)2 * rows * (hd / 8), 256), 256, 0, stream>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)out, (size_t)rows, hd, (size_t)k_row_stride, (size_t)v_row_stride);
  return check_launch("kv_pack");
}
extern "C" int cpb_lse_merge(void* out, float* lse, const void* blk, const float* blk_lse, int B, int T, int H, int D,
                             int t_begin, int blk_T, int blk_t_offset, cudaStream_t stream) {
  const size_t nrow = (size_t)B * (T - t_begin) * H;
  if (nrow == 0) return CPB_OK;
  lse_merge_kernel<<<grid_for(nrow, 8), 256, 0, stream>>>((__nv_bfloat16*)out, lse, (const __nv_bfloat16*)blk, blk_lse, B, T, H, D, t_begin, blk_T, blk_t_offset);
  return check_launch("lse_merge");
}

// scratch: >= (1024 + 2) floats: [0..1023] partials, [1024] ticket (zero-initialised once), out separate
extern "C" int cpb_sumsq(const float* g, long n, float* partial, unsigned int* ticket, float* out, cudaStream_t stream) {
  int grid = grid_for((size_t)(n / 4 + 1), 256, 4);
  if (grid > 1024) grid = 1024;
  sumsq_kernel<<<grid, 256, 0, stream>>>(g, (size_t)n, partial, ticket, out);
  return check_launch("sumsq");
}
// segs: device array of {shard_begin, flat_begin, n, decay} (four longs each).
extern "C" int cpb_adamw_sharded(float* p, const float* g, float* m, float* v, void* p16, float* p32, long n_decay,
                                 const void* segs, int n_segs, int ctas_per_seg, float lr, float b1, float b2, float eps,
                                 float wd, int step, float grad_prescale, float clip, const float* sumsq, int* flag,
                                 cudaStream_t stream) {
  if (n_segs <= 0) return CPB_OK;
  if (n_segs > 65535) return set_error(CPB_ERR_LIMIT, "adamw_sharded: at most 65535 segments");
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  dim3 grid(ctas_per_seg < 1 ? 1 : ctas_per_seg, n_segs);
  adamw_sharded_kernel<<<grid, 256, 0, stream>>>(p, g, m, v, (__nv_bfloat16*)p16, p32, n_decay, (const AdamSeg*)segs, lr, b1, b2,
                                                 eps, wd, bc1, bc2, grad_prescale, clip, sumsq, flag);
  return check_launch("adamw_sharded");
}

extern "C" int cpb_adamw(float* p, const float* g, float* m, float* v, void* p16, long n, float lr, float b1, float b2,
                         float eps, float wd, int step, float grad_prescale, float clip, const float* sumsq, int* flag,
                         cudaStream_t stream) {
  if (n <= 0) return CPB_OK;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  adamw_kernel<<<grid_for((size_t)n, 256), 256, 0, stream>>>(p, g, m, v, (__nv_bfloat16*)p16, (size_t)n, lr, b1, b2, eps, wd, bc1, bc2, grad_prescale, clip, sumsq, flag);
  return check_launch("adamw");
}
extern "C" int cpb_cast_f32_bf16(const float* in, void* out, long n, float scale, cudaStream_t stream) {
  if (n <= 0) return CPB_OK;
  cast_f32_bf16_kernel<<<grid_for((size_t)n, 256), 256, 0, stream>>>(in, (__nv_bfloat16*)out, (size_t)n, scale);
  return check_launch("cast_f32_bf16");
}
extern "C" int cpb_cast_bf16_f32(const void* in, float* out, long n, float scale, int accumulate, cudaStream_t stream) {
  if (n <= 0) return CPB_OK;
  cast_bf16_f32_kernel<<<grid_for((size_t)n, 256), 256, 0, stream>>>((const __nv_bfloat16*)in, out, (size_t)n, scale, accumulate);
  return check_launch("cast_bf16_f32");
}
