// Definitions shared by the one-CTA (gemm.cu) and the CTA-pair (gemm2.cu) bf16 GEMM kernels: parameters, epilogue kinds
// and the epilogue itself (tensor memory -> registers -> global memory, with bias / GELU / SwiGLU / fp32 accumulate).
#pragma once
#include "common.cuh"

namespace cpb {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;

enum : int {
  EPI_BF16 = 0,        // C(bf16) = acc (+bias)
  EPI_F32 = 1,         // C(f32)  = acc (+bias)
  EPI_F32_ACC = 2,     // C(f32) += acc
  EPI_BF16_GELU = 3,   // C(bf16) = gelu_tanh(acc + bias); aux(bf16) = acc + bias (pre-activation) when aux != null
  EPI_BF16_SWIGLU = 4, // B tile = [gate rows | up rows]; C(bf16)[:, n] = silu(g)*u ; aux gets [g | u] when aux != null
};

struct GemmParams {
  int M, N, K;
  int ldc;             // elements
  int ld_aux;
  int epi;
  int num_m_blocks, num_n_blocks, num_k_blocks;
  int swiglu_half;     // number of output features F when epi == SWIGLU (B has 2F rows)
  int band;            // CTA-pair kernel: pair-rows per band of the tile order (1 = rows of tiles, columns fastest)
  void* C;
  void* aux;
  const float* bias;
  int* status;
};

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;   // barriers + alignment slack
};

__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  // tanh(u) = 1 - 2/(exp(2u)+1)
  float e = __expf(2.f * u);
  float t = 1.f - 2.f / (e + 1.f);
  return 0.5f * x * (1.f + t);
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

// Epilogue of one 128 x BN accumulator tile for one thread: `row` is the thread's output row (tensor-memory lane),
// `t_row` the tensor-memory address of that lane's first accumulator column, `nb` the tile's index along N.
template <int BN>
__device__ __forceinline__ void gemm_epilogue_row(const GemmParams& p, uint32_t t_row, int row, int nb) {
  const int n0 = nb * BN;
      if (p.epi == EPI_BF16_SWIGLU) {
  // accumulator columns [0, BN/2) = gate, [BN/2, BN) = up, for features f0..f0+BN/2
  const int f0 = nb * (BN / 2);
#pragma unroll 1
  for (int c = 0; c < BN / 2; c += 32) {
    uint32_t g[32], u[32];
    tmem_ld32(t_row + c, g);
    tmem_ld32(t_row + BN / 2 + c, u);
    tmem_wait_ld();
    if (row < p.M) {
      __nv_bfloat16* crow = (__nv_bfloat16*)p.C + (size_t)row * p.ldc + f0 + c;
      __nv_bfloat16* arow = p.aux ? (__nv_bfloat16*)p.aux + (size_t)row * p.ld_aux : nullptr;
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        if (f0 + c + j < p.swiglu_half) {
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float g0 = __uint_as_float(g[j + 2 * q]), g1 = __uint_as_float(g[j + 2 * q + 1]);
            float u0 = __uint_as_float(u[j + 2 * q]), u1 = __uint_as_float(u[j + 2 * q + 1]);
            o[q] = pack_bf16(silu_f(g0) * u0, silu_f(g1) * u1);
          }
          *(uint4*)(crow + j) = make_uint4(o[0], o[1], o[2], o[3]);
          if (arow) {
            uint32_t pg[4], pu[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              pg[q] = pack_bf16(__uint_as_float(g[j + 2 * q]), __uint_as_float(g[j + 2 * q + 1]));
              pu[q] = pack_bf16(__uint_as_float(u[j + 2 * q]), __uint_as_float(u[j + 2 * q + 1]));
            }
            *(uint4*)(arow + f0 + c + j) = make_uint4(pg[0], pg[1], pg[2], pg[3]);
            *(uint4*)(arow + p.swiglu_half + f0 + c + j) = make_uint4(pu[0], pu[1], pu[2], pu[3]);
          }
        }
      }
    }
  }
} else {
#pragma unroll 1
  for (int c = 0; c < BN; c += 32) {
    uint32_t v[32];
    tmem_ld32(t_row + c, v);
    tmem_wait_ld();
    const int col = n0 + c;
    if (row < p.M && col < p.N) {
      if (p.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col + j < p.N) v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldg(p.bias + col + j));
      }
      if (p.epi == EPI_BF16 || p.epi == EPI_BF16_GELU) {
        __nv_bfloat16* crow = (__nv_bfloat16*)p.C + (size_t)row * p.ldc + col;
        __nv_bfloat16* arow = (p.epi == EPI_BF16_GELU && p.aux) ? (__nv_bfloat16*)p.aux + (size_t)row * p.ld_aux + col : nullptr;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (col + j < p.N) {       // N is a multiple of 8
            uint32_t o[4];
            if (p.epi == EPI_BF16_GELU) {
              if (arow) {
                uint32_t a[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) a[q] = pack_bf16(__uint_as_float(v[j + 2 * q]), __uint_as_float(v[j + 2 * q + 1]));
                *(uint4*)(arow + j) = make_uint4(a[0], a[1], a[2], a[3]);
              }
#pragma unroll
              for (int q = 0; q < 4; ++q)
                o[q] = pack_bf16(gelu_tanh_f(__uint_as_float(v[j + 2 * q])), gelu_tanh_f(__uint_as_float(v[j + 2 * q + 1])));
            } else {
#pragma unroll
              for (int q = 0; q < 4; ++q) o[q] = pack_bf16(__uint_as_float(v[j + 2 * q]), __uint_as_float(v[j + 2 * q + 1]));
            }
            *(uint4*)(crow + j) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      } else {
        float* crow = (float*)p.C + (size_t)row * p.ldc + col;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          if (col + j < p.N) {       // N is a multiple of 4 on this path
            float4 o = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
            if (p.epi == EPI_F32_ACC) {
              float4 old = *(float4*)(crow + j);
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            *(float4*)(crow + j) = o;
          }
        }
      }
    }
  }
}
}

}  // namespace cpb
