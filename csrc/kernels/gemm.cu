// Persistent bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma -> tensor memory ->
// registers -> global, warp-specialised, with a double-buffered accumulator so the epilogue of tile
// i overlaps the main loop of tile i+1.
//
//   C[M,N] (op)= A * B        A is M x K, B is N x K ("NT": both K-major) by default.
//   a_mn = 1 : A is stored as [K, M] (M contiguous)   -> weight-gradient GEMM  dW = dY^T X
//   b_mn = 1 : B is stored as [K, N] (N contiguous)   -> data-gradient GEMM    dX = dY W
// Both majors are native UMMA operand layouts, so no transposed copies are ever made.
//
// Replaces the cuBLAS GEMMs behind nn::Linear in the reference trainers
// (Scripts/Blutrain/bluscriptCP.cpp:212-330, Makefile:129).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = tensor-memory owner + MMA issuer,
// warps 2..5 = epilogue (warp w reads TMEM lanes 32*(w%4)..+31).
#include "common.cuh"
#include "gemm_common.cuh"
#include "host_utils.h"
#include <stdlib.h>

namespace cpb {

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  using L = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;     // [2]
  uint64_t* tempty_bar = tfull_bar + 2;         // [2]
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tfull_bar[s], 1); mbar_init(&tempty_bar[s], 4); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0; uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int m0 = (tile / p.num_n_blocks) * GEMM_BM;
        const int n0 = (tile % p.num_n_blocks) * BN;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 100)) break;
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          const int k0 = kb * GEMM_BK;
          if (A_MN) {
#pragma unroll
            for (int g = 0; g < GEMM_BM / 64; ++g) tma_load_2d(sa + g * 8192, &tmA, &full_bar[stage], m0 + g * 64, k0);
          } else {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
          }
          if (p.epi == EPI_BF16_SWIGLU) {
            // gate rows n0/2.. and up rows F + n0/2.. of the fused [2F, K] weight
            const int f0 = (tile % p.num_n_blocks) * (BN / 2);
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, f0);
            tma_load_2d(sb + (BN / 2) * 128, &tmB, &full_bar[stage], k0, p.swiglu_half + f0);
          } else if (B_MN) {
#pragma unroll
            for (int g = 0; g < BN / 64; ++g) tma_load_2d(sb + g * 8192, &tmB, &full_bar[stage], n0 + g * 64, k0);
          } else {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop convergently and only the elected lane issues, so that the descriptors stay
    // warp-uniform and stepping one is a single add: at BN = 128 an MMA lasts 64 cycles, and the scalar work between
    // two of them must stay well below that.
    {
      const uint32_t leader = elect_one() ? 1u : 0u;
      constexpr uint32_t idesc = make_idesc_bf16(GEMM_BM, BN, A_MN, B_MN);
      const uint32_t s0 = smem_u32(smem);
      const SDesc da0 = sdesc_split(A_MN ? make_sdesc(s0, 8192, 1024) : sdesc_kmajor(s0));                       // stage 0
      const SDesc db0 = sdesc_split(B_MN ? make_sdesc(s0 + L::A_BYTES, 8192, 1024) : sdesc_kmajor(s0 + L::A_BYTES));
      constexpr uint32_t A_STEP = A_MN ? 2048 : 32, B_STEP = B_MN ? 2048 : 32;
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, 200))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 201))) { alive = false; break; }
          tc_fence_after();
          const uint32_t so = (uint32_t)stage * (L::STAGE_BYTES >> 4);
          const SDesc da = SDesc{da0.lo + so, da0.hi}, db = SDesc{db0.lo + so, db0.hi};
          umma_ss_p(leader, d_tmem, sdesc_at(da, 0), sdesc_at(db, 0), idesc, kb != 0);
#pragma unroll
          for (int k = 1; k < GEMM_BK / 16; ++k)
            umma_ss_cp<true>(leader, d_tmem, sdesc_at(da, k * A_STEP), sdesc_at(db, k * B_STEP), idesc);
          umma_commit_p(leader, &empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit_p(leader, &tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int m0 = (tile / p.num_n_blocks) * GEMM_BM;
      const int nb = tile % p.num_n_blocks;
      bool ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, 300);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      gemm_epilogue_row<BN>(p, t_row, row, nb);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, cudaStream_t stream) {
  using L = GemmSmem<BN, STAGES>;
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    CPB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    configured = true;
  }
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, GEMM_THREADS, L::TOTAL, stream>>>(tmA, tmB, p);
  return check_launch("gemm_bf16");
}

int gemm_pair_dispatch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int a_mn, int b_mn, cudaStream_t stream);

}  // namespace cpb

using namespace cpb;

// A: bf16, [M,K] row stride lda (a_mn=0) or [K,M] row stride lda (a_mn=1).
// B: bf16, [N,K] row stride ldb (b_mn=0) or [K,N] row stride ldb (b_mn=1).
// epi: see EPI_* above.  For EPI_BF16_SWIGLU B is the fused [2F, K] weight, N = F output features.
extern "C" int cpb_gemm_bf16(const void* A, const void* B, void* C, void* aux, const float* bias,
                             int M, int N, int K, int lda, int ldb, int ldc, int ld_aux,
                             int a_mn, int b_mn, int epi, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return set_error(CPB_ERR_ARG, "gemm: empty problem %dx%dx%d", M, N, K);
  // the contiguous dimension of every operand and every row stride must be a multiple of 8 elements (16 bytes)
  if ((N % 8) || (lda % 8) || (ldb % 8)) return set_error(CPB_ERR_ARG, "gemm: N,lda,ldb must be multiples of 8 (got N=%d lda=%d ldb=%d)", N, lda, ldb);
  if ((!a_mn || !b_mn) && (K % 8)) return set_error(CPB_ERR_ARG, "gemm: K=%d must be a multiple of 8 for a K-major operand", K);
  if (a_mn && (M % 8)) return set_error(CPB_ERR_ARG, "gemm: M must be a multiple of 8 when A is M-major");
  if (epi == EPI_BF16_SWIGLU && (a_mn || b_mn)) return set_error(CPB_ERR_ARG, "gemm: swiglu epilogue needs K-major operands");
  const int BN = (epi == EPI_BF16_SWIGLU || N > 128) ? 256 : 128;
  // CTA pairs (gemm2.cu: 256 x 256 tiles, half the shared-memory traffic per tensor-core step) for everything large
  // enough to fill pairs; CPB_GEMM_PAIR=0 (read once) keeps the one-CTA kernel.
  static const bool pair_ok = [] { const char* e = getenv("CPB_GEMM_PAIR"); return e == nullptr || e[0] != '0'; }();
  const bool use_pair = pair_ok && BN == 256 && M >= 256;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ld_aux = ld_aux; p.epi = epi;
  p.num_m_blocks = (M + GEMM_BM - 1) / GEMM_BM;
  p.num_k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
  p.swiglu_half = (epi == EPI_BF16_SWIGLU) ? N : 0;
  // banded tile order of the pair kernel once B (N x K bf16) reaches 64 MB, half of L2; CPB_GEMM_BAND (read once) overrides
  static const int band_env = [] { const char* e = getenv("CPB_GEMM_BAND"); return e ? atoi(e) : 0; }();
  p.band = band_env > 0 ? band_env : (((size_t)N * K * 2 >= ((size_t)64 << 20)) ? 8 : 1);
  p.num_n_blocks = (epi == EPI_BF16_SWIGLU) ? (N + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN;
  p.C = C; p.aux = aux; p.bias = bias; p.status = status;

  CUtensorMap tmA, tmB;
  int rc;
  {
    uint64_t dims[2], strides[2]; uint32_t box[2];
    if (a_mn) { dims[0] = (uint64_t)M; dims[1] = (uint64_t)K; box[0] = 64; box[1] = GEMM_BK; }
    else      { dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; box[0] = GEMM_BK; box[1] = GEMM_BM; }
    strides[0] = 0; strides[1] = (uint64_t)lda * 2;
    if ((rc = encode_tmap(&tmA, A, 2, 2, dims, strides, box, 1)) != CPB_OK) return rc;
  }
  {
    uint64_t dims[2], strides[2]; uint32_t box[2];
    const uint64_t b_rows = (epi == EPI_BF16_SWIGLU) ? (uint64_t)2 * N : (uint64_t)N;
    if (b_mn) { dims[0] = b_rows; dims[1] = (uint64_t)K; box[0] = 64; box[1] = GEMM_BK; }
    else      { dims[0] = (uint64_t)K; dims[1] = b_rows; box[0] = GEMM_BK; box[1] = (epi == EPI_BF16_SWIGLU || use_pair) ? BN / 2 : BN; }
    strides[0] = 0; strides[1] = (uint64_t)ldb * 2;
    if ((rc = encode_tmap(&tmB, B, 2, 2, dims, strides, box, 1)) != CPB_OK) return rc;
  }
  if (use_pair) return gemm_pair_dispatch(tmA, tmB, p, a_mn, b_mn, stream);
#define CPB_GEMM_DISPATCH(BN_, ST_)                                                      \
  do {                                                                                   \
    if (!a_mn && !b_mn) return launch_gemm<BN_, ST_, false, false>(tmA, tmB, p, stream);  \
    if (!a_mn && b_mn) return launch_gemm<BN_, ST_, false, true>(tmA, tmB, p, stream);    \
    if (a_mn && !b_mn) return launch_gemm<BN_, ST_, true, false>(tmA, tmB, p, stream);    \
    return launch_gemm<BN_, ST_, true, true>(tmA, tmB, p, stream);                        \
  } while (0)
  if (BN == 256) CPB_GEMM_DISPATCH(256, 4);
  CPB_GEMM_DISPATCH(128, 6);
#undef CPB_GEMM_DISPATCH
}
