// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): two CTAs of a cluster compute one 256 x 256 output tile together.
//
// Why: with one CTA per tile (gemm.cu, 128 x 256) every K=16 step of the tensor core reads (128 + 256) x 16 x 2 = 12 KB of
// operands from shared memory while TMA writes the same 12 KB, i.e. 192 bytes per tensor-core cycle against the 128 bytes
// per cycle a shared memory delivers: that kernel tops out near 0.75 of cuBLAS.  In a pair each CTA stages its own 128 rows
// of A and only HALF of the B tile (128 of the 256 columns); one MMA instruction issued by the even CTA drives both tensor
// cores and each of them reads the other CTA's B half through the pair link, so a CTA moves (128 + 128) x 16 x 2 = 8 KB in
// and 8 KB out per step: 128 bytes per cycle.
//
// Protocol (per CTA: warp 0 = TMA producer, warp 1 = tensor-memory owner and, in the even CTA, MMA issuer, warps 2..5 =
// epilogue).  Every TMA load of either CTA (cta_group::2 form, no multicast) signals the EVEN CTA's `full` barrier, which
// expects the bytes of both CTAs.  After the MMAs of a stage the issuer commits twice, once to its own `empty` barrier and
// once to the odd CTA's (a cluster address), and likewise for the accumulator-ready barriers; the odd CTA's epilogue
// warps release an accumulator by a remote arrival on the even CTA's barrier.  Tensor memory is allocated with the
// cta_group::2 form by the same warp of both CTAs, so an accumulator has the same address in both; each CTA's epilogue
// drains its own 128 rows.  All waits are bounded like everywhere else in this library.
//
// Operand layouts, epilogues and the C ABI are those of gemm.cu, which remains the kernel for small problems.
#include "common.cuh"
#include "gemm_common.cuh"
#include "host_utils.h"

namespace cpb {

constexpr int G2_BN = 256;
constexpr int G2_STAGES = 6;

struct G2Smem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;          // 128 rows of A
  static constexpr int B_BYTES = (G2_BN / 2) * GEMM_BK * 2;      // this CTA's 128 columns of B
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = G2_STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of a CTA pair: the data lands in THIS CTA's shared memory, the bytes are counted on the barrier at `bar_addr`
// (a cluster address: the even CTA's barrier).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem, const CUtensorMap* m, uint32_t bar_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem)), "l"((uint64_t)m), "r"(bar_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {      // same warp of both CTAs
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
template <bool ACC>
__device__ __forceinline__ void umma_pair_ss_cp(uint32_t leader, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "n"(ACC ? 1 : 0), "r"(leader) : "memory");
}
__device__ __forceinline__ void umma_pair_ss_p(uint32_t leader, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader) : "memory");
}
// Arrive on the barrier at `cluster_addr` (any CTA of the cluster) once every MMA issued so far has completed.
__device__ __forceinline__ void umma_pair_commit_p(uint32_t leader, uint32_t cluster_addr) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(cluster_addr), "r"(leader) : "memory");
}

// Tile order: bands of `band` pair-rows swept along N, rows fastest.  With band = 8 the 74 pairs running at one time
// share 8 row tiles of A and about 9 column tiles of B, and successive waves keep the band's A rows in L2, so a GEMM
// whose B operand does not fit in L2 beside A's band (8192^3: 134 MB against 126 MB) streams B once per band instead of
// once per 2.3 rows of tiles.  band = 1 is the plain order (columns fastest), kept while B stays resident anyway.
__device__ __forceinline__ void pair_tile_coords(int tile, int num_m_tiles, int num_n_blocks, int band_rows, int& mt, int& nb) {
  const int per_band = band_rows * num_n_blocks;
  const int band = tile / per_band, idx = tile - band * per_band;
  const int rows = min(band_rows, num_m_tiles - band * band_rows);
  nb = idx / rows;
  mt = band * band_rows + (idx - nb * rows);
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  using L = G2Smem;
  constexpr int BN = G2_BN, STAGES = G2_STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFFSET);      // used in the even CTA only
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;     // [2]
  uint64_t* tempty_bar = tfull_bar + 2;         // [2], used in the even CTA only
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0: even CTA (issues the MMAs), 1: odd CTA
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_m_tiles = (p.M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
  const int num_tiles = num_m_tiles * p.num_n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tfull_bar[s], 1); mbar_init(&tempty_bar[s], 8); }      // 4 epilogue warps of each CTA
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 2 * BN);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                           // both CTAs' barriers exist before anything arrives on them remotely
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0; uint32_t phase = 0;
      for (int tile = pair; tile < num_tiles; tile += num_pairs) {
        int mt, nb;
        pair_tile_coords(tile, num_m_tiles, p.num_n_blocks, p.band, mt, nb);
        const int m0 = mt * (2 * GEMM_BM) + (int)rank * GEMM_BM;      // this CTA's rows
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 110)) break;
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          const uint32_t full_even = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * L::STAGE_BYTES);              // the bytes of both CTAs
          const int k0 = kb * GEMM_BK;
          if (A_MN) {
#pragma unroll
            for (int g = 0; g < GEMM_BM / 64; ++g) tma_load_2d_pair(sa + g * 8192, &tmA, full_even, m0 + g * 64, k0);
          } else {
            tma_load_2d_pair(sa, &tmA, full_even, k0, m0);
          }
          if (p.epi == EPI_BF16_SWIGLU) {
            // the even CTA stages the gate rows of features nb*128.., the odd CTA the matching up rows
            const int f0 = nb * (BN / 2);
            tma_load_2d_pair(sb, &tmB, full_even, k0, (rank == 0 ? 0 : p.swiglu_half) + f0);
          } else if (B_MN) {
            const int n0 = nb * BN + (int)rank * (BN / 2);
#pragma unroll
            for (int g = 0; g < BN / 2 / 64; ++g) tma_load_2d_pair(sb + g * 8192, &tmB, full_even, n0 + g * 64, k0);
          } else {
            tma_load_2d_pair(sb, &tmB, full_even, k0, nb * BN + (int)rank * (BN / 2));
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only; convergent warp, elected lane)
    if (rank == 0) {
      const uint32_t leader = elect_one() ? 1u : 0u;
      constexpr uint32_t idesc = make_idesc_bf16(2 * GEMM_BM, BN, A_MN, B_MN);
      const uint32_t s0 = smem_u32(smem);
      const SDesc da0 = sdesc_split(A_MN ? make_sdesc(s0, 8192, 1024) : sdesc_kmajor(s0));
      const SDesc db0 = sdesc_split(B_MN ? make_sdesc(s0 + L::A_BYTES, 8192, 1024) : sdesc_kmajor(s0 + L::A_BYTES));
      constexpr uint32_t A_STEP = A_MN ? 2048 : 32, B_STEP = B_MN ? 2048 : 32;
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      bool alive = true;
      for (int tile = pair; tile < num_tiles && alive; tile += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, 210))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 211))) { alive = false; break; }
          tc_fence_after();
          const uint32_t so = (uint32_t)stage * (L::STAGE_BYTES >> 4);
          const SDesc da = SDesc{da0.lo + so, da0.hi}, db = SDesc{db0.lo + so, db0.hi};
          umma_pair_ss_p(leader, d_tmem, sdesc_at(da, 0), sdesc_at(db, 0), idesc, kb != 0);
#pragma unroll
          for (int k = 1; k < GEMM_BK / 16; ++k)
            umma_pair_ss_cp<true>(leader, d_tmem, sdesc_at(da, k * A_STEP), sdesc_at(db, k * B_STEP), idesc);
          // the stage is free in both CTAs once these MMAs have read it
          const uint32_t e_own = smem_u32(&empty_bar[stage]);
          umma_pair_commit_p(leader, e_own);
          umma_pair_commit_p(leader, map_to_cta(e_own, 1));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        const uint32_t t_own = smem_u32(&tfull_bar[acc]);
        umma_pair_commit_p(leader, t_own);
        umma_pair_commit_p(leader, map_to_cta(t_own, 1));
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs: own 128 rows)
    const int quarter = warp & 3;
    int it = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      int mt, nb;
      pair_tile_coords(tile, num_m_tiles, p.num_n_blocks, p.band, mt, nb);
      const int m0 = mt * (2 * GEMM_BM) + (int)rank * GEMM_BM;
      bool ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, 310);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      gemm_epilogue_row<BN>(p, t_row, row, nb);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(&tempty_bar[acc]);
        else mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the even CTA's MMAs have finished reading the odd CTA's operands; no remote arrival is in flight
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * BN);
  }
}

template <bool A_MN, bool B_MN>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, cudaStream_t stream) {
  auto kern = gemm_pair_bf16_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    CPB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G2Smem::TOTAL));
    configured = true;
  }
  const int tiles = ((p.M + 2 * GEMM_BM - 1) / (2 * GEMM_BM)) * p.num_n_blocks;
  const int max_pairs = sm_count() / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kern<<<2 * pairs, GEMM_THREADS, G2Smem::TOTAL, stream>>>(tmA, tmB, p);
  return check_launch("gemm_pair_bf16");
}

// Called by cpb_gemm_bf16 (gemm.cu) with tensor maps whose B box holds 128 rows (K-major) resp. 64 x 64 (N-major).
int gemm_pair_dispatch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int a_mn, int b_mn, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_pair<false, false>(tmA, tmB, p, stream);
  if (!a_mn && b_mn) return launch_pair<false, true>(tmA, tmB, p, stream);
  if (a_mn && !b_mn) return launch_pair<true, false>(tmA, tmB, p, stream);
  return launch_pair<true, true>(tmA, tmB, p, stream);
}

}  // namespace cpb
