// Flash-attention backward for sm_100a.  One CTA owns one 128-row K/V tile of one KV head and sweeps
// every query tile (of every query head of the GQA group) that can see it, with all five products
// on tcgen05 tensor cores and every accumulator in tensor memory:
//
//   S  = Q K^T              (smem x smem)          P  = exp2(S*c - LSE)             (registers -> smem, bf16)
//   dP = dO V^T             (smem x smem)          dS = P o (dP - Delta)            (registers -> smem, bf16)
//   dV += P^T dO            (smem x smem, P read M-major)     dK += dS^T Q  (smem x smem, dS read M-major)
//   dQ  = dS K              (smem x smem, dS read K-major) -> staged in shared memory and added to the fp32
//                           dQ buffer by TMA reduce (cp.reduce.async.bulk.tensor .add)
//
// Query rows sit in tensor-memory lanes, so LSE, Delta and the query position are per-thread scalars and
// the inner loop touches no shared-memory vectors.  The bf16 P and dS tiles are written once to shared
// memory in the 128-byte-swizzled layout that serves, unchanged, as the M-major A operand of the dV / dK
// products and as the K-major A operand of the dQ product.  dK / dV stay in tensor memory for the whole
// sweep and are written as bf16, accumulated into fp32 buffers, or (fused ring) added to their owners'
// accumulators over NVLink (the ring calls the kernel once per query shard and sums contributions, like
// the reference's travelling fp32 accumulator, context_parallel/ContextParallelBackward.h:151-158,546-627).
// dS is formed without the softmax scale; dK is scaled in the final epilogue and dQ in the drain warps.
// P is recomputed from the merged LSE (context_parallel/AttentionBackward.cu:446).  Masking is on global
// positions, as in the forward.
//
// Replaces mem_efficient_bwd_unified_kernel_exp11 (context_parallel/AttentionBackward.cu:300-541) and
// gqa_fused_rope_bwd_dQ / _dKdV (context_parallel/GQA_fused_bwd_sm103_cp.cu:135-565).
//
// Warp roles (448 threads): 0 = TMA loader, 1 = MMA issuer, 2..9 = softmax-gradient warps (two threads per query
// row, 64 key columns each, so every scheduler has two such warps to hide tensor-memory and MUFU latency),
// 10..13 = dQ drain warps (thread = query row).
#include "common.cuh"
#include <type_traits>
#include "host_utils.h"

#include <stdlib.h>

namespace cpb {


constexpr int FB_T = 128;            // tile edge (queries and keys)
constexpr int FB_THREADS = 448;

struct BwdParams {
  int B, Tq, Tk, Hq, Hkv, Tq_pad;
  int causal, k_off;
  float scale, scale_log2;
  const float* lse2;        // [B,Hq,Tq_pad] LSE * log2(e), +inf in the padding
  const float* delta;       // [B,Hq,Tq_pad] rowsum(dO o O), 0 in the padding
  const int* q_pos;         // [Tq_pad] global positions, INT_MAX in the padding
  float* dq;                // [B,Tq,Hq,D] fp32, accumulated by TMA reduce-add
  void* dk; void* dv;       // [B,Tk,Hkv,D] bf16 (store) or fp32 (accumulate)
  int dkv_f32_accumulate;
  // fused ring (dkv_f32_accumulate == 2): K/V row kidx belongs to chunk c = kidx / route_rows, owned by some
  // rank; route_k[c] / route_v[c] are the addresses (peer-mapped) of that owner's fp32 accumulators at the
  // chunk's first local row for batch 0, whose layout is [B, route_tl, Hkv, D].  The epilogue adds the tile
  // with red.global.add over NVLink.
  const uint64_t* route_k;
  const uint64_t* route_v;
  int route_rows, route_tl;
  int debug_skip_dq;        // diagnostic: do not add dQ tiles to global memory (timing experiments only)
  int* status;
};

template <int D>
struct BwdSmem {
  static constexpr int STAGES = (D == 64) ? 2 : 1;
  static constexpr int TILE = FB_T * D * 2;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE;
  static constexpr int Q_OFF = 2 * TILE;
  static constexpr int DO_OFF = Q_OFF + STAGES * TILE;
  static constexpr int PS_OFF = DO_OFF + STAGES * TILE;           // P : 128 queries x 128 keys bf16, 128B-swizzled
  static constexpr int DS_BUFS = (D == 64) ? 2 : 1;               // head_dim 64: dS double-buffered (pipelined issue order)
  static constexpr int DS_OFF = PS_OFF + FB_T * FB_T * 2;         // dS: same layout
  static constexpr int DQS_OFF = DS_OFF + DS_BUFS * FB_T * FB_T * 2;   // dQ staging: boxes of 128 rows x 32 fp32, 128B-swizzled
  static constexpr int DQ_BOXES = (D == 64) ? 1 : 2;              // boxes staged per TMA-reduce round
  static constexpr int VEC_OFF = DQS_OFF + DQ_BOXES * FB_T * 128;        // per stage: lse2[128], delta[128], qpos[128]
  static constexpr int BAR_OFF = VEC_OFF + STAGES * 3 * 512;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ void bulk_load_1d(void* smem, const void* gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem)), "l"((uint64_t)gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int D>
__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const __grid_constant__ CUtensorMap tmDQ, BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int ST = L::STAGES;
  constexpr int DH = D / 64;
  constexpr uint32_t S_COL = 0, DP_COL = 128, DV_COL = 256, DK_COL = 256 + D;
  constexpr uint32_t DQ_COL = (D == 64) ? 384 : 0;           // D=128: dQ reuses the S columns
  constexpr bool DQ_ALIAS = (D != 64);
  constexpr bool OVERLAP = (D == 64);                         // pipelined issue order (see the MMA issuer)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + L::BAR_OFF);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;        // [2]
  uint64_t* q_empty = bars + 3;       // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* dq_full = bars + 7;
  uint64_t* dq_empty = bars + 8;
  uint64_t* acc_done = bars + 9;
  uint64_t* ds_empty = bars + 10;     // [2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 12);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* qt_start_s = (int*)(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int k0 = kt * FB_T;
  const int num_q_tiles = p.Tq_pad / FB_T;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    mbar_init(s_full, 1); mbar_init(p_full, 8); mbar_init(dq_full, 1); mbar_init(dq_empty, 4); mbar_init(acc_done, 1);
    mbar_init(&ds_empty[0], 1); mbar_init(&ds_empty[1], 1);
    *abort_flag = 0;
    *qt_start_s = num_q_tiles;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // First query tile that can see this K/V tile (q_pos is non-decreasing).
  if (p.causal) {
    const int kpos_min = p.k_off + k0;
    for (int t = threadIdx.x; t < num_q_tiles; t += blockDim.x) {
      const int last = min(t * FB_T + FB_T, p.Tq) - 1;
      if (p.q_pos[last] >= kpos_min) { atomicMin(qt_start_s, t); break; }
    }
  } else if (threadIdx.x == 0) {
    *qt_start_s = 0;
  }
  __syncthreads();
  const int qt_start = *qt_start_s;
  const int n_qt = num_q_tiles - qt_start;
  const int n_it = n_qt * G;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA loader
    if (lane == 0 && n_it > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
      mbar_expect_tx(kv_full, 2 * L::TILE);
#pragma unroll
      for (int h = 0; h < DH; ++h) {
        tma_load_4d(smem + L::K_OFF + h * (FB_T * 128), &tmK, kv_full, h * 64, hkv, k0, b);
        tma_load_4d(smem + L::V_OFF + h * (FB_T * 128), &tmV, kv_full, h * 64, hkv, k0, b);
      }
      for (int i = 0; i < n_it; ++i) {
        const int st = i % ST;
        const uint32_t ph = (i / ST) & 1;
        if (!mbar_wait(&q_empty[st], ph ^ 1, abort_flag, p.status, 800)) break;
        const int hq = hkv * G + i / n_qt;
        const int q0 = (qt_start + i % n_qt) * FB_T;
        mbar_expect_tx(&q_full[st], 2 * L::TILE + 3 * 512);
#pragma unroll
        for (int h = 0; h < DH; ++h) {
          tma_load_4d(smem + L::Q_OFF + st * L::TILE + h * (FB_T * 128), &tmQ, &q_full[st], h * 64, hq, q0, b);
          tma_load_4d(smem + L::DO_OFF + st * L::TILE + h * (FB_T * 128), &tmDO, &q_full[st], h * 64, hq, q0, b);
        }
        uint8_t* vec = smem + L::VEC_OFF + st * 1536;
        const size_t row_off = ((size_t)b * p.Hq + hq) * p.Tq_pad + q0;
        bulk_load_1d(vec, p.lse2 + row_off, 512, &q_full[st]);
        bulk_load_1d(vec + 512, p.delta + row_off, 512, &q_full[st]);
        bulk_load_1d(vec + 1024, p.q_pos + q0, 512, &q_full[st]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs this code convergently and only the elected lane issues, so that the descriptors stay
    // warp-uniform and stepping one is a single add.
    if (n_it > 0) {
      const uint32_t leader = elect_one() ? 1u : 0u;
      constexpr uint32_t idesc_s = make_idesc_bf16(FB_T, FB_T, false, false);     // S, dP
      constexpr uint32_t idesc_acc = make_idesc_bf16(FB_T, D, true, true);         // dV, dK: A M-major smem, B N-major
      constexpr uint32_t idesc_dq = make_idesc_bf16(FB_T, D, false, true);         // dQ: A K-major smem, B N-major
      const SDesc dK_k = sdesc_split(sdesc_kmajor(smem_u32(smem + L::K_OFF))), dV_k = sdesc_split(sdesc_kmajor(smem_u32(smem + L::V_OFF)));
      const SDesc dK_n = sdesc_split(make_sdesc(smem_u32(smem + L::K_OFF), FB_T * 128, 1024));
      const SDesc dQ_k0 = sdesc_split(sdesc_kmajor(smem_u32(smem + L::Q_OFF))), dDO_k0 = sdesc_split(sdesc_kmajor(smem_u32(smem + L::DO_OFF)));
      const SDesc dQ_n0 = sdesc_split(make_sdesc(smem_u32(smem + L::Q_OFF), FB_T * 128, 1024));
      const SDesc dDO_n0 = sdesc_split(make_sdesc(smem_u32(smem + L::DO_OFF), FB_T * 128, 1024));
      const SDesc dP_m = sdesc_split(make_sdesc(smem_u32(smem + L::PS_OFF), FB_T * 128, 1024));
      const SDesc dDS_m0 = sdesc_split(make_sdesc(smem_u32(smem + L::DS_OFF), FB_T * 128, 1024));
      const SDesc dDS_k0 = sdesc_split(sdesc_kmajor(smem_u32(smem + L::DS_OFF)));
      const uint32_t t_s = tmem_base + S_COL, t_dp = tmem_base + DP_COL, t_dv = tmem_base + DV_COL, t_dk = tmem_base + DK_COL, t_dq = tmem_base + DQ_COL;
      auto stage = [](SDesc d, int st) { return SDesc{d.lo + (uint32_t)st * (L::TILE >> 4), d.hi}; };
      auto issue_scores = [&](int st) {
        const SDesc q = stage(dQ_k0, st), g = stage(dDO_k0, st);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {       // S = Q K^T
          const uint32_t off = (k / 4) * (FB_T * 128) + (k % 4) * 32;
          if (k == 0) umma_ss_cp<false>(leader, t_s, sdesc_at(q, off), sdesc_at(dK_k, off), idesc_s);
          else umma_ss_cp<true>(leader, t_s, sdesc_at(q, off), sdesc_at(dK_k, off), idesc_s);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {       // dP = dO V^T
          const uint32_t off = (k / 4) * (FB_T * 128) + (k % 4) * 32;
          if (k == 0) umma_ss_cp<false>(leader, t_dp, sdesc_at(g, off), sdesc_at(dV_k, off), idesc_s);
          else umma_ss_cp<true>(leader, t_dp, sdesc_at(g, off), sdesc_at(dV_k, off), idesc_s);
        }
        umma_commit_p(leader, s_full);
      };
      auto issue_dv = [&](int st, int i) {       // dV += P^T dO : contraction over the 128 queries (tile rows)
        const SDesc g = stage(dDO_n0, st);
        umma_ss_p(leader, t_dv, sdesc_at(dP_m, 0), sdesc_at(g, 0), idesc_acc, i != 0);
#pragma unroll
        for (int k = 1; k < FB_T / 16; ++k) umma_ss_cp<true>(leader, t_dv, sdesc_at(dP_m, k * 2048), sdesc_at(g, k * 2048), idesc_acc);
      };
      auto issue_dk = [&](int st, int buf, int i) {   // dK += dS^T Q
        const SDesc q = stage(dQ_n0, st);
        const SDesc ds = SDesc{dDS_m0.lo + (uint32_t)buf * ((FB_T * FB_T * 2) >> 4), dDS_m0.hi};
        umma_ss_p(leader, t_dk, sdesc_at(ds, 0), sdesc_at(q, 0), idesc_acc, i != 0);
#pragma unroll
        for (int k = 1; k < FB_T / 16; ++k) umma_ss_cp<true>(leader, t_dk, sdesc_at(ds, k * 2048), sdesc_at(q, k * 2048), idesc_acc);
      };
      auto issue_dq = [&](int buf) {             // dQ = dS K : contraction over the 128 keys (tile columns)
        const SDesc ds = SDesc{dDS_k0.lo + (uint32_t)buf * ((FB_T * FB_T * 2) >> 4), dDS_k0.hi};
#pragma unroll
        for (int k = 0; k < FB_T / 16; ++k) {
          const uint32_t off = (k >> 2) * (FB_T * 128) + (k & 3) * 32;
          if (k == 0) umma_ss_cp<false>(leader, t_dq, sdesc_at(ds, off), sdesc_at(dK_n, 0), idesc_dq);
          else umma_ss_cp<true>(leader, t_dq, sdesc_at(ds, off), sdesc_at(dK_n, k * 2048), idesc_dq);
        }
      };
      bool ok = __all_sync(0xffffffffu, mbar_wait(kv_full, 0, abort_flag, p.status, 900));
      if (ok && OVERLAP) {
        // Pipelined order (head_dim 64).  When the softmax-gradient warps finish tile i the issuer queues
        //   dV(i) | S(i+1), dP(i+1) | dK(i), dQ(i)
        // so the warps start on tile i+1 as soon as its score products are done while dK(i) and dQ(i), which
        // read the double-buffered dS tile, still run on the tensor cores.  P is single-buffered: dV(i) is
        // ordered before S(i+1), whose completion is what lets the warps overwrite P.
        ok = __all_sync(0xffffffffu, mbar_wait(&q_full[0], 0, abort_flag, p.status, 901));
        if (ok) {
          tc_fence_after();
          issue_scores(0);
        }
        for (int i = 0; ok && i < n_it; ++i) {
          const int st = i % ST;
          if (!__all_sync(0xffffffffu, mbar_wait(p_full, i & 1, abort_flag, p.status, 903))) break;
          tc_fence_after();
          issue_dv(st, i);
          if (i + 1 < n_it) {
            const int sn = (i + 1) % ST;
            if (!__all_sync(0xffffffffu, mbar_wait(&q_full[sn], ((i + 1) / ST) & 1, abort_flag, p.status, 901))) break;
            tc_fence_after();
            issue_scores(sn);
          }
          issue_dk(st, i & 1, i);
          if (i > 0 && !__all_sync(0xffffffffu, mbar_wait(dq_empty, (i - 1) & 1, abort_flag, p.status, 904))) break;
          tc_fence_after();
          issue_dq(i & 1);
          umma_commit_p(leader, &q_empty[st]);
          umma_commit_p(leader, &ds_empty[i & 1]);
          umma_commit_p(leader, dq_full);
        }
      } else if (ok) {
        for (int i = 0; i < n_it; ++i) {
          const int st = i % ST;
          if (!__all_sync(0xffffffffu, mbar_wait(&q_full[st], (i / ST) & 1, abort_flag, p.status, 901))) break;
          if (DQ_ALIAS && i > 0 && !__all_sync(0xffffffffu, mbar_wait(dq_empty, (i - 1) & 1, abort_flag, p.status, 902))) break;
          tc_fence_after();
          issue_scores(st);
          if (!__all_sync(0xffffffffu, mbar_wait(p_full, i & 1, abort_flag, p.status, 903))) break;
          if (!DQ_ALIAS && i > 0 && !__all_sync(0xffffffffu, mbar_wait(dq_empty, (i - 1) & 1, abort_flag, p.status, 904))) break;
          tc_fence_after();
          issue_dv(st, i);
          issue_dk(st, 0, i);
          issue_dq(0);
          umma_commit_p(leader, &q_empty[st]);
          umma_commit_p(leader, dq_full);
        }
      }
      umma_commit_p(leader, acc_done);
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ softmax-gradient warps
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;                   // which 64 key columns of the tile this thread owns
    const int cbase = half * 64;
    const int r = quarter * 32 + lane;                  // query row inside the tile (epilogue: K/V row)
    const int kidx = k0 + r;                            // epilogue only: the K/V row this thread drains
    const bool k_valid = kidx < p.Tk;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    uint8_t* p_row = smem + L::PS_OFF + half * (FB_T * 128) + r * 128;
    uint8_t* ds_row0 = smem + L::DS_OFF + half * (FB_T * 128) + r * 128;
    const int kcol0 = k0 + cbase;                       // key index of this thread's first column
    bool alive = true;
    for (int i = 0; i < n_it && alive; ++i) {
      const int st = i % ST;
      bool ok = mbar_wait(&q_full[st], (i / ST) & 1, abort_flag, p.status, 1000) &&
                mbar_wait(s_full, i & 1, abort_flag, p.status, 1001);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { alive = false; break; }
      tc_fence_after();
      const float* vec = (const float*)(smem + L::VEC_OFF + st * 1536);
      const float lse2_r = vec[r], delta_r = vec[128 + r];
      const int qpos_r = ((const int*)vec)[256 + r], qpos_min = ((const int*)vec)[256];
      // slow path only for tiles that touch the causal diagonal or the end of the key sequence
      const bool need_mask = (k0 + FB_T > p.Tk) || (p.causal && (p.k_off + k0 + FB_T - 1 > qpos_min));
      const int kmax = min(p.causal ? qpos_r - p.k_off : 0x7fffffff, p.Tk - 1) - kcol0;   // last visible column of my span
      // 4 chunks of 16 columns; the tensor-memory loads of chunk ch+1 are in flight while chunk ch is processed.
      uint8_t* ds_row = ds_row0 + (OVERLAP ? (i & 1) * (FB_T * FB_T * 2) : 0);
      if (OVERLAP) {
        // this parity's dS buffer was last read by dK/dQ of tile i-2
        bool ok2 = mbar_wait(&ds_empty[i & 1], ((i >> 1) & 1) ^ 1, abort_flag, p.status, 1003);
        ok2 = __all_sync(0xffffffffu, ok2);
        if (!ok2) { alive = false; break; }
      }
      uint32_t sv[4][16], dpv[4][16];
      tmem_ld16(t_lane + S_COL + cbase, sv[0]);
      tmem_ld16(t_lane + DP_COL + cbase, dpv[0]);
      tmem_wait_ld();
      // two copies of the loop: the common one (no tile edge, not on the diagonal) carries no compare/select per element
      auto sweep = [&](auto masked_c) {
        constexpr bool MASKED = decltype(masked_c)::value;
  #pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          if (ch < 3) {
            tmem_ld16(t_lane + S_COL + cbase + 16 * (ch + 1), sv[ch + 1]);
            tmem_ld16(t_lane + DP_COL + cbase + 16 * (ch + 1), dpv[ch + 1]);
          }
          uint32_t pk[8], dk_[8];
  #pragma unroll
          for (int j = 0; j < 16; j += 2) {
            float p0 = ex2f(fmaf(__uint_as_float(sv[ch][j]), p.scale_log2, -lse2_r));
            float p1 = ex2f(fmaf(__uint_as_float(sv[ch][j + 1]), p.scale_log2, -lse2_r));
            if (MASKED) {
              if (ch * 16 + j > kmax) p0 = 0.f;
              if (ch * 16 + j + 1 > kmax) p1 = 0.f;
            }
            const float e0 = p0 * (__uint_as_float(dpv[ch][j]) - delta_r);
            const float e1 = p1 * (__uint_as_float(dpv[ch][j + 1]) - delta_r);
            pk[j >> 1] = pack_bf16(p0, p1);
            dk_[j >> 1] = pack_bf16(e0, e1);
          }
          // row r of P and dS -> shared memory, 128B-swizzled: 16-byte chunk (col % 64) / 8 of this thread's 64-key
          // group goes to chunk position (chunk ^ (r & 7)).
          *(uint4*)(p_row + (((2 * ch) ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *(uint4*)(p_row + (((2 * ch + 1) ^ (r & 7)) << 4)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          *(uint4*)(ds_row + (((2 * ch) ^ (r & 7)) << 4)) = make_uint4(dk_[0], dk_[1], dk_[2], dk_[3]);
          *(uint4*)(ds_row + (((2 * ch + 1) ^ (r & 7)) << 4)) = make_uint4(dk_[4], dk_[5], dk_[6], dk_[7]);
          if (ch < 3) tmem_wait_ld();
        }
      };
      if (need_mask) sweep(std::true_type{}); else sweep(std::false_type{});
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive_warp(p_full);
    }
    // final: dK, dV -> global
    if (n_it == 0) {
      if (!p.dkv_f32_accumulate && k_valid && half == 0) {
        __nv_bfloat16* dkr = (__nv_bfloat16*)p.dk + (((size_t)b * p.Tk + kidx) * p.Hkv + hkv) * D;
        __nv_bfloat16* dvr = (__nv_bfloat16*)p.dv + (((size_t)b * p.Tk + kidx) * p.Hkv + hkv) * D;
#pragma unroll
        for (int c = 0; c < D; c += 8) { *(uint4*)(dkr + c) = make_uint4(0, 0, 0, 0); *(uint4*)(dvr + c) = make_uint4(0, 0, 0, 0); }
      }
    } else if (alive) {
      bool ok = mbar_wait(acc_done, 0, abort_flag, p.status, 1002);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        const size_t off = (((size_t)b * p.Tk + (k_valid ? kidx : 0)) * p.Hkv + hkv) * D;
#pragma unroll 1
        for (int which = half; which <= half; ++which) {          // first warp group drains dK, second dV
          const uint32_t col = which ? DV_COL : DK_COL;
          void* base = which ? p.dv : p.dk;
          const float osc = which ? 1.f : p.scale;          // dS^T was accumulated without the softmax scale
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t v[32];
            tmem_ld32(t_lane + col + c, v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * osc);
            if (k_valid) {
              if (p.dkv_f32_accumulate == 2) {
                const int ch = kidx / p.route_rows, lrow = kidx % p.route_rows;
                float* dst = (float*)(which ? p.route_v[ch] : p.route_k[ch]) +
                             (((size_t)b * p.route_tl + lrow) * p.Hkv + hkv) * D + c;
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  red_add_v4(dst + j, __uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
              } else if (p.dkv_f32_accumulate) {
                float* dst = (float*)base + off + c;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  float4 o = *(float4*)(dst + j);
                  o.x += __uint_as_float(v[j]); o.y += __uint_as_float(v[j + 1]);
                  o.z += __uint_as_float(v[j + 2]); o.w += __uint_as_float(v[j + 3]);
                  *(float4*)(dst + j) = o;
                }
              } else {
                __nv_bfloat16* dst = (__nv_bfloat16*)base + off + c;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  uint4 o;
                  o.x = pack_bf16(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                  o.y = pack_bf16(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                  o.z = pack_bf16(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                  o.w = pack_bf16(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                  *(uint4*)(dst + j) = o;
                }
              }
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ dQ drain warps (10..13)
    // tensor memory -> registers -> 128B-swizzled fp32 staging tile -> TMA reduce-add into the global fp32 dQ
    // (rows past the end of the sequence are clipped by the tensor map).
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                  // query row inside the tile
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    uint8_t* stage = smem + L::DQS_OFF;
    const bool issuer = (warp == 10 && lane == 0);
    if (issuer) tma_prefetch_desc(&tmDQ);
    for (int i = 0; i < n_it; ++i) {
      bool ok = mbar_wait(dq_full, i & 1, abort_flag, p.status, 1100);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int hq = hkv * G + i / n_qt;
      const int q0 = (qt_start + i % n_qt) * FB_T;
      constexpr int NB = L::DQ_BOXES;
#pragma unroll 1
      for (int rnd = 0; rnd < D / (32 * NB); ++rnd) {   // NB boxes of 128 x 32 fp32 per round through the staging tile
#pragma unroll
        for (int bx = 0; bx < NB; ++bx) {
          uint32_t v[32];
          tmem_ld32(t_lane + DQ_COL + (rnd * NB + bx) * 32, v);
          tmem_wait_ld();
          uint8_t* rowp = stage + bx * (FB_T * 128) + r * 128;
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4)        // dS was formed without the softmax scale: apply it here
            *(float4*)(rowp + ((c4 ^ (r & 7)) << 4)) = make_float4(__uint_as_float(v[4 * c4]) * p.scale, __uint_as_float(v[4 * c4 + 1]) * p.scale,
                                                                   __uint_as_float(v[4 * c4 + 2]) * p.scale, __uint_as_float(v[4 * c4 + 3]) * p.scale);
        }
        if (rnd == D / (32 * NB) - 1) { tc_fence_before(); mbar_arrive_warp(dq_empty); }   // tensor-memory dQ is free again
        fence_proxy_async_smem();
        asm volatile("bar.sync 5, 128;" ::: "memory");
        if (issuer && !p.debug_skip_dq) {
#pragma unroll
          for (int bx = 0; bx < NB; ++bx)
            asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                         ::"l"((uint64_t)&tmDQ), "r"(smem_u32(stage + bx * (FB_T * 128))), "r"((rnd * NB + bx) * 32), "r"(hq), "r"(q0), "r"(b)
                         : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        }
        asm volatile("bar.sync 5, 128;" ::: "memory");                             // staging may be overwritten
      }
    }
    if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// delta[b,h,t] = sum_d dO*O ; lse2 = lse*log2(e) ; padding rows get delta 0 / lse2 +inf.  One warp per row.
template <int D>
__global__ void bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                const float* __restrict__ lse, float* __restrict__ delta, float* __restrict__ lse2,
                                int B, int Tq, int Hq, int Tq_pad) {
  const int lane = threadIdx.x & 31;
  const size_t nrow = (size_t)B * Hq * Tq_pad;
  for (size_t w = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5); w < nrow; w += (size_t)gridDim.x * (blockDim.x >> 5)) {
    const int t = (int)(w % Tq_pad);
    const int h = (int)((w / Tq_pad) % Hq);
    const int b = (int)(w / ((size_t)Tq_pad * Hq));
    if (t >= Tq) {
      if (lane == 0) { if (delta) delta[w] = 0.f; if (lse2) lse2[w] = INFINITY; }
      continue;
    }
    if (delta) {
      const size_t off = (((size_t)b * Tq + t) * Hq + h) * D;
      float s = 0.f;
#pragma unroll
      for (int e = lane * 2; e < D; e += 64) {
        const uint32_t a = *(const uint32_t*)(o + off + e), g = *(const uint32_t*)(dout + off + e);
        s += bf16_lo(a) * bf16_lo(g) + bf16_hi(a) * bf16_hi(g);
      }
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
      if (lane == 0) delta[w] = s;
    }
    if (lse2 && lane == 0) {
      const float l = lse[((size_t)b * Hq + h) * Tq + t];
      lse2[w] = (l == -INFINITY) ? INFINITY : l * 1.4426950408889634f;
    }
  }
}

static int make_tmap4(CUtensorMap* m, const void* ptr, int D, int H, int T, int B, long s_head, long s_tok, long s_batch) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)T, (uint64_t)B};
  uint64_t strides[4] = {0, (uint64_t)s_head * 2, (uint64_t)s_tok * 2, (uint64_t)s_batch * 2};
  uint32_t box[4] = {64, 1, (uint32_t)FB_T, 1};
  return encode_tmap(m, ptr, 2, 4, dims, strides, box, 1);
}

}  // namespace cpb

using namespace cpb;

// o and dout are contiguous [B,Tq,Hq,D]; delta/lse2 are [B,Hq,Tq_pad] with Tq_pad = ceil(Tq/128)*128.
// Either output may be null (then its inputs are not read): the Ulysses backward computes delta where the
// tokens live and lse2 where the heads live.
extern "C" int cpb_flash_bwd_prep(const void* o, const void* dout, const float* lse, float* delta, float* lse2,
                                  int B, int Tq, int Hq, int D, int Tq_pad, cudaStream_t stream) {
  const size_t nrow = (size_t)B * Hq * Tq_pad;
  size_t g = (nrow + 7) / 8;
  const size_t cap = (size_t)sm_count() * 16;
  if (g > cap) g = cap;
  if (D == 64) bwd_prep_kernel<64><<<(int)g, 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse, delta, lse2, B, Tq, Hq, Tq_pad);
  else if (D == 128) bwd_prep_kernel<128><<<(int)g, 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse, delta, lse2, B, Tq, Hq, Tq_pad);
  else return set_error(CPB_ERR_ARG, "flash_bwd_prep: head_dim %d not in {64,128}", D);
  return check_launch("flash_bwd_prep");
}

// q,k,v: strided views (element strides: head, token, batch); dout contiguous [B,Tq,Hq,D].
// dq: fp32 [B,Tq,Hq,D] (accumulated; caller zeroes).  dk/dv: [B,Tk,Hkv,D] bf16 (written) or fp32 (+=).
// q_pos: int32 [Tq_pad] (INT_MAX padding) -- required.
extern "C" int cpb_flash_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse2,
                             const float* delta, float* dq, void* dk, void* dv,
                             int B, int Tq, int Tk, int Hq, int Hkv, int D, int Tq_pad,
                             long q_sh, long q_st, long q_sb, long k_sh, long k_st, long k_sb,
                             float scale, int causal, int k_off, const int* q_pos, int dkv_f32_accumulate,
                             const uint64_t* route_k, const uint64_t* route_v, int route_rows, int route_tl,
                             int* status, cudaStream_t stream) {
  if (D != 64 && D != 128) return set_error(CPB_ERR_ARG, "flash_bwd: head_dim %d not in {64,128}", D);
  if (Hq % Hkv) return set_error(CPB_ERR_ARG, "flash_bwd: Hq %% Hkv != 0");
  if (Tq_pad % FB_T || Tq_pad < Tq) return set_error(CPB_ERR_ARG, "flash_bwd: bad Tq_pad");
  if (q_pos == nullptr) return set_error(CPB_ERR_ARG, "flash_bwd: q_pos is required");
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_tmap4(&tq, q, D, Hq, Tq, B, q_sh, q_st, q_sb)) != CPB_OK) return rc;
  if ((rc = make_tmap4(&tk, k, D, Hkv, Tk, B, k_sh, k_st, k_sb)) != CPB_OK) return rc;
  if ((rc = make_tmap4(&tv, v, D, Hkv, Tk, B, k_sh, k_st, k_sb)) != CPB_OK) return rc;
  if ((rc = make_tmap4(&tdo, dout, D, Hq, Tq, B, D, (long)Hq * D, (long)Tq * Hq * D)) != CPB_OK) return rc;
  CUtensorMap tdq;
  {
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hq, (uint64_t)Tq, (uint64_t)B};
    uint64_t strides[4] = {0, (uint64_t)D * 4, (uint64_t)Hq * D * 4, (uint64_t)Tq * Hq * D * 4};
    uint32_t box[4] = {32, 1, (uint32_t)FB_T, 1};
    if ((rc = encode_tmap(&tdq, dq, 4, 4, dims, strides, box, 1)) != CPB_OK) return rc;
  }
  BwdParams p;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hkv = Hkv; p.Tq_pad = Tq_pad; p.causal = causal; p.k_off = k_off;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse2 = lse2; p.delta = delta; p.q_pos = q_pos; p.dq = dq; p.dk = dk; p.dv = dv;
  p.dkv_f32_accumulate = dkv_f32_accumulate; p.status = status;
  p.route_k = route_k; p.route_v = route_v; p.route_rows = route_rows; p.route_tl = route_tl;
  // diagnostic switch, read once per process and announced when set
  static const bool skip_dq = [] {
    const char* e = getenv("CPB_BWD_SKIP_DQ");
    const bool on = e != nullptr && e[0] == '1';
    if (on) fprintf(stderr, "CPB_BWD_SKIP_DQ=1: the attention backward does NOT produce dQ (timing experiment only)\n");
    return on;
  }();
  p.debug_skip_dq = skip_dq;
  if (dkv_f32_accumulate == 2 && (route_k == nullptr || route_v == nullptr || route_rows <= 0))
    return set_error(CPB_ERR_ARG, "flash_bwd: routed dK/dV needs route tables");
  dim3 grid((Tk + FB_T - 1) / FB_T, Hkv, B);
  if (D == 64) {
    static bool cfg = false;
    if (!cfg) { CPB_CUDA_OK(cudaFuncSetAttribute(flash_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<64>::TOTAL)); cfg = true; }
    flash_bwd_kernel<64><<<grid, FB_THREADS, BwdSmem<64>::TOTAL, stream>>>(tq, tk, tv, tdo, tdq, p);
  } else {
    static bool cfg = false;
    if (!cfg) { CPB_CUDA_OK(cudaFuncSetAttribute(flash_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<128>::TOTAL)); cfg = true; }
    flash_bwd_kernel<128><<<grid, FB_THREADS, BwdSmem<128>::TOTAL, stream>>>(tq, tk, tv, tdo, tdq, p);
  }
  return check_launch("flash_bwd");
}
