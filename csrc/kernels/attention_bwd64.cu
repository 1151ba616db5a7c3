// Flash-attention backward specialised for head_dim 64 (the flagship 1B shape and GPT-2).
//
// At head_dim 64 the general kernel (attention_bwd.cu) is bound by shared-memory bandwidth: three of its
// five products read a 128x128 bf16 A tile from shared memory for only 64 output columns.  This kernel
// keeps the K/V rows in tensor-memory lanes instead (S^T = K Q^T, dP^T = V dO^T), so P^T and dS^T are
// tensor-memory A operands of the dV / dK products, and removes every per-column vector from the inner loop
// by folding them into the tensor-core products:
//
//     S'^T  = K Q^T   - 1 (x) L^T        L[q]     = LSE[q] / scale   (three bf16 terms: hi + mid + lo)
//     dP'^T = V dO^T  - 1 (x) Delta^T    Delta[q] = rowsum(dO o O)   (three bf16 terms)
//
// as one extra K=16 UMMA each, whose A operand is a constant tile of ones and whose B operand is a
// [128 queries x 8] bf16 tile produced by `bwd64_aug_kernel` and loaded with one bulk copy.  Then
//     P^T = exp2(S'^T * scale*log2e)        dS^T = P^T o dP'^T            (no loads, no subtraction)
//     dV += P^T dO  (A in tensor memory)    dK += dS^T Q  (A in tensor memory)
//     dQ  = dS K    (A = dS^T staged M-major in shared memory) -> TMA reduce-add into the fp32 dQ buffer.
//
// Issue order of the MMA warp (tile i = one 128x128 query/key tile pair):
//     S'(i+1) as soon as the warps have read S'(i);   then after the warps finish tile i:
//     dK(i), dP'(i+1), dV(i), dQ(i)
// so the exponentials of tile i+1 overlap the gradient products of tile i, and dP'(i+1) is ready long before the
// warps want it.  The warps keep P^T and dS^T in registers until dQ(i-1) has finished and store them at the end of
// the tile: two barrier waits in the middle of a tile, one at its end.  Tensor memory (512 columns):
// S'^T 128 | dP'^T 128 (dS^T bf16 written back into it) | dV 64 | dK 64 | dQ 64 | P^T 64.
//
// Same interface, masking rules, dK/dV output modes and bounded waits as the general kernel.
#include "common.cuh"
#include "host_utils.h"

#include <stdio.h>
#include <stdlib.h>

namespace cpb {

// Diagnostics (cycle counters and an event timeline of CTA (0,0,0), tiles 64..71) are compiled in only with
// -DCPB_BWD64_PROF; without it the predicates below are constant false and the code disappears.
#ifdef CPB_BWD64_PROF
#define B64_PROF_ON(x) (x)
#else
#define B64_PROF_ON(x) false
#endif
// diagnostic timeline: CTA (0,0,0), tiles 64..71: event e of tile t -> prof[16 + (t-64)*32 + e]
#define B64_STAMP(cond, t, e) do { if ((cond) && (t) >= 64 && (t) < 72) p.prof[16 + ((t) - 64) * 32 + (e)] = clock64(); } while (0)

constexpr int B64_T = 128;
constexpr int B64_D = 64;
// Warps: 0 = TMA loader, 1 = MMA issuer, then 4*NG softmax-gradient warps (NG column groups of 128/NG queries; a warp
// can only touch the 32 tensor-memory lanes of its quarter, so every group has four warps), then 4 dQ drain warps.
constexpr int b64_threads(int ng) { return 64 + 128 * ng + 128; }
constexpr int B64_NG = 4;          // column groups of the softmax-gradient warps (2: 64 queries per thread, 4: 32)
constexpr int B64_POLY = 0;        // share (of 8) of the exponentials computed on the FMA pipe: measured neutral (846 to 855 TFLOP/s for 0..4), kept off

static __device__ long long g_bwd64_prof[16 + 32 * 8];

struct Bwd64Params {
  int B, Tq, Tk, Hq, Hkv, Tq_pad;
  int causal, k_off;
  float scale, scale_log2;
  const __nv_bfloat16* aug_l;   // [B,Hq,Tq_pad,8]  (-L_hi, -L_mid, -L_lo, 0...)
  const __nv_bfloat16* aug_d;   // [B,Hq,Tq_pad,8]  (-Delta_hi, -Delta_mid, -Delta_lo, 0...)
  const int* q_pos;             // [Tq_pad]
  void* dk; void* dv;
  int dkv_mode;                 // 0 bf16 store, 1 fp32 accumulate, 2 routed red.add (fused ring)
  const uint64_t* route_k;
  const uint64_t* route_v;
  int route_rows, route_tl;
  int debug_skip_dq;
  long long* prof;              // diagnostic: CTA (0,0,0) writes cycle breakdowns here (16 counters)
  int* status;
};

struct Bwd64Smem {
  static constexpr int TILE = B64_T * B64_D * 2;          // 16 KB
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE;
  static constexpr int NST = 3;                           // Q / dO ring depth: a stage is released only when dQ of its tile
                                                          // has finished, and S' of the tile after next wants to start then
  static constexpr int Q_OFF = 2 * TILE;
  static constexpr int DO_OFF = Q_OFF + NST * TILE;
  static constexpr int DS_OFF = DO_OFF + NST * TILE;      // dS^T 128 keys x 128 queries bf16 (32 KB)
  static constexpr int DQS_OFF = DS_OFF + 32768;          // dQ staging: per drain warp two boxes of 32 rows x 32 fp32 (4 x 8 KB)
  static constexpr int ONES_OFF = DQS_OFF + 32768;        // [128 x 8] bf16 (1,1,1,0,...)           2 KB
  static constexpr int AUGL_OFF = ONES_OFF + 2048;        // NST x 2 KB
  static constexpr int AUGD_OFF = AUGL_OFF + NST * 2048;  // NST x 2 KB
  static constexpr int ZERO_OFF = AUGD_OFF + NST * 2048;        // zero block: second K chunk of every augmenting tile (after them: offsets > 0)
  static constexpr int QPOS_OFF = ZERO_OFF + 2048;        // NST x 512 B
  static constexpr int BAR_OFF = QPOS_OFF + NST * 512;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

// K-major operand without swizzle: core matrices of 8 rows x 16 bytes; the two 16-byte K chunks of a K=16 step are
// `lbo` bytes apart, successive 8-row groups `sbo` bytes apart.
__device__ __forceinline__ uint64_t make_sdesc_noswz(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;       // version
  return d;                     // layout type 0: no swizzle
}

__device__ __forceinline__ void bulk_load_1d_64(void* smem, const void* gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem)), "l"((uint64_t)gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// A global load that stays where it is written (the compiler would otherwise sink it to its first use, one tile later).
__device__ __forceinline__ int ld_pinned_s32(const int* ptr) {
  int v;
  asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(v) : "l"(ptr));
  return v;
}
__device__ __forceinline__ void red_add_v4_64(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// POLY: of the 8 column pairs of every 16-column group of an unmasked tile, the last POLY take their exponentials from
// exp2_poly_f32x2 (FMA pipe) and the others from ex2.approx (special-function unit).
template <int POLY, int NG>
__global__ void __launch_bounds__(b64_threads(NG), 1)
flash_bwd64_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmDQ, Bwd64Params p) {
  using L = Bwd64Smem;
  constexpr int D = B64_D;
  constexpr int CW = B64_T / NG;            // query columns per softmax-gradient thread
  constexpr int NCH = CW / 16;              // 16-column groups per thread
  constexpr uint32_t ST_COL = 0, DPT_COL = 128, DV_COL = 256, DK_COL = 320, DQ_COL = 384, PT_COL = 448;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + L::BAR_OFF);
  uint64_t* kv_full = bars + 0;
  constexpr int NST = L::NST;
  uint64_t* q_full = bars + 1;        // [NST]
  uint64_t* q_empty = bars + 4;       // [NST]
  uint64_t* s_ready = bars + 7;
  uint64_t* s_consumed = bars + 8;
  uint64_t* dp_ready = bars + 9;
  uint64_t* p_full = bars + 11;
  uint64_t* dq_full = bars + 12;
  uint64_t* dq_empty = bars + 13;
  uint64_t* acc_done = bars + 14;
  uint32_t* tmem_slot = (uint32_t*)(bars + 16);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* qt_start_s = (int*)(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int k0 = kt * B64_T;
  const int num_q_tiles = p.Tq_pad / B64_T;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < NST; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    mbar_init(s_ready, 1); mbar_init(s_consumed, 4 * NG); mbar_init(dp_ready, 1);
    mbar_init(p_full, 4 * NG); mbar_init(dq_full, 1); mbar_init(dq_empty, 4); mbar_init(acc_done, 1);
    *abort_flag = 0;
    *qt_start_s = num_q_tiles;
    fence_mbar_init();
  }
  // constant augmenting operands: ones tile (first three of eight K elements) and the zero block
  for (int i = threadIdx.x; i < 128; i += blockDim.x) {
    uint32_t one2 = 0x3F803F80u;      // (1.0bf16, 1.0bf16)
    *(uint4*)(smem + L::ONES_OFF + i * 16) = make_uint4(one2, 0x00003F80u, 0u, 0u);
    *(uint4*)(smem + L::ZERO_OFF + i * 16) = make_uint4(0u, 0u, 0u, 0u);
  }
  fence_proxy_async_smem();
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (p.causal) {
    const int kpos_min = p.k_off + k0;
    for (int t = threadIdx.x; t < num_q_tiles; t += blockDim.x) {
      const int last = min(t * B64_T + B64_T, p.Tq) - 1;
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
      tma_load_4d(smem + L::K_OFF, &tmK, kv_full, 0, hkv, k0, b);
      tma_load_4d(smem + L::V_OFF, &tmV, kv_full, 0, hkv, k0, b);
      for (int i = 0; i < n_it; ++i) {
        const int st = i % NST;
        const uint32_t ph = (i / NST) & 1;
        if (!mbar_wait(&q_empty[st], ph ^ 1, abort_flag, p.status, 800)) break;
        const int hq = hkv * G + i / n_qt;
        const int q0 = (qt_start + i % n_qt) * B64_T;
        mbar_expect_tx(&q_full[st], 2 * L::TILE + 2 * 2048 + 512);
        tma_load_4d(smem + L::Q_OFF + st * L::TILE, &tmQ, &q_full[st], 0, hq, q0, b);
        tma_load_4d(smem + L::DO_OFF + st * L::TILE, &tmDO, &q_full[st], 0, hq, q0, b);
        const size_t row_off = ((size_t)b * p.Hq + hq) * p.Tq_pad + q0;
        bulk_load_1d_64(smem + L::AUGL_OFF + st * 2048, p.aug_l + row_off * 8, 2048, &q_full[st]);
        bulk_load_1d_64(smem + L::AUGD_OFF + st * 2048, p.aug_d + row_off * 8, 2048, &q_full[st]);
        bulk_load_1d_64(smem + L::QPOS_OFF + st * 512, p.q_pos + q0, 512, &q_full[st]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs this code convergently; only the elected lane issues the MMAs and commits.
    if (n_it > 0) {
      const uint32_t leader = elect_one() ? 1u : 0u;
      constexpr uint32_t idesc_s = make_idesc_bf16(B64_T, B64_T, false, false);    // S'^T, dP'^T (and their augmenting steps)
      constexpr uint32_t idesc_acc = make_idesc_bf16(B64_T, D, false, true);       // dV, dK: A in tensor memory, B N-major
      constexpr uint32_t idesc_dq = make_idesc_bf16(B64_T, D, true, true);         // dQ: A M-major smem, B N-major
      // descriptor bases, built once; per MMA only the start-address field is stepped
      const uint32_t sOnes = smem_u32(smem + L::ONES_OFF), sZero = smem_u32(smem + L::ZERO_OFF);
      const uint32_t sAL = smem_u32(smem + L::AUGL_OFF), sAD = smem_u32(smem + L::AUGD_OFF);
      const SDesc dK_k = sdesc_split(sdesc_kmajor(smem_u32(smem + L::K_OFF)));                       // K as K-major A (scores)
      const SDesc dV_k = sdesc_split(sdesc_kmajor(smem_u32(smem + L::V_OFF)));
      const SDesc dQ_k = sdesc_split(sdesc_kmajor(smem_u32(smem + L::Q_OFF)));                       // stage 0; stage st: + st * TILE
      const SDesc dDO_k = sdesc_split(sdesc_kmajor(smem_u32(smem + L::DO_OFF)));
      const SDesc dQ_n = sdesc_split(make_sdesc(smem_u32(smem + L::Q_OFF), B64_T * 128, 1024));      // Q / dO / K as N-major B
      const SDesc dDO_n = sdesc_split(make_sdesc(smem_u32(smem + L::DO_OFF), B64_T * 128, 1024));
      const SDesc dK_n = sdesc_split(make_sdesc(smem_u32(smem + L::K_OFF), B64_T * 128, 1024));
      const SDesc dDS_m = sdesc_split(make_sdesc(smem_u32(smem + L::DS_OFF), B64_T * 128, 1024));    // dS^T as M-major A
      const uint64_t d_ones = make_sdesc_noswz(sOnes, sZero - sOnes, 128);
      // augmenting tiles: the zero block lies NST * 2048 (lse) resp. fewer bytes behind stage 0; stepping the stage moves
      // the start address forward and the leading offset back by the same amount
      const uint32_t t_s = tmem_base + ST_COL, t_dp = tmem_base + DPT_COL, t_dv = tmem_base + DV_COL, t_dk = tmem_base + DK_COL,
                     t_dq = tmem_base + DQ_COL, t_pt = tmem_base + PT_COL;
      auto issue_s = [&](int st) {          // S'^T = K Q^T - 1 (x) L^T
        const SDesc q = SDesc{dQ_k.lo + st * (L::TILE >> 4), dQ_k.hi};
        const uint32_t sA = sAL + st * 2048;
        umma_ss_cp<false>(leader, t_s, sdesc_at(dK_k, 0), sdesc_at(q, 0), idesc_s);
        umma_ss_cp<true>(leader, t_s, sdesc_at(dK_k, 32), sdesc_at(q, 32), idesc_s);
        umma_ss_cp<true>(leader, t_s, sdesc_at(dK_k, 64), sdesc_at(q, 64), idesc_s);
        umma_ss_cp<true>(leader, t_s, sdesc_at(dK_k, 96), sdesc_at(q, 96), idesc_s);
        umma_ss_cp<true>(leader, t_s, d_ones, make_sdesc_noswz(sA, sZero - sA, 128), idesc_s);
        umma_commit_p(leader, s_ready);
      };
      auto issue_dp = [&](int st) {         // dP'^T = V dO^T - 1 (x) Delta^T
        const SDesc g = SDesc{dDO_k.lo + st * (L::TILE >> 4), dDO_k.hi};
        const uint32_t sA = sAD + st * 2048;
        umma_ss_cp<false>(leader, t_dp, sdesc_at(dV_k, 0), sdesc_at(g, 0), idesc_s);
        umma_ss_cp<true>(leader, t_dp, sdesc_at(dV_k, 32), sdesc_at(g, 32), idesc_s);
        umma_ss_cp<true>(leader, t_dp, sdesc_at(dV_k, 64), sdesc_at(g, 64), idesc_s);
        umma_ss_cp<true>(leader, t_dp, sdesc_at(dV_k, 96), sdesc_at(g, 96), idesc_s);
        umma_ss_cp<true>(leader, t_dp, d_ones, make_sdesc_noswz(sA, sZero - sA, 128), idesc_s);
        umma_commit_p(leader, dp_ready);
      };
      const bool wr_prof = B64_PROF_ON(p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0);
      bool ok = __all_sync(0xffffffffu, mbar_wait(kv_full, 0, abort_flag, p.status, 900) && mbar_wait(&q_full[0], 0, abort_flag, p.status, 901));
      if (ok) {
        tc_fence_after();
        issue_s(0);
        issue_dp(0);
      }
      for (int i = 0; ok && i < n_it; ++i) {
        const int st = i % NST;
        const SDesc qn = SDesc{dQ_n.lo + st * (L::TILE >> 4), dQ_n.hi}, gn = SDesc{dDO_n.lo + st * (L::TILE >> 4), dDO_n.hi};
        if (i + 1 < n_it) {
          // the warps have read S'(i): the next score tile can be produced while they work on tile i
          if (!__all_sync(0xffffffffu, mbar_wait(s_consumed, i & 1, abort_flag, p.status, 902))) break;
          B64_STAMP(wr_prof, i, 0);
          if (!__all_sync(0xffffffffu, mbar_wait(&q_full[(i + 1) % NST], ((i + 1) / NST) & 1, abort_flag, p.status, 903))) break;
          tc_fence_after();
          B64_STAMP(wr_prof, i, 1);
          issue_s((i + 1) % NST);
          B64_STAMP(wr_prof, i, 2);
        }
        if (!__all_sync(0xffffffffu, mbar_wait(p_full, i & 1, abort_flag, p.status, 904))) break;
        tc_fence_after();
        B64_STAMP(wr_prof, i, 3);
        umma_ts_p(leader, t_dk, t_dp, sdesc_at(qn, 0), idesc_acc, i != 0);            // dK += dS^T Q  (frees the dS^T alias)
#pragma unroll
        for (int k = 1; k < B64_T / 16; ++k)
          umma_ts_cp<true>(leader, t_dk, t_dp + ((16 * k) / CW) * CW + (((16 * k) % CW) / 16) * 8, sdesc_at(qn, k * 2048), idesc_acc);
        B64_STAMP(wr_prof, i, 4);
        if (i + 1 < n_it) issue_dp((i + 1) % NST);                                     // dP'(i+1): early, off the warps' critical path
        B64_STAMP(wr_prof, i, 5);
        umma_ts_p(leader, t_dv, t_pt, sdesc_at(gn, 0), idesc_acc, i != 0);            // dV += P^T dO
#pragma unroll
        for (int k = 1; k < B64_T / 16; ++k)
          umma_ts_cp<true>(leader, t_dv, t_pt + k * 8, sdesc_at(gn, k * 2048), idesc_acc);
        umma_commit_p(leader, &q_empty[st]);    // Q(i), dO(i) and their vectors are free
        B64_STAMP(wr_prof, i, 6);
        if (i > 0 && !__all_sync(0xffffffffu, mbar_wait(dq_empty, (i - 1) & 1, abort_flag, p.status, 905))) break;
        tc_fence_after();
        B64_STAMP(wr_prof, i, 7);
        umma_ss_cp<false>(leader, t_dq, sdesc_at(dDS_m, 0), sdesc_at(dK_n, 0), idesc_dq);      // dQ = dS K
#pragma unroll
        for (int k = 1; k < B64_T / 16; ++k)
          umma_ss_cp<true>(leader, t_dq, sdesc_at(dDS_m, k * 2048), sdesc_at(dK_n, k * 2048), idesc_dq);
        umma_commit_p(leader, dq_full);         // also: dV(i) has read P^T, dQ(i) the shared-memory dS^T
        B64_STAMP(wr_prof, i, 8);
      }
      umma_commit_p(leader, acc_done);
#ifdef CPB_BWD64_PROF
      if (wr_prof) p.prof[15] = n_it;
#endif
    }
  } else if (warp >= 2 && warp < 2 + 4 * NG) {
    // ------------------------------------------------------------------ softmax-gradient warps (thread = key row, CW queries)
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;                    // which CW query columns of the tile this thread owns
    const int cbase = grp * CW;
    const int r = quarter * 32 + lane;                  // key row inside the tile
    const int kidx = k0 + r;
    const bool k_valid = kidx < p.Tk;
    const int kpos = p.k_off + kidx;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    // dS^T in shared memory: two [128 keys x 64 queries] halves, 128-byte swizzled rows; this thread's queries start at
    // 16-byte chunk `chunk0` of its row in half cbase / 64
    uint8_t* ds_row = smem + L::DS_OFF + (cbase / 64) * (B64_T * 128) + r * 128;
    constexpr int DS_CHUNKS = CW / 8;
    const int chunk0 = (cbase % 64) / 8;
    bool alive = true;
    const bool wprof = B64_PROF_ON(p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 64);
    // first query position of a tile decides whether it needs masking; read one tile ahead, straight from global memory
    int qmin_next = n_it > 0 ? ld_pinned_s32(p.q_pos + qt_start * B64_T) : 0;
    for (int i = 0; i < n_it && alive; ++i) {
      const int st = i % NST;
      const int qmin = qmin_next;
      if (i + 1 < n_it) qmin_next = ld_pinned_s32(p.q_pos + (qt_start + (i + 1) % n_qt) * B64_T);
      // slow path only for tiles that touch the causal diagonal or the end of the key sequence
      const bool need_mask = (k0 + B64_T > p.Tk) || (p.causal && (p.k_off + k0 + B64_T - 1 > qmin));
      B64_STAMP(wprof, i, 16);
      bool ok = mbar_wait(s_ready, i & 1, abort_flag, p.status, 1001);
      B64_STAMP(wprof, i, 17);
      if (need_mask) ok = ok && mbar_wait(&q_full[st], (i / NST) & 1, abort_flag, p.status, 1000);   // query positions in shared memory
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { alive = false; break; }
      tc_fence_after();
      B64_STAMP(wprof, i, 9);
      const int* qpos = (const int*)(smem + L::QPOS_OFF + st * 512);
      uint32_t sv[NCH][16];
#pragma unroll
      for (int ch = 0; ch < NCH; ++ch) tmem_ld16(t_lane + ST_COL + cbase + 16 * ch, sv[ch]);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive_warp(s_consumed);                         // the next score tile may overwrite S'^T
      uint32_t pk[CW / 2];                              // P^T of this thread's queries, bf16 pairs
      if (!need_mask) {
        const uint64_t c2 = pack_f32x2(p.scale_log2, p.scale_log2);
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            if ((j >> 1) >= 8 - POLY) {                 // resolved at compile time (the loops are unrolled)
              float p0, p1;
              unpack_f32x2(exp2_poly_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(sv[ch][j]), __uint_as_float(sv[ch][j + 1])), c2)), p0, p1);
              pk[ch * 8 + (j >> 1)] = pack_bf16(p0, p1);
            } else {
              pk[ch * 8 + (j >> 1)] = pack_bf16(ex2f(__uint_as_float(sv[ch][j]) * p.scale_log2), ex2f(__uint_as_float(sv[ch][j + 1]) * p.scale_log2));
            }
          }
      } else {
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const int c = cbase + ch * 16 + j;
            const bool v0 = k_valid && (!p.causal || kpos <= qpos[c]), v1 = k_valid && (!p.causal || kpos <= qpos[c + 1]);
            const float p0 = v0 ? ex2f(__uint_as_float(sv[ch][j]) * p.scale_log2) : 0.f;
            const float p1 = v1 ? ex2f(__uint_as_float(sv[ch][j + 1]) * p.scale_log2) : 0.f;
            pk[ch * 8 + (j >> 1)] = pack_bf16(p0, p1);
          }
      }
      // dp_ready(i): dP'(i) is complete, and so is dK(i-1), which read the previous dS^T alias inside the dP'^T columns
      bool ok3 = mbar_wait(dp_ready, i & 1, abort_flag, p.status, 1004);
      ok3 = __all_sync(0xffffffffu, ok3);
      if (!ok3) { alive = false; break; }
      tc_fence_after();
      B64_STAMP(wprof, i, 12);
      // dS^T = P^T o dP'^T with the bf16-rounded P (the value dV is computed from), kept packed in registers
      uint32_t dsk[CW / 2];
      {
        uint32_t dpv[2][16];
        tmem_ld16(t_lane + DPT_COL + cbase, dpv[0]);
        tmem_wait_ld();
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          if (ch < NCH - 1) tmem_ld16(t_lane + DPT_COL + cbase + 16 * (ch + 1), dpv[(ch + 1) & 1]);
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const uint32_t pp = pk[ch * 8 + (j >> 1)];
            dsk[ch * 8 + (j >> 1)] = pack_bf16(bf16_lo(pp) * __uint_as_float(dpv[ch & 1][j]), bf16_hi(pp) * __uint_as_float(dpv[ch & 1][j + 1]));
          }
          if (ch < NCH - 1) tmem_wait_ld();
        }
      }
      // dq_full(i-1): dV(i-1) has read the previous P^T and dQ(i-1) the previous dS^T in shared memory
      if (i > 0) {
        bool ok4 = mbar_wait(dq_full, (i - 1) & 1, abort_flag, p.status, 1005);
        ok4 = __all_sync(0xffffffffu, ok4);
        if (!ok4) { alive = false; break; }
        tc_fence_after();
      }
      // P^T -> its own columns (A operand of dV); dS^T -> the front half of this thread's dP'^T span (A operand of dK: the
      // k-step of queries 16k.. sits at columns (16k / CW) * CW + ((16k % CW) / 16) * 8) and -> shared memory (row = key,
      // 64 queries per 128-byte swizzled row; M-major A of dQ)
      B64_STAMP(wprof, i, 14);
      if constexpr (CW == 64) {
        tmem_st32(t_lane + PT_COL + cbase / 2, pk);
        tmem_st32(t_lane + DPT_COL + cbase, dsk);
      } else {
        tmem_st16(t_lane + PT_COL + cbase / 2, pk);
        tmem_st16(t_lane + DPT_COL + cbase, dsk);
      }
#pragma unroll
      for (int c8 = 0; c8 < DS_CHUNKS; ++c8)
        *(uint4*)(ds_row + (((chunk0 + c8) ^ (r & 7)) << 4)) = make_uint4(dsk[4 * c8], dsk[4 * c8 + 1], dsk[4 * c8 + 2], dsk[4 * c8 + 3]);
      tmem_wait_st();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive_warp(p_full);
      B64_STAMP(wprof, i, 15);
    }
    // final: dK, dV -> global
    if (n_it == 0) {
      if (p.dkv_mode == 0 && k_valid && grp == 0) {
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
        const int which = grp >= NG / 2;                 // the first half of the warp groups drains dK, the second dV
        constexpr int DCOLS = D / (NG / 2);              // accumulator columns per warp group
        const int c_lo = (grp % (NG / 2)) * DCOLS;
        const uint32_t col = which ? DV_COL : DK_COL;
        void* base = which ? p.dv : p.dk;
        const float osc = which ? 1.f : p.scale;         // dS^T was accumulated without the softmax scale
#pragma unroll 1
        for (int c = c_lo; c < c_lo + DCOLS; c += 32) {
          uint32_t v[32];
          tmem_ld32(t_lane + col + c, v);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * osc);
          if (k_valid) {
            if (p.dkv_mode == 2) {
              const int ch = kidx / p.route_rows, lrow = kidx % p.route_rows;
              float* dst = (float*)(which ? p.route_v[ch] : p.route_k[ch]) + (((size_t)b * p.route_tl + lrow) * p.Hkv + hkv) * D + c;
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                red_add_v4_64(dst + j, __uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
            } else if (p.dkv_mode == 1) {
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
  } else {
    // ------------------------------------------------------------------ dQ drain warps (the last four)
    // tensor memory -> registers -> 128B-swizzled fp32 staging -> TMA reduce-add into the global fp32 dQ (rows past the
    // end of the sequence are clipped by the tensor map).  Every warp drains its own 32 query rows through its own
    // staging slice with its own bulk group, so the four warps never wait for one another; the reduce of tile i is read
    // out of the slice while the warp waits for tile i+1.
    const int quarter = warp & 3;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    uint8_t* stage = smem + L::DQS_OFF + quarter * 8192;      // [2 column halves][32 rows][128 B]
    const bool issuer = (lane == 0);
    if (issuer) tma_prefetch_desc(&tmDQ);
    for (int i = 0; i < n_it; ++i) {
      const bool dprof = B64_PROF_ON(p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && warp == 2 + 4 * NG && issuer);
      const bool dprof_all = B64_PROF_ON(p.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && i >= 64 && i < 72);
      bool ok = mbar_wait(dq_full, i & 1, abort_flag, p.status, 1100);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (dprof_all) atomicMax((unsigned long long*)&p.prof[16 + (i - 64) * 32 + 10], (unsigned long long)clock64());
      const int hq = hkv * G + i / n_qt;
      const int q0 = (qt_start + i % n_qt) * B64_T;
      uint32_t v[2][32];
      tmem_ld32(t_lane + DQ_COL, v[0]);
      tmem_ld32(t_lane + DQ_COL + 32, v[1]);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive_warp(dq_empty);                          // tensor-memory dQ is free again
      if (dprof_all) atomicMax((unsigned long long*)&p.prof[16 + (i - 64) * 32 + 11], (unsigned long long)clock64());
      if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous tile has left the slice
      __syncwarp();
#pragma unroll
      for (int h = 0; h < D / 32; ++h) {
        uint8_t* rowp = stage + h * 4096 + lane * 128;
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4)                  // dS was formed without the softmax scale: apply it here
          *(float4*)(rowp + ((c4 ^ (lane & 7)) << 4)) = make_float4(__uint_as_float(v[h][4 * c4]) * p.scale, __uint_as_float(v[h][4 * c4 + 1]) * p.scale,
                                                                    __uint_as_float(v[h][4 * c4 + 2]) * p.scale, __uint_as_float(v[h][4 * c4 + 3]) * p.scale);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (issuer && !p.debug_skip_dq) {
#pragma unroll
        for (int h = 0; h < D / 32; ++h)
          asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                       ::"l"((uint64_t)&tmDQ), "r"(smem_u32(stage + h * 4096)), "r"(h * 32), "r"(hq), "r"(q0 + quarter * 32), "r"(b)
                       : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
      B64_STAMP(dprof, i, 13);
    }
    if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// aug_l[row] = -(hi, mid, lo) of lse2[row] / scale_log2 and aug_d[row] = -(hi, mid, lo) of delta[row], each padded to
// eight bf16 (16 bytes per query row).  Rows whose lse2 is +inf (padding, fully masked) get a large finite magnitude so
// that their probabilities underflow to exactly zero.
__global__ void bwd64_aug_kernel(const float* __restrict__ lse2, const float* __restrict__ delta,
                                 uint4* __restrict__ aug_l, uint4* __restrict__ aug_d, size_t n, float inv_scale_log2) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float src[2] = {lse2[i], delta[i]};
    uint4 out[2];
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      float x = src[w];
      if (w == 0) x = (x > 1e37f) ? 1e30f : x * inv_scale_log2;
      x = -x;
      const __nv_bfloat16 h = __float2bfloat16_rn(x);
      const float r1 = x - __bfloat162float(h);
      const __nv_bfloat16 m = __float2bfloat16_rn(r1);
      const float r2 = r1 - __bfloat162float(m);
      const __nv_bfloat16 l = __float2bfloat16_rn(r2);
      out[w] = make_uint4((uint32_t)__bfloat16_as_ushort(h) | ((uint32_t)__bfloat16_as_ushort(m) << 16),
                          (uint32_t)__bfloat16_as_ushort(l), 0u, 0u);
    }
    aug_l[i] = out[0];
    aug_d[i] = out[1];
  }
}

static int make_tmap4_64(CUtensorMap* m, const void* ptr, int H, int T, int B, long s_head, long s_tok, long s_batch) {
  uint64_t dims[4] = {(uint64_t)B64_D, (uint64_t)H, (uint64_t)T, (uint64_t)B};
  uint64_t strides[4] = {0, (uint64_t)s_head * 2, (uint64_t)s_tok * 2, (uint64_t)s_batch * 2};
  uint32_t box[4] = {64, 1, (uint32_t)B64_T, 1};
  return encode_tmap(m, ptr, 2, 4, dims, strides, box, 1);
}

}  // namespace cpb

using namespace cpb;

// lse2 / delta: fp32 [B,Hq,Tq_pad] as produced by cpb_flash_bwd_prep; aug_l / aug_d: bf16 [B,Hq,Tq_pad,8].
extern "C" int cpb_flash_bwd64_aug(const float* lse2, const float* delta, void* aug_l, void* aug_d, long n, float scale,
                                   cudaStream_t stream) {
  if (n <= 0) return CPB_OK;
  size_t g = ((size_t)n + 255) / 256;
  const size_t cap = (size_t)sm_count() * 8;
  if (g > cap) g = cap;
  bwd64_aug_kernel<<<(int)g, 256, 0, stream>>>(lse2, delta, (uint4*)aug_l, (uint4*)aug_d, (size_t)n, 1.f / (scale * 1.4426950408889634f));
  return check_launch("flash_bwd64_aug");
}

// Same contract as cpb_flash_bwd for head_dim 64, with the per-row vectors passed in their augmented bf16 form.
extern "C" int cpb_flash_bwd64(const void* q, const void* k, const void* v, const void* dout, const void* aug_l,
                               const void* aug_d, float* dq, void* dk, void* dv,
                               int B, int Tq, int Tk, int Hq, int Hkv, int Tq_pad,
                               long q_sh, long q_st, long q_sb, long k_sh, long k_st, long k_sb,
                               float scale, int causal, int k_off, const int* q_pos, int dkv_mode,
                               const uint64_t* route_k, const uint64_t* route_v, int route_rows, int route_tl,
                               int* status, cudaStream_t stream) {
  if (Hq % Hkv) return set_error(CPB_ERR_ARG, "flash_bwd64: Hq %% Hkv != 0");
  if (Tq_pad % B64_T || Tq_pad < Tq) return set_error(CPB_ERR_ARG, "flash_bwd64: bad Tq_pad");
  if (q_pos == nullptr || aug_l == nullptr || aug_d == nullptr) return set_error(CPB_ERR_ARG, "flash_bwd64: q_pos and the augmented vectors are required");
  if (((uintptr_t)aug_l | (uintptr_t)aug_d | (uintptr_t)q_pos) & 15) return set_error(CPB_ERR_ARG, "flash_bwd64: vectors must be 16-byte aligned");
  if (dkv_mode == 2 && (route_k == nullptr || route_v == nullptr || route_rows <= 0))
    return set_error(CPB_ERR_ARG, "flash_bwd64: routed dK/dV needs route tables");
  CUtensorMap tq, tk, tv, tdo, tdq;
  int rc;
  if ((rc = make_tmap4_64(&tq, q, Hq, Tq, B, q_sh, q_st, q_sb)) != CPB_OK) return rc;
  if ((rc = make_tmap4_64(&tk, k, Hkv, Tk, B, k_sh, k_st, k_sb)) != CPB_OK) return rc;
  if ((rc = make_tmap4_64(&tv, v, Hkv, Tk, B, k_sh, k_st, k_sb)) != CPB_OK) return rc;
  if ((rc = make_tmap4_64(&tdo, dout, Hq, Tq, B, B64_D, (long)Hq * B64_D, (long)Tq * Hq * B64_D)) != CPB_OK) return rc;
  {
    uint64_t dims[4] = {(uint64_t)B64_D, (uint64_t)Hq, (uint64_t)Tq, (uint64_t)B};
    uint64_t strides[4] = {0, (uint64_t)B64_D * 4, (uint64_t)Hq * B64_D * 4, (uint64_t)Tq * Hq * B64_D * 4};
    uint32_t box[4] = {32, 1, 32, 1};      // one drain warp: 32 query rows x 32 columns
    if ((rc = encode_tmap(&tdq, dq, 4, 4, dims, strides, box, 1)) != CPB_OK) return rc;
  }
  Bwd64Params p;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hkv = Hkv; p.Tq_pad = Tq_pad; p.causal = causal; p.k_off = k_off;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.aug_l = (const __nv_bfloat16*)aug_l; p.aug_d = (const __nv_bfloat16*)aug_d; p.q_pos = q_pos;
  p.dk = dk; p.dv = dv; p.dkv_mode = dkv_mode; p.status = status;
  p.route_k = route_k; p.route_v = route_v; p.route_rows = route_rows; p.route_tl = route_tl;
  // diagnostic switches and the tuning knob are read once per process, not per launch
  static const bool skip_dq = [] {
    const char* e = getenv("CPB_BWD_SKIP_DQ");
    const bool on = e != nullptr && e[0] == '1';
    if (on) fprintf(stderr, "CPB_BWD_SKIP_DQ=1: the attention backward does NOT produce dQ (timing experiment only)\n");
    return on;
  }();
  static const bool want_prof = [] { const char* e = getenv("CPB_BWD_PROF"); return e != nullptr && e[0] == '1'; }();
  static const int poly = [] { const char* e = getenv("CPB_BWD64_POLY"); return e ? atoi(e) : B64_POLY; }();
  p.debug_skip_dq = skip_dq;
  p.prof = nullptr;
  if (want_prof) {
    void* sym = nullptr;
    if (cudaGetSymbolAddress(&sym, g_bwd64_prof) == cudaSuccess) { p.prof = (long long*)sym; cudaMemsetAsync(sym, 0, sizeof(long long) * (16 + 32 * 8), stream); }
  }
  dim3 grid((Tk + B64_T - 1) / B64_T, Hkv, B);
#define CPB_BWD64_LAUNCH(PP, GG)                                                                                        \
  do {                                                                                                                  \
    static bool cfg = false;                                                                                            \
    if (!cfg) { CPB_CUDA_OK(cudaFuncSetAttribute(flash_bwd64_kernel<PP, GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, Bwd64Smem::TOTAL)); cfg = true; } \
    flash_bwd64_kernel<PP, GG><<<grid, b64_threads(GG), Bwd64Smem::TOTAL, stream>>>(tq, tk, tv, tdo, tdq, p);           \
  } while (0)
  static const int ng = [] { const char* e = getenv("CPB_BWD64_NG"); return e ? atoi(e) : B64_NG; }();
  if (ng == 2) {
    switch (poly) {
      case 3: CPB_BWD64_LAUNCH(3, 2); break;
      default: CPB_BWD64_LAUNCH(0, 2); break;
    }
  } else {
    switch (poly) {
      case 2: CPB_BWD64_LAUNCH(2, 4); break;
      case 3: CPB_BWD64_LAUNCH(3, 4); break;
      case 4: CPB_BWD64_LAUNCH(4, 4); break;
      default: CPB_BWD64_LAUNCH(0, 4); break;
    }
  }
#undef CPB_BWD64_LAUNCH
  if (p.prof != nullptr) {
    long long h[16 + 32 * 8];
    cudaStreamSynchronize(stream);
    if (cudaMemcpy(h, p.prof, sizeof(h), cudaMemcpyDeviceToHost) == cudaSuccess && h[15] > 0)
      fprintf(stderr, "[flash_bwd64 prof] tiles=%lld cycles/tile of the MMA warp: wait_s_consumed+issue_S=%lld wait_p_full=%lld wait_dq_empty=%lld issue_grads=%lld\n",
              h[15], h[0] / h[15], h[1] / h[15], h[2] / h[15], h[3] / h[15]);
    if (cudaMemcpy(h, p.prof, sizeof(h), cudaMemcpyDeviceToHost) == cudaSuccess && h[15] > 72) {
      const long long base = h[16 + 9];
      const int NE = 18;
      static const char* names[18] = {"M:s_consumed", "M:q_full", "M:S'issued", "M:p_full", "M:dK issued", "M:dP' issued", "M:dV issued", "M:dq_empty",
                                      "M:dQ issued", "W:s_ready", "D:dq_full seen(last warp)", "D:dq_empty arrive(last warp)", "W:dp_ready", "D:staged", "W:dq_full", "W:p_full arrive", "W:tile top", "W:s_ready try ok"};
      for (int t = 0; t < 4; ++t) {
        fprintf(stderr, "  tile %d:", 64 + t);
        // chronological order
        int order[18]; for (int e = 0; e < NE; ++e) order[e] = e;
        for (int a2 = 0; a2 < NE; ++a2) for (int b2 = a2 + 1; b2 < NE; ++b2) if (h[16 + t * 32 + order[b2]] < h[16 + t * 32 + order[a2]]) { int x = order[a2]; order[a2] = order[b2]; order[b2] = x; }
        for (int e = 0; e < NE; ++e) fprintf(stderr, " %s@%lld", names[order[e]], h[16 + t * 32 + order[e]] - base);
        fprintf(stderr, " [dq_empty polls: %lld]", h[16 + t * 32 + 20]);
        fprintf(stderr, "\n");
      }
    }
  }
  return check_launch("flash_bwd64");
}
