// Flash-attention forward for sm_100a: S = Q K^T and O += P V on tcgen05 tensor cores with S, P and O
// resident in tensor memory; K tiles streamed by TMA (no multicast) through a 3-stage and V tiles through a
// 2-stage ring; online softmax with lazy rescaling in eight softmax warps (two threads per query row, 64 key
// columns each, row maxima exchanged through shared memory), so each scheduler has enough warps to hide MUFU
// and tensor-memory latency.  The exponentials of a tile are computed into registers before the wait for the
// previous tile's P V product, so the tensor core's latency is off the softmax warps' per-tile chain.
//
// One kernel serves every attention mode of the framework:
//   * local causal / non-causal attention with GQA (Ulysses, world size 1);
//   * ring attention over a K/V buffer laid out in GLOBAL position order, masking on global
//     positions (q_pos[] gives each local query row its global position), which replaces the
//     reference's per-step Full / KHeadHalf / QTailHalf sub-chunk slicing and its separate
//     online-softmax merge (context_parallel/ContextParallel.h:730-784,
//     context_parallel/SDPAMerger.h:108-121): (m, l, O) simply persist across K/V blocks;
//   * the fused ring: K/V blocks owned by other ranks arrive in the local buffer while the kernel
//     runs; before the first tile of block c the loader waits (bounded) on ready[c].
//
// Tensors are token-major: Q [B,Tq,Hq,D], K/V [B,Tk,Hkv,D] with arbitrary 16-byte-aligned strides (views
// into a packed QKV buffer work without a copy), O [B,Tq,Hq,D] contiguous, LSE [B,Hq,Tq] fp32 (natural log).
//
// Replaces fused_attn_forward_kernel_tc (context_parallel/AttentionForward.cu:490-844) and
// gqa_fused_rope_v2 (context_parallel/GQA_fused_fwd_sm103_cp.cu:117-281).
#include "common.cuh"
#include <stdio.h>
#include <stdlib.h>
#include "host_utils.h"
#include "ring_copy.cuh"

namespace cpb {

constexpr int FA_BQ = 128;
constexpr int FA_BK = 128;
constexpr int FA_THREADS = 320;
constexpr int FA_KSTAGES = 3;      // K is wanted one tile ahead of V (the next score tile overlaps the softmax of this one)
constexpr int FA_VSTAGES = 2;
constexpr int FA_POLY_D64 = 0;     // default share (of 8) of the exponentials taken off the special-function unit
constexpr int FA_POLY_D128 = 2;

struct FwdParams {
  int B, Tq, Tk, Hq, Hkv;
  int causal;
  int k_off;                 // global position of K row 0
  float scale_log2;          // softmax scale * log2(e)
  const int* q_pos;          // [Tq] global position of each query row, or null (= row index)
  __nv_bfloat16* O;          // [B,Tq,Hq,D]
  float* lse;                // [B,Hq,Tq]
  // fused-ring readiness flags: K/V rows [c*block_rows, (c+1)*block_rows) may be read once
  // ready[c] >= ready_epoch.  null -> everything is ready.
  int* ready;
  int ready_epoch;
  int block_rows;
  // fused ring: the first n_copy CTAs (blockIdx.x < n_copy, y = z = 0) pull the K/V blocks listed in segs into
  // the local position-ordered buffer and bump ready[]; the compute CTAs start on the chunk that holds
  // their own diagonal (local data) and wrap around while remote chunks land.
  const CopySeg* segs;
  int n_segs;
  int n_copy;
  // Ulysses: when o_peers != null the epilogue stores each output row straight into the arena of the rank
  // that owns the token: row qi -> peer qi / o_rows_per_peer, local row qi % o_rows_per_peer, layout
  // [B, o_rows_per_peer, o_heads_total, D] at byte offset o_off, head slot o_head_off + hq.
  const uint64_t* o_peers;
  long o_off;
  int o_rows_per_peer, o_head_off, o_heads_total;
  int* status;
};

// Diagnostics: with -DCPB_FWD_PROF the CTA that owns the last query tile of (head 0, batch 0) records an event
// timeline of K/V tiles 32..35 into a static device array that the launcher prints.
#ifdef CPB_FWD_PROF
static __device__ long long g_fwd_prof[4 * 16];
#define FWD_STAMP(cond, j, e) do { if ((cond) && (j) >= 32 && (j) < 36) g_fwd_prof[((j) - 32) * 16 + (e)] = clock64(); } while (0)
#else
#define FWD_STAMP(cond, j, e) do { } while (0)
#endif

template <int D>
struct FwdSmem {
  static constexpr int Q_BYTES = FA_BQ * D * 2;
  static constexpr int KV_BYTES = FA_BK * D * 2;
  static constexpr int K_OFF = Q_BYTES;
  static constexpr int V_OFF = K_OFF + FA_KSTAGES * KV_BYTES;
  static constexpr int BAR_OFF = V_OFF + FA_VSTAGES * KV_BYTES;
  static constexpr int XCH_OFF = BAR_OFF + 256;            // [2 tiles][2 halves][128 rows] fp32 row-max exchange
  static constexpr int TOTAL = XCH_OFF + 2048 + 1024;
};

// Bounded acquire-spin on a readiness flag in global memory (written by a copy kernel or a peer).
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int value, volatile int* abort_flag, int* status, int site) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= value) return true;
    if (*abort_flag) return false;
    __nanosleep(200);
  }
  *abort_flag = 1;
  report(status, ST_TIMEOUT_FLAG, site, value);
  return false;
}

// POLY: of the 8 column pairs of every 16-column group, the last POLY take exp2_poly_f32x2 and the others ex2.approx.
template <int D, int POLY>
__global__ void __launch_bounds__(FA_THREADS, (D == 64 ? 2 : 1))
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, FwdParams p) {
  using L = FwdSmem<D>;
  if (p.n_copy > 0 && blockIdx.x < (unsigned)p.n_copy) {
    if (blockIdx.y == 0 && blockIdx.z == 0) ring_copy_cta(p.segs, p.n_segs, p.n_copy, blockIdx.x, p.ready);
    return;
  }
  const int bx = (int)blockIdx.x - p.n_copy;
  constexpr int DH = D / 64;                // 64-wide halves of the head dimension
  // tensor memory: S (128 fp32 columns) | O (D columns) | P (bf16, 64 columns).  P has columns of its own, so the next
  // score tile is computed while the warps still work on the current one.
  constexpr uint32_t TMEM_COLS = (D == 64) ? 256 : 512;
  constexpr uint32_t O_COL = 128;
  constexpr uint32_t P_COL = 128 + D;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + L::BAR_OFF);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;              // [3]
  uint64_t* k_empty = bars + 4;             // [3]
  uint64_t* v_full = bars + 7;              // [2]
  uint64_t* v_empty = bars + 9;             // [2]
  uint64_t* s_full = bars + 11;
  uint64_t* p_full = bars + 12;
  uint64_t* o_done = bars + 13;
  uint64_t* s_consumed = bars + 14;
  uint64_t* pv_done = bars + 15;
  uint32_t* tmem_slot = (uint32_t*)(bars + 16);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int num_q_tiles = (p.Tq + FA_BQ - 1) / FA_BQ;
  const int qt = num_q_tiles - 1 - bx / G;                   // heaviest tiles first
  const int hkv = blockIdx.y;
  const int hq = hkv * G + bx % G;
  const int b = blockIdx.z;
  const int q0 = qt * FA_BQ;

  // Range of K/V tiles this query tile attends to.
  const int q_last = min(q0 + FA_BQ, p.Tq) - 1;
  const int qpos_min = p.q_pos ? p.q_pos[q0] : q0;
  const int qpos_max = p.q_pos ? p.q_pos[q_last] : q_last;
  int n_kv = (p.Tk + FA_BK - 1) / FA_BK;
  if (p.causal) {
    const int last_idx = qpos_max - p.k_off;                  // last visible K index
    n_kv = last_idx < 0 ? 0 : min(n_kv, last_idx / FA_BK + 1);
  }
  // Order of the K/V sweep: tile (j + j_start) % n_kv.  With readiness flags the sweep starts at the chunk
  // that contains this tile's own positions (resident locally), so remote chunks have time to arrive.
  int j_start = 0;
  if (p.ready != nullptr && n_kv > 0 && (p.block_rows % FA_BK) == 0) {
    const int c = max(qpos_min - p.k_off, 0) / p.block_rows;
    j_start = min(c * (p.block_rows / FA_BK), n_kv - 1);
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FA_KSTAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < FA_VSTAGES; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_full, 256);
    mbar_init(o_done, 1);
    mbar_init(s_consumed, 8);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA loader
    if (lane == 0 && n_kv > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int h = 0; h < DH; ++h) tma_load_4d(smem + h * (FA_BQ * 128), &tmQ, q_full, h * 64, hq, q0, b);
      int ready_block = -1;
      for (int j = 0; j < n_kv; ++j) {
        const int ks = j % FA_KSTAGES, vs = j % FA_VSTAGES;
        if (!mbar_wait(&k_empty[ks], ((j / FA_KSTAGES) & 1) ^ 1, abort_flag, p.status, 500)) break;
        const int jj = j + j_start;
        const int k0 = (jj >= n_kv ? jj - n_kv : jj) * FA_BK;
        if (p.ready != nullptr) {
          // a tile may straddle two blocks when block_rows is not a multiple of the tile
          const int blk_hi = min(k0 + FA_BK, p.Tk) - 1;
          for (int c = k0 / p.block_rows; c <= blk_hi / p.block_rows; ++c) {
            if (c == ready_block) continue;
            if (!wait_flag_ge(p.ready + c, p.ready_epoch, abort_flag, p.status, 501)) break;
            ready_block = c;
          }
          if (*abort_flag) break;
          // The copy CTAs wrote these rows with ordinary (generic-proxy) stores; the loads below go through the
          // async proxy (TMA).  The acquire above orders generic accesses only, so a cross-proxy fence is needed
          // before the first bulk-tensor read of a freshly arrived block.
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        uint8_t* sk = smem + L::K_OFF + ks * L::KV_BYTES;
        uint8_t* sv = smem + L::V_OFF + vs * L::KV_BYTES;
        mbar_expect_tx(&k_full[ks], L::KV_BYTES);
#pragma unroll
        for (int h = 0; h < DH; ++h) tma_load_4d(sk + h * (FA_BK * 128), &tmK, &k_full[ks], h * 64, hkv, k0, b);
        if (!mbar_wait(&v_empty[vs], ((j / FA_VSTAGES) & 1) ^ 1, abort_flag, p.status, 502)) break;
        mbar_expect_tx(&v_full[vs], L::KV_BYTES);
#pragma unroll
        for (int h = 0; h < DH; ++h) tma_load_4d(sv + h * (FA_BK * 128), &tmV, &v_full[vs], h * 64, hkv, k0, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs this code convergently and only the elected lane issues: the descriptors then stay
    // warp-uniform, and stepping one is a single add (see sdesc_at).
    if (n_kv > 0) {
      const bool mprof = (bx == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0);
      const uint32_t leader = elect_one() ? 1u : 0u;
      constexpr uint32_t idesc_qk = make_idesc_bf16(FA_BQ, FA_BK, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(FA_BQ, D, false, true);
      const SDesc dq = sdesc_split(sdesc_kmajor(smem_u32(smem)));
      const SDesc dk0 = sdesc_split(sdesc_kmajor(smem_u32(smem + L::K_OFF)));                            // stage 0
      const SDesc dv0 = sdesc_split(make_sdesc(smem_u32(smem + L::V_OFF), FA_BK * 128, 1024));           // V tile, N-major
      const uint32_t s_tmem = tmem_base;
      const uint32_t o_tmem = tmem_base + O_COL;
      const uint32_t p_tmem = tmem_base + P_COL;
      auto issue_qk = [&](int j) {
        const SDesc dk = SDesc{dk0.lo + (uint32_t)(j % FA_KSTAGES) * (L::KV_BYTES >> 4), dk0.hi};
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (FA_BQ * 128) + (k % 4) * 32;
          if (k == 0) umma_ss_cp<false>(leader, s_tmem, sdesc_at(dq, off), sdesc_at(dk, off), idesc_qk);
          else umma_ss_cp<true>(leader, s_tmem, sdesc_at(dq, off), sdesc_at(dk, off), idesc_qk);
        }
        umma_commit_p(leader, s_full);
        umma_commit_p(leader, &k_empty[j % FA_KSTAGES]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 600) && mbar_wait(&k_full[0], 0, abort_flag, p.status, 601);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
        for (int j = 0; j < n_kv; ++j) {
          const int st = j % FA_VSTAGES;
          if (j + 1 < n_kv) {
            // the warps hold S(j) in registers: the next score tile can be computed while they work on it
            bool w0 = mbar_wait(s_consumed, j & 1, abort_flag, p.status, 605) && mbar_wait(&k_full[(j + 1) % FA_KSTAGES], ((j + 1) / FA_KSTAGES) & 1, abort_flag, p.status, 604);
            if (!__all_sync(0xffffffffu, w0)) break;
            tc_fence_after();
            FWD_STAMP(mprof, j, 2);
            issue_qk(j + 1);
            FWD_STAMP(mprof, j, 3);
          }
          bool w = mbar_wait(p_full, j & 1, abort_flag, p.status, 602) && mbar_wait(&v_full[st], (j / FA_VSTAGES) & 1, abort_flag, p.status, 603);
          if (!__all_sync(0xffffffffu, w)) break;
          tc_fence_after();
          FWD_STAMP(mprof, j, 0);
          const SDesc dv = SDesc{dv0.lo + (uint32_t)st * (L::KV_BYTES >> 4), dv0.hi};
          // A = P (bf16, 8 tensor-memory columns per 16 keys); B = V tile, N-major: 16 key rows = 2 KB
          umma_ts_p(leader, o_tmem, p_tmem, sdesc_at(dv, 0), idesc_pv, j != 0);
#pragma unroll
          for (int k = 1; k < FA_BK / 16; ++k)
            umma_ts_cp<true>(leader, o_tmem, p_tmem + k * 8, sdesc_at(dv, k * 2048), idesc_pv);
          umma_commit_p(leader, &v_empty[st]);
          umma_commit_p(leader, pv_done);
          FWD_STAMP(mprof, j, 1);
          if (j + 1 == n_kv) umma_commit_p(leader, o_done);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (warps 2..9)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;                  // which 64 key columns of every tile this thread owns
    const int cbase = half * 64;
    const int row = quarter * 32 + lane;
    const int qi = q0 + row;
    const bool row_valid = qi < p.Tq;
    const int my_qpos = row_valid ? (p.q_pos ? p.q_pos[qi] : qi) : 0x7fffffff;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    float* xch = (float*)(smem + L::XCH_OFF);
    float m_used = -INFINITY;    // running max (scaled, log2 domain) the accumulators are relative to
    float l = 0.f;               // this thread's share of the row sum
    bool alive = n_kv > 0;
    const bool wprof = (bx == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 64);
    for (int j = 0; j < n_kv && alive; ++j) {
      FWD_STAMP(wprof, j, 4);
      bool ok = mbar_wait(s_full, j & 1, abort_flag, p.status, 700);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { alive = false; break; }
      tc_fence_after();
      FWD_STAMP(wprof, j, 5);
      const int jj = j + j_start;
      const int k0 = (jj >= n_kv ? jj - n_kv : jj) * FA_BK;
      const bool need_mask = (k0 + FA_BK > p.Tk) || (p.causal && (k0 + FA_BK - 1 + p.k_off > qpos_min));
      const int kmax_causal = p.causal ? (my_qpos - p.k_off) : 0x7fffffff;   // last visible index
      const int kmax = min(kmax_causal, p.Tk - 1) - k0 - cbase;               // last visible column of my span
      // this thread's 64 scores, one tensor-memory round trip
      uint32_t sv[4][16];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) tmem_ld16(t_lane + cbase + 16 * ch, sv[ch]);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive_warp(s_consumed);                     // S(j) is in registers: the next score tile may overwrite it
      FWD_STAMP(wprof, j, 6);
      float mx = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
#pragma unroll
          for (int i = 0; i < 16; ++i) if (ch * 16 + i <= kmax) mx = fmaxf(mx, __uint_as_float(sv[ch][i]));
      } else {
        // four independent chains of eight three-input maxima instead of one chain of thirty-two
        float m4[4];
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          m4[ch] = fmaxf(__uint_as_float(sv[ch][0]), __uint_as_float(sv[ch][1]));
#pragma unroll
          for (int i = 2; i < 16; i += 2) m4[ch] = fmax3(m4[ch], __uint_as_float(sv[ch][i]), __uint_as_float(sv[ch][i + 1]));
        }
        mx = fmaxf(fmax3(m4[0], m4[1], m4[2]), m4[3]);
      }
      // row maximum over both halves: exchange through shared memory with the partner warp (same rows)
      float* slot = xch + (j & 1) * 256;
      slot[half * 128 + row] = mx;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
      mx = fmaxf(mx, slot[(half ^ 1) * 128 + row]);
      FWD_STAMP(wprof, j, 7);
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      // lazy rescale: keep the old reference maximum unless it fell behind by more than 2^8
      const bool need = (m_new > m_used + 8.f);
      float alpha = 1.f;
      if (need) {
        alpha = (m_used == -INFINITY) ? 0.f : ex2f(m_used - m_new);
        m_used = m_new;
        l *= alpha;
      }
      // p = exp2(s*scale - m) as bf16 pairs, kept in registers: the exponentials need only S(j) and the maximum, so they
      // run while the tensor core still works on P(j-1) V(j-1); tensor memory (the P columns, O) is touched after pv_done
      const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
      uint32_t pk[32];
      // two copies of the loop: the common one (no tile edge, not on the diagonal) carries no compare/select per element
      float l0 = 0.f, l1 = 0.f;
      if (!need_mask) {
        const uint64_t c2 = pack_f32x2(p.scale_log2, p.scale_log2), m2 = pack_f32x2(-m_sub, -m_sub);
        uint64_t l2 = pack_f32x2(0.f, 0.f);
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            float p0, p1;
            const uint64_t x2 = fma_f32x2(pack_f32x2(__uint_as_float(sv[ch][i]), __uint_as_float(sv[ch][i + 1])), c2, m2);
            if ((i >> 1) >= 8 - POLY) {                      // resolved at compile time (the loop is unrolled)
              const uint64_t p2 = exp2_poly_f32x2(x2);
              l2 = add_f32x2(l2, p2);
              unpack_f32x2(p2, p0, p1);
            } else {
              float x0, x1;
              unpack_f32x2(x2, x0, x1);
              p0 = ex2f(x0); p1 = ex2f(x1);
              l2 = add_f32x2(l2, pack_f32x2(p0, p1));
            }
            pk[ch * 8 + (i >> 1)] = pack_bf16(p0, p1);
          }
        }
        unpack_f32x2(l2, l0, l1);
      } else {
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float p0 = (ch * 16 + i > kmax) ? 0.f : ex2f(fmaf(__uint_as_float(sv[ch][i]), p.scale_log2, -m_sub));
            const float p1 = (ch * 16 + i + 1 > kmax) ? 0.f : ex2f(fmaf(__uint_as_float(sv[ch][i + 1]), p.scale_log2, -m_sub));
            l0 += p0; l1 += p1;
            pk[ch * 8 + (i >> 1)] = pack_bf16(p0, p1);
          }
        }
      }
      FWD_STAMP(wprof, j, 9);
      if (j > 0) {
        // PV(j-1) has read the previous P and finished updating O
        bool okp = mbar_wait(pv_done, (j - 1) & 1, abort_flag, p.status, 702);
        okp = __all_sync(0xffffffffu, okp);
        if (!okp) { alive = false; break; }
        tc_fence_after();
      }
      if (j > 0 && __any_sync(0xffffffffu, need)) {
        // each thread of the pair rescales its own half of the O columns
#pragma unroll 1
        for (int c = half * (D / 2); c < (half + 1) * (D / 2); c += 32) {
          uint32_t v[32];
          tmem_ld32(t_lane + O_COL + c, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st32(t_lane + O_COL + c, v);
        }
      }
      FWD_STAMP(wprof, j, 8);
      // bf16 P into its columns: k-step 4*half+ch at column (4*half+ch)*8
      tmem_st32(t_lane + P_COL + half * 32, pk);
      l += l0 + l1;
      tmem_wait_st();
      tc_fence_before();
      FWD_STAMP(wprof, j, 10);
      mbar_arrive(p_full);
      FWD_STAMP(wprof, j, 11);
    }
    // epilogue: O / l -> bf16, LSE
    if (alive) {
      float* slot = xch + (n_kv & 1) * 256;
      slot[half * 128 + row] = l;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
      l += slot[(half ^ 1) * 128 + row];
      bool ok = mbar_wait(o_done, 0, abort_flag, p.status, 701);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        const float inv_l = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* orow = p.O + (((size_t)b * p.Tq + (row_valid ? qi : 0)) * p.Hq + hq) * D;
        if (p.o_peers != nullptr && row_valid) {
          const int peer = qi / p.o_rows_per_peer, lrow = qi % p.o_rows_per_peer;
          orow = (__nv_bfloat16*)(p.o_peers[peer] + p.o_off) +
                 (((size_t)b * p.o_rows_per_peer + lrow) * p.o_heads_total + p.o_head_off + hq) * D;
        }
#pragma unroll 1
        for (int c = half * (D / 2); c < (half + 1) * (D / 2); c += 32) {
          uint32_t v[32];
          tmem_ld32(t_lane + O_COL + c, v);
          tmem_wait_ld();
          if (row_valid) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(v[i]) * inv_l, __uint_as_float(v[i + 1]) * inv_l);
              o.y = pack_bf16(__uint_as_float(v[i + 2]) * inv_l, __uint_as_float(v[i + 3]) * inv_l);
              o.z = pack_bf16(__uint_as_float(v[i + 4]) * inv_l, __uint_as_float(v[i + 5]) * inv_l);
              o.w = pack_bf16(__uint_as_float(v[i + 6]) * inv_l, __uint_as_float(v[i + 7]) * inv_l);
              *(uint4*)(orow + c + i) = o;
            }
          }
        }
        if (row_valid && half == 0)
          p.lse[((size_t)b * p.Hq + hq) * p.Tq + qi] = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
    } else if (n_kv == 0 && row_valid && half == 0) {
      // no visible key at all: zero output, LSE = -inf
      __nv_bfloat16* orow = p.O + (((size_t)b * p.Tq + qi) * p.Hq + hq) * D;
      if (p.o_peers != nullptr) {
        const int peer = qi / p.o_rows_per_peer, lrow = qi % p.o_rows_per_peer;
        orow = (__nv_bfloat16*)(p.o_peers[peer] + p.o_off) +
               (((size_t)b * p.o_rows_per_peer + lrow) * p.o_heads_total + p.o_head_off + hq) * D;
      }
#pragma unroll
      for (int c = 0; c < D; c += 8) *(uint4*)(orow + c) = make_uint4(0, 0, 0, 0);
      p.lse[((size_t)b * p.Hq + hq) * p.Tq + qi] = -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

static int make_qkv_tmap(CUtensorMap* m, const void* ptr, int D, int H, int T, int B, long s_head, long s_tok,
                         long s_batch, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)T, (uint64_t)B};
  uint64_t strides[4] = {0, (uint64_t)s_head * 2, (uint64_t)s_tok * 2, (uint64_t)s_batch * 2};
  uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return encode_tmap(m, ptr, 2, 4, dims, strides, box, 1);
}

}  // namespace cpb

using namespace cpb;

// strides are in elements: (head, token, batch) for q and for k/v (k and v share strides).
extern "C" int cpb_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                             int B, int Tq, int Tk, int Hq, int Hkv, int D,
                             long q_sh, long q_st, long q_sb, long k_sh, long k_st, long k_sb,
                             float scale, int causal, int k_off, const int* q_pos,
                             int* ready, int ready_epoch, int block_rows,
                             const void* segs, int n_segs, int n_copy,
                             const uint64_t* o_peers, long o_off, int o_rows_per_peer, int o_head_off, int o_heads_total,
                             int* status, cudaStream_t stream) {
  if (D != 64 && D != 128) return set_error(CPB_ERR_ARG, "flash_fwd: head_dim %d not in {64,128}", D);
  if (Hq % Hkv) return set_error(CPB_ERR_ARG, "flash_fwd: Hq %% Hkv != 0");
  if (B <= 0 || Tq <= 0 || Tk <= 0) return set_error(CPB_ERR_ARG, "flash_fwd: empty problem");
  if (ready != nullptr && block_rows <= 0) return set_error(CPB_ERR_ARG, "flash_fwd: block_rows must be positive with ready flags");
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_qkv_tmap(&tq, q, D, Hq, Tq, B, q_sh, q_st, q_sb, FA_BQ)) != CPB_OK) return rc;
  if ((rc = make_qkv_tmap(&tk, k, D, Hkv, Tk, B, k_sh, k_st, k_sb, FA_BK)) != CPB_OK) return rc;
  if ((rc = make_qkv_tmap(&tv, v, D, Hkv, Tk, B, k_sh, k_st, k_sb, FA_BK)) != CPB_OK) return rc;
  FwdParams p;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.k_off = k_off;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.q_pos = q_pos; p.O = (__nv_bfloat16*)o; p.lse = lse;
  p.ready = ready; p.ready_epoch = ready_epoch; p.block_rows = block_rows; p.status = status;
  p.segs = (const CopySeg*)segs; p.n_segs = n_segs; p.n_copy = (segs != nullptr && n_segs > 0) ? n_copy : 0;
  p.o_peers = o_peers; p.o_off = o_off; p.o_rows_per_peer = o_rows_per_peer; p.o_head_off = o_head_off;
  p.o_heads_total = o_heads_total;
  if (p.n_copy > 0 && ready == nullptr) return set_error(CPB_ERR_ARG, "flash_fwd: copy CTAs need ready flags");
  const int G = Hq / Hkv;
  dim3 grid(p.n_copy + ((Tq + FA_BQ - 1) / FA_BQ) * G, Hkv, B);
  // Share of the exponentials computed on the FMA pipe (column pairs out of 8); CPB_FWD_POLY overrides the tuned
  // default and is read once.
  static const int poly = [] { const char* e = getenv("CPB_FWD_POLY"); return e ? atoi(e) : -1; }();
#define CPB_FWD_LAUNCH(DD, PP)                                                                                         \
  do {                                                                                                                 \
    static bool cfg = false;                                                                                           \
    if (!cfg) { CPB_CUDA_OK(cudaFuncSetAttribute(flash_fwd_kernel<DD, PP>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<DD>::TOTAL)); cfg = true; } \
    flash_fwd_kernel<DD, PP><<<grid, FA_THREADS, FwdSmem<DD>::TOTAL, stream>>>(tq, tk, tv, p);                         \
  } while (0)
  if (D == 64) {
    switch (poly < 0 ? FA_POLY_D64 : poly) {
      case 0: CPB_FWD_LAUNCH(64, 0); break;
      case 1: CPB_FWD_LAUNCH(64, 1); break;
      case 2: CPB_FWD_LAUNCH(64, 2); break;
      case 4: CPB_FWD_LAUNCH(64, 4); break;
      case 5: CPB_FWD_LAUNCH(64, 5); break;
      default: CPB_FWD_LAUNCH(64, 3); break;
    }
  } else {
    switch (poly < 0 ? FA_POLY_D128 : poly) {
      case 0: CPB_FWD_LAUNCH(128, 0); break;
      case 1: CPB_FWD_LAUNCH(128, 1); break;
      case 3: CPB_FWD_LAUNCH(128, 3); break;
      case 4: CPB_FWD_LAUNCH(128, 4); break;
      default: CPB_FWD_LAUNCH(128, 2); break;
    }
  }
#undef CPB_FWD_LAUNCH
#ifdef CPB_FWD_PROF
  {
    long long h[64];
    cudaStreamSynchronize(stream);
    if (cudaMemcpyFromSymbol(h, g_fwd_prof, sizeof(h)) == cudaSuccess && h[4] != 0) {
      static const char* names[12] = {"M:p_full+v_full", "M:PV issued", "M:k_full", "M:QK issued", "W:tile top", "W:s_full", "W:S loaded", "W:max exchanged",
                                      "W:rescale done", "W:exp done", "W:P stored", "W:arrived"};
      const long long base = h[4];
      for (int t = 0; t < 4; ++t) {
        int order[12]; for (int e = 0; e < 12; ++e) order[e] = e;
        for (int a2 = 0; a2 < 12; ++a2) for (int b2 = a2 + 1; b2 < 12; ++b2) if (h[t * 16 + order[b2]] < h[t * 16 + order[a2]]) { int x = order[a2]; order[a2] = order[b2]; order[b2] = x; }
        fprintf(stderr, "[flash_fwd prof D=%d] tile %d:", D, 32 + t);
        for (int e = 0; e < 12; ++e) fprintf(stderr, " %s@%lld", names[order[e]], h[t * 16 + order[e]] - base);
        fprintf(stderr, "\n");
      }
    }
  }
#endif
  return check_launch("flash_fwd");
}
