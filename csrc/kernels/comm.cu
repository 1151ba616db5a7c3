// Peer-memory communication kernels (NVLink / NVSwitch, plain loads and stores on peer-mapped
// addresses; no TMA multicast, no multimem): cross-rank barrier on flag pads, K/V block gather for
// the ring, Ulysses sequence<->head exchanges, the two-shot gradient all-reduce with the bf16
// cast/scale folded in, and the transport of the sharded optimiser (fp32 reduce-scatter of the gradients
// straight from the peers' gradient buffers, all-gather of the updated parameters).
//
// Every rank owns an arena of identical layout (csrc/runtime/symm.cpp); `peers[r]` is the address of
// rank r's arena in this process.  Flags are int32 epochs that only grow, so they are never reset.
// Every wait is bounded and reports into the status word instead of hanging.
//
// These replace the NCCL call sites of the reference: ring send/recv (context_parallel/RingRotator.h:
// 150-152), the Ulysses all-to-all (context_parallel/UlyssesAttention.h:61,91), and the parameter
// gradient all-reduce (Scripts/Blutrain/gpt2_cp_test.cpp:1594-1600, bluscriptCP.cpp:1003-1012,1716).
#include "common.cuh"
#include "host_utils.h"
#include "ring_copy.cuh"

namespace cpb {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ---------------------------------------------------------------------------- barrier
// Thread r (< world) publishes `epoch` into slot [my_rank] of rank r's flag row, then waits until rank
// r's epoch shows up in the local row.  Launched on the compute stream it orders everything before it
// on every rank before everything after it on every rank.
__global__ void barrier_kernel(const uint64_t* __restrict__ peers, long flag_off, int world, int my_rank, int epoch,
                               long spin_limit, int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  int* remote = (int*)(peers[r] + flag_off) + my_rank;
  st_release_sys(remote, epoch);
  const int* local = (const int*)(peers[my_rank] + flag_off) + r;
  for (long it = 0; it < spin_limit; ++it) {
    if (ld_acquire_sys(local) >= epoch) return;
    __nanosleep(100);
  }
  report(status, ST_TIMEOUT_FLAG, 2000, r);
}

// ---------------------------------------------------------------------------- ring K/V gather
__global__ void ring_gather_kernel(const CopySeg* __restrict__ segs, int n_segs, int* ready) {
  ring_copy_cta(segs, n_segs, gridDim.x, blockIdx.x, ready);
}

// ---------------------------------------------------------------------------- Ulysses exchanges
struct A2APart {
  const __nv_bfloat16* src;   // local [B, Tl, *, D] view: element (b,t,h,:) at src + (b*Tl + t)*src_tok_stride + h*D
  long src_tok_stride;
  int n_local;                // heads of this part every peer receives
  int rep;                    // source head = (peer*n_local + j) / rep  (rep > 1: KV heads replicated)
  int dst_head_off;           // first head slot of this part in the destination row
};
struct A2AParams {
  A2APart part[3];
  int n_parts;
  int B, Tl, D, P, my_rank;
  int dst_heads;              // heads per destination row
  long dst_off;               // byte offset of the landing buffer inside every arena
  const uint64_t* peers;
};

// sequence -> head: this rank's Tl tokens of every head go to the ranks that own the heads; destination
// layout [B, P*Tl, dst_heads, D] with this rank's tokens at rows my_rank*Tl...   One warp per (b, t, peer).
__global__ void a2a_push_kernel(A2AParams p) {
  const int lane = threadIdx.x & 31;
  const size_t n_items = (size_t)p.B * p.Tl * p.P;
  const int vec_per_head = p.D / 8;                  // 16-byte vectors per head
  for (size_t w = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5); w < n_items; w += (size_t)gridDim.x * (blockDim.x >> 5)) {
    const int peer = (int)(w % p.P);
    const int t = (int)((w / p.P) % p.Tl);
    const int b = (int)(w / ((size_t)p.P * p.Tl));
    uint4* dst_row = (uint4*)(p.peers[peer] + p.dst_off) +
                     (((size_t)b * p.P * p.Tl + (size_t)p.my_rank * p.Tl + t) * p.dst_heads) * vec_per_head;
    for (int pi = 0; pi < p.n_parts; ++pi) {
      const A2APart& a = p.part[pi];
      const int nvec = a.n_local * vec_per_head;
      for (int i = lane; i < nvec; i += 32) {
        const int j = i / vec_per_head, c = i % vec_per_head;
        const int sh = (peer * a.n_local + j) / a.rep;
        const uint4 v = *((const uint4*)(a.src + ((size_t)b * p.Tl + t) * a.src_tok_stride + (size_t)sh * p.D) + c);
        dst_row[(size_t)(a.dst_head_off + j) * vec_per_head + c] = v;
      }
    }
  }
}

struct A2APullPart {
  __nv_bfloat16* dst;         // local [B, Tl, *, D] view, element (b,t,h,:) at dst + (b*Tl+t)*dst_tok_stride + h*D
  long dst_tok_stride;
  int n_heads;                // heads of this part in the local (sequence-sharded) layout
  int n_local;                // heads of this part per peer in the head-sharded layout
  int rep;                    // replicas to sum (KV heads replicated over rep peers)
  int src_head_off;           // first head slot of this part in the source row
  int src_heads;              // heads per source row of this part's buffer
  long src_off;               // byte offset of this part's head-sharded buffer inside every arena
};
struct A2APullParams {
  A2APullPart part[3];
  int n_parts;
  int B, Tl, D, P, my_rank;
  const uint64_t* peers;
};

// head -> sequence: every rank pulls, for its own Tl tokens, each head from the rank(s) that own it in the
// head-sharded layout [B, P*Tl, src_heads, D], summing KV replicas in fp32.  One group of D/8 lanes per (b, t, part, head).
__global__ void a2a_pull_kernel(A2APullParams p) {
  const int lane = threadIdx.x & 31;
  int heads_total = 0;
  for (int i = 0; i < p.n_parts; ++i) heads_total += p.part[i].n_heads;
  const size_t n_items = (size_t)p.B * p.Tl * heads_total;
  const int vec_per_head = p.D / 8;
  // a warp covers 32 / vec_per_head heads per pass (four at head_dim 64): every lane carries a 16-byte peer load
  const int ipw = 32 / vec_per_head, sub = lane / vec_per_head, c = lane % vec_per_head;
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  for (size_t w0 = (blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5)) * ipw; w0 < n_items; w0 += warps * ipw) {
    const size_t w = w0 + sub;
    if (sub >= ipw || w >= n_items) continue;
    int hh = (int)(w % heads_total);
    const int t = (int)((w / heads_total) % p.Tl);
    const int b = (int)(w / ((size_t)heads_total * p.Tl));
    int pi = 0;
    while (hh >= p.part[pi].n_heads) { hh -= p.part[pi].n_heads; ++pi; }
    const A2APullPart& a = p.part[pi];
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int rr = 0; rr < a.rep; ++rr) {
      const int peer = a.rep > 1 ? hh * a.rep + rr : hh / a.n_local;
      const int j = a.rep > 1 ? 0 : hh % a.n_local;
      const uint4* src_row = (const uint4*)(p.peers[peer] + a.src_off) +
                             (((size_t)b * p.P * p.Tl + (size_t)p.my_rank * p.Tl + t) * a.src_heads) * vec_per_head;
      const uint4 v = src_row[(size_t)(a.src_head_off + j) * vec_per_head + c];
      acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
      acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
    }
    uint4 o = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
    *((uint4*)(a.dst + ((size_t)b * p.Tl + t) * a.dst_tok_stride + (size_t)hh * p.D) + c) = o;
  }
}

// fp32 row vectors [B, H, Tl_pad] (sequence-sharded) -> [B, Hl, T_pad_total] on the head owners: used for the
// attention backward's delta = rowsum(dO o O), computed where O lives.  dst row stride = dst_T.
__global__ void a2a_push_rows_f32_kernel(const float* __restrict__ src, int B, int H, int Tl, int src_T, int n_local,
                                         int P, int my_rank, long dst_off, int dst_T, const uint64_t* __restrict__ peers) {
  const size_t n = (size_t)B * H * Tl;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i % Tl);
    const int h = (int)((i / Tl) % H);
    const int b = (int)(i / ((size_t)Tl * H));
    const int peer = h / n_local, j = h % n_local;
    float* dst = (float*)(peers[peer] + dst_off) + ((size_t)b * n_local + j) * dst_T + (size_t)my_rank * Tl + t;
    *dst = src[((size_t)b * H + h) * src_T + t];
  }
}

// ---------------------------------------------------------------------------- gradient all-reduce (two-shot)
// Phase 1 (after a barrier): rank r owns slice r of the bucket; it reads slice r of every rank's bf16 staging
// copy (grad * scale, written by cast_f32_bf16), sums in fp32, rounds to bf16 (the wire format of this
// replicated-optimiser path) and writes the rounded result into its own gradient buffer and staging slice.
// Phase 2 (after another barrier): every rank pulls the reduced bf16 slices of the other ranks into its fp32
// gradient buffer.
__global__ void allreduce_reduce_kernel(const uint64_t* __restrict__ peers, long stage_off, float* __restrict__ grad,
                                        long n, int world, int my_rank) {
  const long per = ((n + world - 1) / world + 7) / 8 * 8;
  const long lo = per * my_rank, hi = min(n, lo + per);
  const long nvec = (hi > lo) ? (hi - lo + 7) / 8 : 0;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      const int src = (my_rank + r) % world;         // stagger the peers so links are used evenly
      const uint4 v = *((const uint4*)(peers[src] + stage_off) + (lo >> 3) + i);
      acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
      acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
    }
    const long e = lo + i * 8;
    // the owner keeps the SAME bf16-rounded values the other ranks will gather, so that the replicated optimiser
    // states stay bit-identical on every rank
    const uint4 o = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
    const float rr[8] = {bf16_lo(o.x), bf16_hi(o.x), bf16_lo(o.y), bf16_hi(o.y), bf16_lo(o.z), bf16_hi(o.z), bf16_lo(o.w), bf16_hi(o.w)};
#pragma unroll
    for (int j = 0; j < 8; ++j) if (e + j < n) grad[e + j] = rr[j];
    *((uint4*)(peers[my_rank] + stage_off) + (lo >> 3) + i) = o;
  }
}
__global__ void allreduce_gather_kernel(const uint64_t* __restrict__ peers, long stage_off, float* __restrict__ grad,
                                        long n, int world, int my_rank) {
  const long per = ((n + world - 1) / world + 7) / 8 * 8;
  const long nvec_total = (n + 7) / 8;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec_total; i += (long)gridDim.x * blockDim.x) {
    const long e = i * 8;
    const int owner = (int)(e / per);
    if (owner == my_rank || owner >= world) continue;
    const uint4 v = *((const uint4*)(peers[owner] + stage_off) + i);
    const float f[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y), bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
#pragma unroll
    for (int j = 0; j < 8; ++j) if (e + j < n) grad[e + j] = f[j];
  }
}

// ---------------------------------------------------------------------------- sharded optimiser transport
// The flat fp32 gradient buffer of every rank lives at the same arena offset.  It is cut into buckets; inside a
// bucket of n elements starting at flat index `start`, rank r owns the sub-slice [start + r*per, start + (r+1)*per)
// (clipped to the bucket), per a multiple of 8.  Reduce-scatter: the owner reads its sub-slice of EVERY rank's
// gradient buffer in fp32 straight over NVLink (no staging copy, no cast), adds the values in rank order 0..N-1
// (one fixed order per element: bit-reproducible run to run and identical to what any other rank would compute),
// scales by 1/N and writes them to its shard-contiguous reduced-gradient buffer.  The loads of up to eight peers
// are issued before the first add so all links are busy at once.
__global__ void reduce_scatter_f32_kernel(const uint64_t* __restrict__ peers, long grad_off, long start, long n, long per,
                                          float* __restrict__ out, int world, int my_rank, float scale) {
  const long lo = per * my_rank, hi = min(n, lo + per);
  const long nvec = hi > lo ? (hi - lo) >> 2 : 0;               // every boundary is a multiple of 8 elements
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r0 = 0; r0 < world; r0 += 8) {
      float4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (r0 + j < world) v[j] = *((const float4*)(peers[r0 + j] + grad_off) + ((start + lo) >> 2) + i);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (r0 + j < world) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    ((float4*)out)[i] = acc;
  }
}

// All-gather by pulling: a buffer (bf16 compute copy of the matrices, or the fp32 copy of the vectors) that lives at
// the same arena offset on every rank is made whole on this rank by copying, for every bucket segment, the
// sub-slices the other ranks own from their arenas.  One segment per blockIdx.y.
struct GatherSeg {
  long elem_start;      // flat index of the segment's first element
  long elem_n;          // elements in the segment
  long bucket_start;    // flat index of the bucket's first element (ownership is counted from here)
  long per;             // elements per owner inside the bucket
};
__global__ void allgather_pull_kernel(const uint64_t* __restrict__ peers, long buf_off, long buf_elem0, int elem_bytes,
                                      const GatherSeg* __restrict__ segs, int world, int my_rank) {
  const GatherSeg sg = segs[blockIdx.y];
  const int epv = 16 / elem_bytes;                          // elements per 16-byte vector
  const long nvec = sg.elem_n / epv;
  const long stride = (long)gridDim.x * blockDim.x;
  const long seg_off = sg.elem_start - sg.bucket_start;     // a bucket has far fewer than 2^31 elements: 32-bit ownership math
  uint4* mine = (uint4*)(peers[my_rank] + buf_off);
  constexpr int U = 8;                                      // eight peer loads in flight per thread before the first store
  for (long i0 = blockIdx.x * (long)blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
    uint4 v[U];
    long at[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long i = i0 + u * stride;
      at[u] = -1;
      if (i < nvec) {
        const int owner = (int)((uint32_t)(seg_off + i * epv) / (uint32_t)sg.per);
        if (owner != my_rank && owner < world) {
          at[u] = ((sg.elem_start + i * epv - buf_elem0) * elem_bytes) >> 4;
          v[u] = *((const uint4*)(peers[owner] + buf_off) + at[u]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (at[u] >= 0) mine[at[u]] = v[u];
  }
}

// Cross-rank sum of one fp32 scalar per rank (the partial squared gradient norms): share_scalar stores this rank's
// value into slot [my_rank] of every rank's slot row; after a barrier sum_slots adds the N slots in rank order, so
// every rank obtains the same bits.
__global__ void share_scalar_kernel(const uint64_t* __restrict__ peers, long slot_off, const float* __restrict__ value,
                                    int world, int my_rank) {
  const int r = threadIdx.x;
  if (r < world) ((float*)(peers[r] + slot_off))[my_rank] = value[0];
}
__global__ void sum_slots_kernel(const float* __restrict__ slots, int world, float* __restrict__ out) {
  float s = 0.f;
  for (int r = 0; r < world; ++r) s += slots[r];
  out[0] = s;
}

// Deterministic dK/dV reduction of the fused ring ("pull" mode): every rank has written its contributions for the
// whole sequence into a local fp32 buffer at the same arena offset; the owner of a chunk adds the chunk's rows of
// the contributing ranks in rank order and writes bf16.  One segment per blockIdx.y.
struct PullSeg {
  long src_elem;        // first element of the chunk rows inside every rank's full-length buffer
  long dst_elem;        // first element inside the local output
  long n;               // elements (multiple of 8)
  unsigned int mask;    // bit s set: rank s contributes
  int pad;
};
__global__ void dkv_pull_reduce_kernel(const uint64_t* __restrict__ peers, long buf_off, const PullSeg* __restrict__ segs,
                                       __nv_bfloat16* __restrict__ out, int world) {
  const PullSeg sg = segs[blockIdx.y];
  const long nvec = sg.n >> 3;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      if (!((sg.mask >> r) & 1u)) continue;
      const float4* src = (const float4*)(peers[r] + buf_off) + ((sg.src_elem >> 2) + i * 2);
      const float4 a = src[0], b = src[1];
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    *((uint4*)(out + sg.dst_elem) + i) =
        make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
  }
}

static inline int grid_cap(size_t work, int block, int per_sm) {
  size_t g = (work + block - 1) / block;
  size_t cap = (size_t)sm_count() * per_sm;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace cpb

using namespace cpb;

extern "C" int cpb_barrier(const uint64_t* peers, long flag_off, int world, int my_rank, int epoch, double timeout_s,
                           int* status, cudaStream_t stream) {
  if (world > 32) return set_error(CPB_ERR_LIMIT, "barrier: at most 32 ranks");
  const long spins = (long)(timeout_s * 1e9 / 150.0) + 1000;
  barrier_kernel<<<1, 32, 0, stream>>>(peers, flag_off, world, my_rank, epoch, spins, status);
  return check_launch("barrier");
}

// segs: device array of CopySeg (see ring_copy.cuh), sorted by chunk; ready[chunk] += n_ctas when a chunk landed.
extern "C" int cpb_ring_gather(const void* segs, int n_segs, int* ready, int n_ctas, cudaStream_t stream) {
  if (n_segs <= 0) return CPB_OK;
  ring_gather_kernel<<<n_ctas, 256, 0, stream>>>((const CopySeg*)segs, n_segs, ready);
  return check_launch("ring_gather");
}

// parts: up to 3 entries of {src ptr, src token stride, n_local, rep, dst_head_off} passed as flat arrays.
extern "C" int cpb_a2a_push(const void* const* src, const long* src_tok_stride, const int* n_local, const int* rep,
                            const int* dst_head_off, int n_parts, int B, int Tl, int D, int P, int my_rank,
                            int dst_heads, long dst_off, const uint64_t* peers, cudaStream_t stream) {
  if (n_parts < 1 || n_parts > 3 || (D % 8)) return set_error(CPB_ERR_ARG, "a2a_push: bad arguments");
  A2AParams p;
  for (int i = 0; i < n_parts; ++i) {
    p.part[i].src = (const __nv_bfloat16*)src[i]; p.part[i].src_tok_stride = src_tok_stride[i];
    p.part[i].n_local = n_local[i]; p.part[i].rep = rep[i] < 1 ? 1 : rep[i]; p.part[i].dst_head_off = dst_head_off[i];
  }
  p.n_parts = n_parts; p.B = B; p.Tl = Tl; p.D = D; p.P = P; p.my_rank = my_rank; p.dst_heads = dst_heads;
  p.dst_off = dst_off; p.peers = peers;
  a2a_push_kernel<<<grid_cap((size_t)B * Tl * P, 8, 8), 256, 0, stream>>>(p);
  return check_launch("a2a_push");
}

extern "C" int cpb_a2a_pull(void* const* dst, const long* dst_tok_stride, const int* n_heads, const int* n_local,
                            const int* rep, const int* src_head_off, const int* src_heads, const long* src_off,
                            int n_parts, int B, int Tl, int D, int P, int my_rank, const uint64_t* peers,
                            cudaStream_t stream) {
  if (n_parts < 1 || n_parts > 3 || (D % 8) || D > 256) return set_error(CPB_ERR_ARG, "a2a_pull: bad arguments");
  A2APullParams p;
  size_t heads = 0;
  for (int i = 0; i < n_parts; ++i) {
    p.part[i].dst = (__nv_bfloat16*)dst[i]; p.part[i].dst_tok_stride = dst_tok_stride[i];
    p.part[i].n_heads = n_heads[i]; p.part[i].n_local = n_local[i]; p.part[i].rep = rep[i] < 1 ? 1 : rep[i];
    p.part[i].src_head_off = src_head_off[i]; p.part[i].src_heads = src_heads[i]; p.part[i].src_off = src_off[i];
    heads += n_heads[i];
  }
  p.n_parts = n_parts; p.B = B; p.Tl = Tl; p.D = D; p.P = P; p.my_rank = my_rank; p.peers = peers;
  a2a_pull_kernel<<<grid_cap((size_t)B * Tl * heads, 8, 8), 256, 0, stream>>>(p);
  return check_launch("a2a_pull");
}

extern "C" int cpb_a2a_push_rows_f32(const float* src, int B, int H, int Tl, int src_T, int n_local, int P, int my_rank,
                                     long dst_off, int dst_T, const uint64_t* peers, cudaStream_t stream) {
  a2a_push_rows_f32_kernel<<<grid_cap((size_t)B * H * Tl, 256, 8), 256, 0, stream>>>(src, B, H, Tl, src_T, n_local, P, my_rank, dst_off, dst_T, peers);
  return check_launch("a2a_push_rows_f32");
}

extern "C" int cpb_allreduce_reduce(const uint64_t* peers, long stage_off, float* grad, long n, int world, int my_rank,
                                    int n_ctas, cudaStream_t stream) {
  if (n <= 0) return CPB_OK;
  allreduce_reduce_kernel<<<n_ctas, 512, 0, stream>>>(peers, stage_off, grad, n, world, my_rank);
  return check_launch("allreduce_reduce");
}
extern "C" int cpb_allreduce_gather(const uint64_t* peers, long stage_off, float* grad, long n, int world, int my_rank,
                                    int n_ctas, cudaStream_t stream) {
  if (n <= 0) return CPB_OK;
  allreduce_gather_kernel<<<n_ctas, 512, 0, stream>>>(peers, stage_off, grad, n, world, my_rank);
  return check_launch("allreduce_gather");
}

extern "C" int cpb_reduce_scatter_f32(const uint64_t* peers, long grad_off, long start, long n, long per, float* out,
                                      int world, int my_rank, float scale, int n_ctas, cudaStream_t stream) {
  if (n <= 0) return CPB_OK;
  if ((start % 8) || (per % 8) || (n % 8) || per <= 0)
    return set_error(CPB_ERR_ARG, "reduce_scatter_f32: start, n and per must be multiples of 8 elements");
  reduce_scatter_f32_kernel<<<n_ctas < 1 ? 1 : n_ctas, 512, 0, stream>>>(peers, grad_off, start, n, per, out, world, my_rank, scale);
  return check_launch("reduce_scatter_f32");
}

// segs: device array of {elem_start, elem_n, bucket_start, per} (four longs each).
extern "C" int cpb_allgather_pull(const uint64_t* peers, long buf_off, long buf_elem0, int elem_bytes, const void* segs,
                                  int n_segs, int world, int my_rank, int ctas_per_seg, cudaStream_t stream) {
  if (n_segs <= 0) return CPB_OK;
  if (elem_bytes != 2 && elem_bytes != 4) return set_error(CPB_ERR_ARG, "allgather_pull: element size must be 2 or 4");
  if (n_segs > 65535) return set_error(CPB_ERR_LIMIT, "allgather_pull: at most 65535 segments");
  dim3 grid(ctas_per_seg < 1 ? 1 : ctas_per_seg, n_segs);
  allgather_pull_kernel<<<grid, 512, 0, stream>>>(peers, buf_off, buf_elem0, elem_bytes, (const GatherSeg*)segs, world, my_rank);
  return check_launch("allgather_pull");
}

extern "C" int cpb_share_scalar(const uint64_t* peers, long slot_off, const float* value, int world, int my_rank,
                                cudaStream_t stream) {
  if (world > 32) return set_error(CPB_ERR_LIMIT, "share_scalar: at most 32 ranks");
  share_scalar_kernel<<<1, 32, 0, stream>>>(peers, slot_off, value, world, my_rank);
  return check_launch("share_scalar");
}
extern "C" int cpb_sum_slots(const float* slots, int world, float* out, cudaStream_t stream) {
  sum_slots_kernel<<<1, 1, 0, stream>>>(slots, world, out);
  return check_launch("sum_slots");
}

// segs: device array of {src_elem, dst_elem, n, mask, pad} (three longs and two ints each).
extern "C" int cpb_dkv_pull_reduce(const uint64_t* peers, long buf_off, const void* segs, int n_segs, void* out, int world,
                                   int ctas_per_seg, cudaStream_t stream) {
  if (n_segs <= 0) return CPB_OK;
  if (world > 32) return set_error(CPB_ERR_LIMIT, "dkv_pull_reduce: at most 32 ranks");
  dim3 grid(ctas_per_seg < 1 ? 1 : ctas_per_seg, n_segs);
  dkv_pull_reduce_kernel<<<grid, 256, 0, stream>>>(peers, buf_off, (const PullSeg*)segs, (__nv_bfloat16*)out, world);
  return check_launch("dkv_pull_reduce");
}
