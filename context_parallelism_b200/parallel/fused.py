"""Fused communication + compute paths over NVLink peer memory (the product path on a B200 node).

``FusedComm`` owns one symmetric arena per rank (``parallel.symm``), the flag pads and the epoch
counters, and provides:

* ``ring_attention``     – one attention kernel per direction that also moves the K/V: a few of its CTAs
  pull the other ranks' K/V blocks into a position-ordered local buffer with peer loads while the
  tcgen05 tiles consume what has already landed (local diagonal chunk first); the online-softmax
  state persists across blocks, so there is no per-step merge.  Backward re-gathers K/V the same way
  and either pushes dK/dV tiles into their owners' fp32 accumulators with ``red.add`` straight from the
  gradient kernel's epilogue (``CP_DKV_MODE=route``, the default) or writes them to a local fp32 buffer
  that the owners then pull and add in rank order (``CP_DKV_MODE=pull``: bit-reproducible, like the
  reference's travelling accumulator, context_parallel/ContextParallelBackward.h:546-627).
* ``ulysses_attention``  – sequence→head exchange by peer stores into per-layer landing buffers, local
  attention whose epilogue stores each output row directly into the token owner's arena, and the mirrored
  backward (dO / delta pushed to head owners, dQ/dK/dV pulled back with KV-replica summation).
* the gradient transport – either the two-shot all-reduce with the bf16 cast and 1/N scale fused in
  (``allreduce_avg_``, replicated optimiser) or, by default, the transport of the sharded optimiser:
  ``reduce_scatter_bucket`` (fp32, read straight from the peers' gradient buffers), ``sum_over_ranks_`` (the
  squared norm) and ``allgather_params`` (``ops.optim``).

Every operation is a sequence of *phases* separated by cross-rank barriers; a phase only launches kernels
that never wait for another rank.  The autograd functions below run phase, barrier, phase, ...; the
single-GPU tests build one ``FusedComm`` per emulated rank over arenas on one device (``EmulatedHeap``,
barriers are no-ops) and run each phase for every rank in turn, which exercises every index formula, peer
table and kernel without a second GPU.

The NCCL rotators, ``all_to_all_single`` and ``all_reduce`` (``parallel.ring``, ``parallel.ulysses``,
``parallel.ddp``) remain as the measured baseline (``CP_ROTATOR=p2p|alltoall|allgather``).
"""
from __future__ import annotations

import ctypes
import functools
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native as nv
from ..ops import attention as A
from ..ops import attention_bwd as AB
from ..ops import permute
from ..utils.debug import DebugTools
from .symm import SymmetricHeap, tensor_from_ptr

N_COPY_CTAS = 16


@functools.lru_cache(maxsize=None)
def _gather_ctas(device) -> int:
    """CTAs of a stand-alone K/V gather (nothing else runs beside it): two per SM, so that enough peer loads are in flight to
    cover the NVLink latency."""
    return 2 * torch.cuda.get_device_properties(device).multi_processor_count
FLAG_BYTES = 4096


class EmulatedHeap:
    """``n`` arenas on ONE device standing in for the arenas of ``n`` ranks: ``for_rank(r)`` has the interface of
    ``SymmetricHeap`` with ``peer_bases`` pointing at the local arenas.  Sub-allocations must be made in the same
    order on every emulated rank, exactly like on real ranks."""

    def __init__(self, n: int, nbytes: int, device: torch.device):
        self.nbytes = (nbytes + 4095) // 4096 * 4096
        self.arenas = [torch.zeros(self.nbytes, dtype=torch.uint8, device=device) for _ in range(n)]
        self.bases = [a.data_ptr() for a in self.arenas]
        self.device = device

    def for_rank(self, r: int) -> "_EmulatedRankHeap":
        return _EmulatedRankHeap(self, r)


class _EmulatedRankHeap:
    emulated = True

    def __init__(self, parent: EmulatedHeap, rank: int):
        self.parent, self.rank, self.device = parent, rank, parent.device
        self.nbytes = parent.nbytes
        self.arena = parent.arenas[rank]
        self.base = parent.bases[rank]
        self.peer_bases = list(parent.bases)
        self._off = 0
        self._named: Dict[str, Tuple[int, int]] = {}

    alloc = SymmetricHeap.alloc
    view = SymmetricHeap.view
    tensor = SymmetricHeap.tensor
    raw_tensor = SymmetricHeap.raw_tensor

    def close(self) -> None:
        pass


class _Group:
    """A sub-group of the heap's ranks with its own peer table, flag row and barrier epoch."""

    def __init__(self, heap, ranks_in_heap: List[int], my_index: int, flag_off: int, device):
        self.heap, self.size, self.rank = heap, len(ranks_in_heap), my_index
        self.peer_list = [heap.peer_bases[r] for r in ranks_in_heap]
        self.peers = torch.tensor(self.peer_list, dtype=torch.int64, device=device)
        self.flag_off = flag_off
        self.epoch = 0


class FusedComm:
    def __init__(self, cfg, device: torch.device, heap, world_rank: int, world_size: int,
                 ring: Optional[Tuple[List[int], int]] = None, uly: Optional[Tuple[List[int], int]] = None,
                 world_group=None):
        """``ring`` / ``uly``: ``(ranks of the group inside the heap, this rank's index in it)``."""
        self.cfg, self.device, self.heap = cfg, device, heap
        self.world, self.rank = world_size, world_rank
        self.world_group = world_group
        self.ring_pg = None            # torch.distributed group of the ring axis (control plane of the debug tools)
        self.emulated = bool(getattr(heap, "emulated", False))
        flags_off = heap.alloc("flags", 4 * FLAG_BYTES)
        self.g_world = _Group(heap, list(range(world_size)), world_rank, flags_off, device)
        self.g_ring = _Group(heap, ring[0], ring[1], flags_off + FLAG_BYTES, device) if ring is not None else None
        self.g_uly = _Group(heap, uly[0], uly[1], flags_off + 2 * FLAG_BYTES, device) if uly is not None else None
        self.shard_world, self.shard_rank = world_size, world_rank
        self.timeout_s = min(cfg.watchdog_s, 20.0)
        self.dkv_mode = cfg.dkv_mode
        self.load_balance = cfg.load_balance or cfg.attn_mode == "hybrid"
        self.n_slots = max(cfg.n_layer, 2)
        # CP_SHARE_FWD_ROTATOR: one pair of published K/V slots for all layers instead of one per layer; backward then
        # publishes the layer's K/V again before it gathers (the reference shares one forward staging set across layers
        # the same way, Scripts/Blutrain/gpt2_cp_test.cpp:406-415)
        self.share_ring_slots = bool(cfg.share_fwd_rotator)
        self.ring_slots = 2 if self.share_ring_slots else self.n_slots
        self._ring_state: Dict[tuple, "_RingBuffers"] = {}
        self._uly_state: Dict[tuple, "_UlyssesBuffers"] = {}
        self._layer_counter = {"ring": 0, "uly": 0}      # one slot sequence per exchange (hybrid runs both in every layer)
        self._ar_stage_off: Optional[int] = None
        self.ar_ctas = int(os.environ.get("CP_AR_CTAS", "32"))
        self.dbg = DebugTools(cfg, world_rank)
        self.no_overlap_fwd = bool(cfg.debug.no_overlap or cfg.debug.no_overlap_fwd)

    # ------------------------------------------------------------------ construction
    @staticmethod
    def estimate_bytes(cfg, ctx, world: int) -> int:
        B, T, D = cfg.B, cfg.T, cfg.head_dim
        L = max(cfg.n_layer, 2)
        Lr = 2 if cfg.share_fwd_rotator else L
        Hq, Hkv = cfg.n_head, cfg.n_kv_head
        U = ctx.ulysses_size if cfg.attn_mode != "ring" else 1
        R = ctx.ring_size
        total = 64 << 20
        if R > 1:
            hkv = max(1, Hkv // (U if cfg.attn_mode == "hybrid" else 1))
            tl = T // R
            total += Lr * 2 * B * tl * hkv * D * 2           # published K/V slots
            total += 2 * B * T * hkv * D * 2                 # gathered K/V (shared)
            total += 2 * B * tl * hkv * D * 4                # dK/dV fp32 accumulators
            if cfg.dkv_mode == "pull":
                total += 2 * B * T * hkv * D * 4             # full-length local dK/dV contributions
        if U > 1:
            P = U
            tl = T // ctx.cp_size
            tt = tl * P
            hl = Hq // P + 2 * max(1, Hkv // P)
            total += L * B * tt * hl * D * 2                 # per-layer q/k/v landing
            total += L * B * tl * Hq * D * 2                 # per-layer o landing
            total += B * tt * (Hq // P) * D * 2              # dO landing
            total += B * (Hq // P) * (tt + 128 * P) * 4      # delta landing
            total += B * tt * hl * D * 2                     # dq/dk/dv staging
        n_params = cfg.n_layer * (cfg.n_embd * (Hq + 2 * Hkv) * D + Hq * D * cfg.n_embd
                                  + (3 if cfg.family == "llama" else 2) * cfg.n_embd * cfg.ffn_hidden + 16 * cfg.n_embd) \
            + 2 * cfg.vocab_padded * cfg.n_embd + (cfg.T + 1024) * cfg.n_embd + (1 << 22)
        # sharded optimiser: fp32 gradient + bf16 compute copy in the arena; replicated: bf16 gradient staging
        total += n_params * (6 if cfg.shard_optim else 2) + (64 << 20)
        return int(total * 1.05)

    @staticmethod
    def create(cfg, ctx, device) -> Optional["FusedComm"]:
        world = dist.get_world_size()
        if world > min(torch.cuda.device_count(), max(1, cfg.gpus_per_node)):
            return None            # more ranks than GPUs of one node (NO_GPUS_PER_NODE): not a single-node job, CUDA IPC does not apply
        heap = SymmetricHeap(None, FusedComm.estimate_bytes(cfg, ctx, world), device)
        mesh = ctx.mesh
        ring = uly = None
        if cfg.attn_mode == "ring":
            ring = (mesh.ranks("cp"), ctx.cp_rank)
        elif cfg.attn_mode == "ulysses":
            uly = (mesh.ranks("cp"), ctx.cp_rank)
        elif cfg.attn_mode == "hybrid":
            ring = (mesh.ranks("ring"), ctx.ring_rank)
            uly = (mesh.ranks("ulysses"), ctx.ulysses_rank)
        fc = FusedComm(cfg, device, heap, dist.get_rank(), world, ring, uly)
        fc.ring_pg = ctx.ring_group
        return fc

    def covers_world(self) -> bool:
        return True

    def supports_ring_group(self) -> bool:
        return self.g_ring is not None

    def close(self) -> None:
        self.heap.close()

    # ------------------------------------------------------------------ primitives
    def barrier(self, g: _Group, timeout_s: Optional[float] = None) -> None:
        """Cross-rank barrier kernel on the current stream (bounded wait; expiry lands in the status word)."""
        if self.emulated:
            return
        sync = self.cfg.debug.sync_ring
        if sync:
            torch.cuda.synchronize(self.device)
        g.epoch += 1
        st = nv.status_for(self.device)
        nv.call("barrier", nv.ptr(g.peers), nv.l(g.flag_off), nv.i(g.size), nv.i(g.rank), nv.i(g.epoch),
                ctypes.c_double(self.timeout_s if timeout_s is None else timeout_s), st.ptr(), nv.stream_ptr(self.device))
        if sync:
            torch.cuda.synchronize(self.device)

    def next_layer_slot(self, kind: str = "ring") -> int:
        """Per-layer buffer slot of the next forward call.  There are ``max(n_layer, 2)`` slots: a slot is rewritten
        two forward calls later at the earliest, i.e. after a barrier that every rank joined after its last read of
        the slot, also for one-layer models and forward-only loops."""
        s = self._layer_counter[kind] % (self.ring_slots if kind == "ring" else self.n_slots)
        self._layer_counter[kind] += 1
        return s

    # ------------------------------------------------------------------ gradient all-reduce (replicated optimiser)
    def grad_allreduce_for(self, flat) -> "FusedComm":
        if not flat.sharded:
            self._ar_stage_off = self.heap.alloc("grad_stage", flat.total * 2 + 64)
        self._ar_flat = flat
        return self

    def allreduce_avg_(self, buf: torch.Tensor, offset: int) -> None:
        """In-place average of a slice of the flat fp32 gradient buffer over all ranks.
        cast(grad/N)→bf16 staging | barrier | owner reduces its slice from every peer | barrier | gather.
        The wire format is bf16 (the reference all-reduces fp32); the owner keeps the same rounded values the other
        ranks gather, so the replicated optimiser states stay bit-identical."""
        g = self.g_world
        n = buf.numel()
        stage_off = self._ar_stage_off + offset * 2
        stage = self.heap.view(stage_off, (n,), torch.bfloat16)
        s = nv.stream_ptr(self.device)
        nv.call("cast_f32_bf16", nv.ptr(buf), nv.ptr(stage), nv.l(n), nv.f(1.0 / g.size), s)
        self.barrier(g)
        ctas = max(8, min(2 * self.ar_ctas, n // (1 << 16)))
        nv.call("allreduce_reduce", nv.ptr(g.peers), nv.l(stage_off), nv.ptr(buf), nv.l(n), nv.i(g.size), nv.i(g.rank), nv.i(ctas), s)
        self.barrier(g)
        nv.call("allreduce_gather", nv.ptr(g.peers), nv.l(stage_off), nv.ptr(buf), nv.l(n), nv.i(g.size), nv.i(g.rank), nv.i(ctas), s)

    def allreduce_finish(self) -> None:
        """Closing barrier after the last bucket of a step: no rank may overwrite its gradient buffer (or staging
        slices) with the next step's gradients while a slower rank is still reading from them."""
        self.barrier(self.g_world)

    # ------------------------------------------------------------------ sharded optimiser transport
    def reduce_scatter_launch(self, flat, b: int) -> None:
        """The kernel of ``reduce_scatter_bucket`` alone (no barrier)."""
        g = self.g_world
        s, n, per, off = flat.plan.buckets[b]
        ctas = max(4, min(self.ar_ctas, per // (1 << 13)))
        nv.call("reduce_scatter_f32", nv.ptr(g.peers), nv.l(flat.grad_off), nv.l(s), nv.l(n), nv.l(per),
                nv.ptr(flat.gshard[off:]), nv.i(g.size), nv.i(g.rank), nv.f(1.0 / g.size), nv.i(ctas), nv.stream_ptr(self.device))

    def reduce_scatter_bucket(self, flat, b: int) -> None:
        """Average bucket ``b`` of the flat fp32 gradient over all ranks into this rank's shard: after a barrier
        (every rank's gradients of the bucket are final) the owner of each sub-slice reads it from every rank's
        gradient buffer over NVLink, fp32 on the wire, fixed summation order."""
        self.barrier(self.g_world)
        self.reduce_scatter_launch(flat, b)

    def share_scalar_launch(self, value: torch.Tensor, slots_off: int) -> None:
        g = self.g_world
        nv.call("share_scalar", nv.ptr(g.peers), nv.l(slots_off), nv.ptr(value), nv.i(g.size), nv.i(g.rank), nv.stream_ptr(self.device))

    def sum_slots_launch(self, value: torch.Tensor, slots: torch.Tensor) -> None:
        nv.call("sum_slots", nv.ptr(slots), nv.i(self.g_world.size), nv.ptr(value), nv.stream_ptr(self.device))

    def sum_over_ranks_(self, value: torch.Tensor, slots_off: int, slots: torch.Tensor) -> None:
        """``value[0]`` (fp32, device) becomes the sum of every rank's value, added in rank order (same bits on
        every rank)."""
        self.share_scalar_launch(value, slots_off)
        self.barrier(self.g_world)
        self.sum_slots_launch(value, slots)

    def allgather_launch(self, flat) -> None:
        g = self.g_world
        s = nv.stream_ptr(self.device)
        if flat._g16_segs is not None:
            nv.call("allgather_pull", nv.ptr(g.peers), nv.l(flat.p16_off), nv.l(0), nv.i(2), nv.ptr(flat._g16_segs),
                    nv.i(flat._g16_segs.shape[0]), nv.i(g.size), nv.i(g.rank), nv.i(max(1, self.ar_ctas // 2)), s)
        if flat._g32_segs is not None:
            nv.call("allgather_pull", nv.ptr(g.peers), nv.l(flat.p32_off), nv.l(flat.n_decay), nv.i(4), nv.ptr(flat._g32_segs),
                    nv.i(flat._g32_segs.shape[0]), nv.i(g.size), nv.i(g.rank), nv.i(4), s)

    def allgather_params(self, flat) -> None:
        """After the owners' AdamW: every rank pulls the other ranks' slices of the bf16 (matrices) and fp32
        (vectors) compute copies."""
        self.barrier(self.g_world)
        self.allgather_launch(flat)

    # ------------------------------------------------------------------ ring
    def ring_attention(self, q, k, v, pos, T: int, scale: float) -> torch.Tensor:
        return _FusedRingFn.apply(q, k, v, pos, self, T, scale)

    # ------------------------------------------------------------------ ulysses
    def ulysses_attention(self, q, k, v, scale: float) -> torch.Tensor:
        return _FusedUlyssesFn.apply(q, k, v, self, scale)


# ============================================================================ ring
def ring_chunk_owner(c: int, N: int, load_balance: bool = True) -> Tuple[int, int]:
    """``(owner, half)`` of chunk c of the 2N position-ordered chunks.  HeadTail: rank c's first half (c < N) or
    rank 2N-1-c's second half.  Contiguous shards (``CP_LOAD_BALANCE=0``): rank c // 2, half c % 2."""
    if not load_balance:
        return c // 2, c % 2
    return (c, 0) if c < N else (2 * N - 1 - c, 1)


def ring_rank_chunks(r: int, N: int, load_balance: bool = True) -> List[int]:
    """The two chunks rank r owns (first half, second half)."""
    return [r, 2 * N - 1 - r] if load_balance else [2 * r, 2 * r + 1]


class _RingBuffers:
    """Symmetric buffers and tables of the fused ring for one problem shape."""

    def __init__(self, fc: FusedComm, B: int, Tl: int, Hkv: int, D: int):
        g, heap, dev = fc.g_ring, fc.heap, fc.device
        N, r = g.size, g.rank
        L = fc.ring_slots
        T = Tl * N
        self.B, self.Tl, self.Hkv, self.D, self.T, self.N = B, Tl, Hkv, D, T, N
        self.cs = Tl // 2
        self.lb = fc.load_balance
        tag = f"ring{B}x{Tl}x{Hkv}x{D}"
        blk_bytes = 2 * B * Tl * Hkv * D * 2
        self.pub_off = heap.alloc(tag + ".kvpub", L * blk_bytes)
        self.pub_bytes = blk_bytes
        self.gathered, _ = heap.tensor(tag + ".gathered", (2, B, T, Hkv, D), torch.bfloat16)
        self.dkv_acc, self.acc_off = heap.tensor(tag + ".dkvacc", (2, B, Tl, Hkv, D), torch.float32)
        self.dkv_full = self.full_off = None
        if fc.dkv_mode == "pull":
            self.dkv_full, self.full_off = heap.tensor(tag + ".dkvfull", (2, B, T, Hkv, D), torch.float32)
        self.ready = torch.zeros(2 * N, dtype=torch.int32, device=dev)
        self.ready_bwd = torch.zeros(2 * N, dtype=torch.int32, device=dev)
        self.gather_calls = 0
        self.peer_bases = list(g.peer_list)
        self._segs: Dict[int, torch.Tensor] = {}
        # chunk c (of 2N, cs rows each) is owned by rank c (head) or 2N-1-c (tail) at local row 0 or cs
        cs = self.cs
        rk, rv = [], []
        row_bytes = Hkv * D * 4
        for c in range(2 * N):
            owner, half = ring_chunk_owner(c, N, self.lb)
            lrow0 = half * cs
            base = self.peer_bases[owner] + self.acc_off
            rk.append(base + lrow0 * row_bytes)
            rv.append(base + B * Tl * row_bytes + lrow0 * row_bytes)
        self.route = (torch.tensor(rk, dtype=torch.int64, device=dev), torch.tensor(rv, dtype=torch.int64, device=dev), cs, Tl)
        # copy order: the two local chunks first, then the others in position order
        mine = ring_rank_chunks(r, N, self.lb)
        self.chunk_order = mine + [c for c in range(2 * N) if c not in mine]
        # deterministic reduction: rank s contributes to chunk c iff some query of s can see it, i.e. its last chunk
        # is not before c
        self._pull_segs = None
        if fc.dkv_mode == "pull":
            rows = []
            row_el = Hkv * D
            for half, c in enumerate(mine):
                mask = 0
                for s in range(N):
                    if ring_rank_chunks(s, N, self.lb)[1] >= c:
                        mask |= 1 << s
                for kv in range(2):
                    for b in range(B):
                        rows.append([((kv * B + b) * T + c * cs) * row_el, ((kv * B + b) * Tl + half * cs) * row_el, cs * row_el, mask])
            self._pull_segs = torch.tensor(rows, dtype=torch.int64, device=dev)
            # {long, long, long, uint32 mask, int pad}: the mask sits in the low half of the fourth 8-byte word

    def pub_view(self, fc: FusedComm, slot: int) -> torch.Tensor:
        return fc.heap.view(self.pub_off + slot * self.pub_bytes, (2, self.B, self.Tl, self.Hkv, self.D), torch.bfloat16)

    def segs(self, fc: FusedComm, slot: int) -> torch.Tensor:
        t = self._segs.get(slot)
        if t is None:
            B, Tl, Hkv, D, T, N, cs = self.B, self.Tl, self.Hkv, self.D, self.T, self.N, self.cs
            row = Hkv * D * 2
            rows = []
            gbase = self.gathered.data_ptr()
            for c in self.chunk_order:
                owner, half = ring_chunk_owner(c, N, self.lb)
                lrow0 = half * cs
                src0 = self.peer_bases[owner] + self.pub_off + slot * self.pub_bytes
                for kv in range(2):
                    for b in range(B):
                        src = src0 + ((kv * B + b) * Tl + lrow0) * row
                        dst = gbase + ((kv * B + b) * T + c * cs) * row
                        rows.append([src, dst, cs * row // 16, c])
            t = self._segs[slot] = torch.tensor(rows, dtype=torch.int64, device=fc.device)
        return t


def _ring_buffers(fc: FusedComm, k: torch.Tensor) -> _RingBuffers:
    B, Tl, Hkv, D = k.shape
    key = (B, Tl, Hkv, D)
    rb = fc._ring_state.get(key)
    if rb is None:
        if Tl % 2 or ((Tl // 2) * Hkv * D * 2) % 16:
            raise ValueError("fused ring: local sequence must split into two 16-byte aligned chunks")
        rb = fc._ring_state[key] = _RingBuffers(fc, B, Tl, Hkv, D)
    return rb


# phases of the fused ring (each launches only kernels that never wait for another rank)
def ring_fwd_publish(fc: FusedComm, k, v) -> Tuple[_RingBuffers, int]:
    """Pack this rank's K/V block into its published per-layer slot, where the peers' copy CTAs read it."""
    rb = _ring_buffers(fc, k)
    slot = fc.next_layer_slot("ring")
    permute.kv_pack(k, v, out=rb.pub_view(fc, slot))
    return rb, slot


def ring_fwd_compute(fc: FusedComm, rb: _RingBuffers, slot: int, q, pos32, scale: float):
    """ONE attention launch: its first CTAs gather every rank's chunks into the position-ordered local buffer while
    the compute CTAs consume what has landed."""
    segs = rb.segs(fc, slot)
    if fc.no_overlap_fwd:
        # diagnostics (CP_NO_OVERLAP[_FWD]): the gather is a launch of its own that finishes before attention starts
        nv.call("ring_gather", nv.ptr(segs), nv.i(segs.shape[0]), nv.ptr(rb.ready_bwd), nv.i(_gather_ctas(q.device)), nv.stream_ptr(q.device))
        return A.flash_fwd(q, rb.gathered[0], rb.gathered[1], scale, True, pos32, 0)
    rb.gather_calls += 1
    return A.flash_fwd(q, rb.gathered[0], rb.gathered[1], scale, True, pos32, 0,
                       ready=rb.ready, ready_epoch=rb.gather_calls * N_COPY_CTAS, block_rows=rb.cs,
                       segs=segs, n_segs=segs.shape[0], n_copy=N_COPY_CTAS)


def ring_fwd_settled(fc: FusedComm, rb: _RingBuffers, q, pos32, scale: float):
    """The forward again on the K/V that ``ring_fwd_compute`` gathered, with nothing in flight and the same tile order
    (the reference computation of ``CP_SELFCHECK``)."""
    if fc.no_overlap_fwd:
        return A.flash_fwd(q, rb.gathered[0], rb.gathered[1], scale, True, pos32, 0)
    return A.flash_fwd(q, rb.gathered[0], rb.gathered[1], scale, True, pos32, 0,
                       ready=rb.ready, ready_epoch=rb.gather_calls * N_COPY_CTAS, block_rows=rb.cs)


def ring_kv_checksums(fc: FusedComm, rb: _RingBuffers, slot: int):
    """``(sent [2,2], received [2N,2], owners)`` for ``DebugTools.compare_kv``."""
    cs, N = rb.cs, rb.N
    pub = rb.pub_view(fc, slot)
    sent = torch.stack([DebugTools.checksum(pub[:, :, h * cs:(h + 1) * cs]) for h in range(2)])
    received = torch.stack([DebugTools.checksum(rb.gathered[:, :, c * cs:(c + 1) * cs]) for c in range(2 * N)])
    return sent, received, [ring_chunk_owner(c, N, rb.lb) for c in range(2 * N)]


def ring_bwd_prepare(fc: FusedComm, rb: _RingBuffers) -> None:
    (rb.dkv_full if fc.dkv_mode == "pull" else rb.dkv_acc).zero_()


def ring_bwd_compute(fc: FusedComm, rb: _RingBuffers, slot: int, q, out, lse, do, pos32, scale: float) -> torch.Tensor:
    """Re-gather K/V, then the gradient kernel; dK/dV tiles go to their owners' accumulators (``route``) or into the
    local full-length buffer (``pull``).  Returns dQ (bf16)."""
    dev = q.device
    B, Tl, Hq, D = q.shape
    segs = rb.segs(fc, slot)
    nv.call("ring_gather", nv.ptr(segs), nv.i(segs.shape[0]), nv.ptr(rb.ready_bwd), nv.i(_gather_ctas(dev)), nv.stream_ptr(dev))
    delta, lse2 = AB.flash_bwd_prep(out, do, lse)
    qpos_pad = AB.padded_q_pos(Tl, dev, pos32)
    dq = torch.zeros((B, Tl, Hq, D), dtype=torch.float32, device=dev)
    if fc.dkv_mode == "pull":
        AB.flash_bwd_core(q, rb.gathered[0], rb.gathered[1], do, lse2, delta, qpos_pad, scale, True, 0, dq,
                          rb.dkv_full[0], rb.dkv_full[1], True)
    else:
        AB.flash_bwd_core(q, rb.gathered[0], rb.gathered[1], do, lse2, delta, qpos_pad, scale, True, 0, dq, None, None, True,
                          route=rb.route)
    return AB.cast_to_bf16(dq)


def ring_bwd_finish(fc: FusedComm, rb: _RingBuffers) -> torch.Tensor:
    """dK/dV of this rank's block ``[2,B,Tl,Hkv,D]`` (bf16) once every rank's contributions are in place."""
    if fc.dkv_mode != "pull":
        return AB.cast_to_bf16(rb.dkv_acc)
    g = fc.g_ring
    dkv = torch.empty((2, rb.B, rb.Tl, rb.Hkv, rb.D), dtype=torch.bfloat16, device=fc.device)
    nv.call("dkv_pull_reduce", nv.ptr(g.peers), nv.l(rb.full_off), nv.ptr(rb._pull_segs), nv.i(rb._pull_segs.shape[0]),
            nv.ptr(dkv), nv.i(g.size), nv.i(16), nv.stream_ptr(fc.device))
    return dkv


class _FusedRingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, pos, fc: FusedComm, T: int, scale: float):
        dbg = fc.dbg
        call = dbg.next_call("ring") if dbg.active else 0
        dbg.drain(1)
        rb, slot = ring_fwd_publish(fc, k, v)
        fc.barrier(fc.g_ring)
        pos32 = pos.to(torch.int32)
        out, lse = ring_fwd_compute(fc, rb, slot, q, pos32, scale)
        if dbg.active:
            dbg.shapes("fused ring forward", q=q, k=k, v=v, out=out, lse=lse)
            dbg.sync_if(dbg.d.fwd_sync_recv)
            dbg.drain(2)
            if dbg.d.selfcheck:
                dbg.selfcheck("fused ring forward", call, {"out": out, "lse": lse},
                              lambda: dict(zip(("out", "lse"), ring_fwd_settled(fc, rb, q, pos32, scale))))
            if dbg.want_kv_check(call):
                torch.cuda.synchronize(fc.device)
                sent, received, owners = ring_kv_checksums(fc, rb, slot)
                dbg.compare_kv(call, sent, received, owners, fc.ring_pg)
            dbg.dump(dbg.d.dump_cp_out, "cp_out", call, out=out, lse=lse)
            dbg.sync_if(dbg.d.fwd_sync_return)
        # The slot travels as a (host) saved tensor, not as a ctx attribute: under activation recomputation backward
        # runs on the ORIGINAL ctx with the saved tensors of the re-run forward, and the re-run published into a new slot.
        slot_t = torch.tensor([slot], dtype=torch.int64)
        if fc.share_ring_slots:
            ctx.save_for_backward(q, out, lse, pos32, slot_t, k, v)
        else:
            ctx.save_for_backward(q, out, lse, pos32, slot_t)
        ctx.fc, ctx.rb, ctx.scale = fc, rb, scale
        return out

    @staticmethod
    def backward(ctx, do):
        saved = ctx.saved_tensors          # read exactly once: under activation recomputation a second read is an error
        q, out, lse, pos32, slot_t = saved[:5]
        fc, rb, scale = ctx.fc, ctx.rb, ctx.scale
        slot = int(slot_t.item())
        do = do.contiguous()
        if fc.share_ring_slots:
            rb, slot = ring_fwd_publish(fc, saved[5], saved[6])
        ring_bwd_prepare(fc, rb)
        fc.barrier(fc.g_ring)                  # every accumulator is zero, every published K/V is still in place
        dq = ring_bwd_compute(fc, rb, slot, q, out, lse, do, pos32, scale)
        fc.barrier(fc.g_ring)                  # every rank's contributions have landed
        dkv = ring_bwd_finish(fc, rb)
        if fc.dkv_mode == "pull":
            fc.barrier(fc.g_ring)              # nobody zeroes its contribution buffer while a peer still pulls from it
        fc.dbg.drain(3)
        return dq, dkv[0], dkv[1], None, None, None, None


# ============================================================================ ulysses
class _UlyssesBuffers:
    def __init__(self, fc: FusedComm, B: int, Tl: int, Hq: int, Hkv: int, D: int):
        g, heap = fc.g_uly, fc.heap
        P = g.size
        L = fc.n_slots
        self.B, self.Tl, self.Hq, self.Hkv, self.D, self.P = B, Tl, Hq, Hkv, D, P
        self.T = T = Tl * P
        self.nq = Hq // P
        self.kvl = Hkv // P if Hkv >= P else 1
        self.rep = 1 if Hkv >= P else P // Hkv
        self.hl = self.nq + 2 * self.kvl
        self.t_pad = (T + 127) // 128 * 128
        tag = f"uly{B}x{Tl}x{Hq}x{Hkv}x{D}"
        self.qkv_bytes = B * T * self.hl * D * 2
        self.qkv_off = heap.alloc(tag + ".qkv", L * self.qkv_bytes)
        self.o_bytes = B * Tl * Hq * D * 2
        self.o_off = heap.alloc(tag + ".o", L * self.o_bytes)
        self.do, self.do_off = heap.tensor(tag + ".do", (B, T, self.nq, D), torch.bfloat16)
        self.delta, self.delta_off = heap.tensor(tag + ".delta", (B, self.nq, self.t_pad), torch.float32)
        self.dq, self.dq_off = heap.tensor(tag + ".dq", (B, T, self.nq, D), torch.bfloat16)
        self.dk, self.dk_off = heap.tensor(tag + ".dk", (B, T, self.kvl, D), torch.bfloat16)
        self.dv, self.dv_off = heap.tensor(tag + ".dv", (B, T, self.kvl, D), torch.bfloat16)
        self.qpos_pad = AB.padded_q_pos(T, fc.device, None)

    def qkv_view(self, fc, slot):
        return fc.heap.view(self.qkv_off + slot * self.qkv_bytes, (self.B, self.T, self.hl, self.D), torch.bfloat16)

    def o_view(self, fc, slot):
        return fc.heap.view(self.o_off + slot * self.o_bytes, (self.B, self.Tl, self.Hq, self.D), torch.bfloat16)

    def heads(self, fc, slot):
        land = self.qkv_view(fc, slot)
        return land[:, :, :self.nq], land[:, :, self.nq:self.nq + self.kvl], land[:, :, self.nq + self.kvl:]


def _uly_buffers(fc: FusedComm, q, k) -> _UlyssesBuffers:
    B, Tl, Hq, D = q.shape
    Hkv = k.shape[2]
    key = (B, Tl, Hq, Hkv, D)
    ub = fc._uly_state.get(key)
    if ub is None:
        ub = fc._uly_state[key] = _UlyssesBuffers(fc, B, Tl, Hq, Hkv, D)
    return ub


def _carr(ctype, vals):
    return (ctype * len(vals))(*vals)


def _a2a_push(fc: FusedComm, g: _Group, parts, B, Tl, D, dst_heads, dst_off):
    """parts: list of (tensor view [B,Tl,h,D], n_local, rep, dst_head_off)."""
    srcs = _carr(ctypes.c_void_p, [p[0].data_ptr() for p in parts])
    strides = _carr(ctypes.c_long, [p[0].stride(1) for p in parts])
    for p in parts:
        assert p[0].stride(3) == 1 and p[0].stride(2) == D and p[0].stride(0) == Tl * p[0].stride(1)
    nv.call("a2a_push", srcs, strides, _carr(ctypes.c_int, [p[1] for p in parts]), _carr(ctypes.c_int, [p[2] for p in parts]),
            _carr(ctypes.c_int, [p[3] for p in parts]), nv.i(len(parts)), nv.i(B), nv.i(Tl), nv.i(D), nv.i(g.size), nv.i(g.rank),
            nv.i(dst_heads), nv.l(dst_off), nv.ptr(g.peers), nv.stream_ptr(fc.device))


def _a2a_pull(fc: FusedComm, g: _Group, parts, B, Tl, D):
    """parts: list of (dst view [B,Tl,h,D], n_heads, n_local, rep, src_head_off, src_heads, src_off)."""
    for p in parts:
        assert p[0].stride(3) == 1 and p[0].stride(2) == D and p[0].stride(0) == Tl * p[0].stride(1)
    nv.call("a2a_pull", _carr(ctypes.c_void_p, [p[0].data_ptr() for p in parts]), _carr(ctypes.c_long, [p[0].stride(1) for p in parts]),
            _carr(ctypes.c_int, [p[1] for p in parts]), _carr(ctypes.c_int, [p[2] for p in parts]), _carr(ctypes.c_int, [p[3] for p in parts]),
            _carr(ctypes.c_int, [p[4] for p in parts]), _carr(ctypes.c_int, [p[5] for p in parts]), _carr(ctypes.c_long, [p[6] for p in parts]),
            nv.i(len(parts)), nv.i(B), nv.i(Tl), nv.i(D), nv.i(g.size), nv.i(g.rank), nv.ptr(g.peers), nv.stream_ptr(fc.device))


def _seq_layout(t: torch.Tensor, Tl: int, D: int) -> torch.Tensor:
    ok = t.stride(3) == 1 and t.stride(2) == D and t.stride(0) == Tl * t.stride(1) and t.data_ptr() % 16 == 0 and (t.stride(1) * 2) % 16 == 0
    return t if ok else t.contiguous()


# phases of the fused Ulysses attention
def uly_fwd_push(fc: FusedComm, q, k, v) -> Tuple[_UlyssesBuffers, int]:
    """sequence -> head: peer stores straight into the head owners' landing buffers."""
    ub = _uly_buffers(fc, q, k)
    slot = fc.next_layer_slot("uly")
    B, Tl, D = ub.B, ub.Tl, ub.D
    q, k, v = _seq_layout(q, Tl, D), _seq_layout(k, Tl, D), _seq_layout(v, Tl, D)
    _a2a_push(fc, fc.g_uly, [(q, ub.nq, 1, 0), (k, ub.kvl, ub.rep, ub.nq), (v, ub.kvl, ub.rep, ub.nq + ub.kvl)],
              B, Tl, D, ub.hl, ub.qkv_off + slot * ub.qkv_bytes)
    return ub, slot


def uly_fwd_compute(fc: FusedComm, ub: _UlyssesBuffers, slot: int, scale: float) -> torch.Tensor:
    """Local attention over the full sequence for this rank's heads; the epilogue stores every row into its token
    owner's arena.  Returns the LSE."""
    g = fc.g_uly
    qh, kh, vh = ub.heads(fc, slot)
    _, lse = A.flash_fwd(qh, kh, vh, scale, True,
                         o_scatter=(g.peers, ub.o_off + slot * ub.o_bytes, ub.Tl, g.rank * ub.nq, ub.Hq))
    return lse


def uly_bwd_push(fc: FusedComm, ub: _UlyssesBuffers, slot: int, do: torch.Tensor) -> None:
    """delta = rowsum(dO∘O) where the tokens live, then dO and delta go to the head owners."""
    g = fc.g_uly
    B, Tl, Hq, D = ub.B, ub.Tl, ub.Hq, ub.D
    delta = AB.flash_bwd_delta(ub.o_view(fc, slot), do)                     # [B,Hq,Tl_pad]
    _a2a_push(fc, g, [(do, ub.nq, 1, 0)], B, Tl, D, ub.nq, ub.do_off)
    nv.call("a2a_push_rows_f32", nv.ptr(delta), nv.i(B), nv.i(Hq), nv.i(Tl), nv.i(delta.shape[-1]), nv.i(ub.nq), nv.i(g.size),
            nv.i(g.rank), nv.l(ub.delta_off), nv.i(ub.t_pad), nv.ptr(g.peers), nv.stream_ptr(fc.device))


def uly_bwd_compute(fc: FusedComm, ub: _UlyssesBuffers, slot: int, lse: torch.Tensor, scale: float) -> None:
    dev = fc.device
    lse2 = AB.flash_bwd_lse2(lse, ub.D)
    qh, kh, vh = ub.heads(fc, slot)
    dq32 = torch.zeros((ub.B, ub.T, ub.nq, ub.D), dtype=torch.float32, device=dev)
    AB.flash_bwd_core(qh, kh, vh, ub.do, lse2, ub.delta, ub.qpos_pad, scale, True, 0, dq32, ub.dk, ub.dv, False)
    nv.call("cast_f32_bf16", nv.ptr(dq32), nv.ptr(ub.dq), nv.l(dq32.numel()), nv.f(1.0), nv.stream_ptr(dev))


def uly_bwd_pull(fc: FusedComm, ub: _UlyssesBuffers):
    """head -> sequence: pull this rank's tokens of every head from the head owners, summing KV replicas."""
    B, Tl, Hq, Hkv, D = ub.B, ub.Tl, ub.Hq, ub.Hkv, ub.D
    dqkv = torch.empty((B, Tl, Hq + 2 * Hkv, D), dtype=torch.bfloat16, device=fc.device)
    dq, dk, dv = dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hkv], dqkv[:, :, Hq + Hkv:]
    _a2a_pull(fc, fc.g_uly, [(dq, Hq, ub.nq, 1, 0, ub.nq, ub.dq_off), (dk, Hkv, ub.kvl, ub.rep, 0, ub.kvl, ub.dk_off),
                             (dv, Hkv, ub.kvl, ub.rep, 0, ub.kvl, ub.dv_off)], B, Tl, D)
    return dq, dk, dv


class _FusedUlyssesFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, fc: FusedComm, scale: float):
        g = fc.g_uly
        dbg = fc.dbg
        call = dbg.next_call("ulysses") if dbg.active else 0
        dbg.drain(1)
        ub, slot = uly_fwd_push(fc, q, k, v)
        fc.barrier(g)
        dbg.sync_if(dbg.d.fwd_sync_recv)
        lse = uly_fwd_compute(fc, ub, slot, scale)
        fc.barrier(g)
        out = ub.o_view(fc, slot)
        if dbg.active:
            dbg.shapes("fused ulysses forward", q=q, k=k, v=v, out=out, lse=lse)
            dbg.drain(2)
            if dbg.d.selfcheck:
                def again():
                    lse2 = uly_fwd_compute(fc, ub, slot, scale)
                    fc.barrier(g)
                    return {"out": ub.o_view(fc, slot), "lse": lse2}
                dbg.selfcheck("fused ulysses forward", call, {"out": out, "lse": lse}, again)
            dbg.dump(dbg.d.dump_cp_out, "cp_out", call, out=out, lse=lse)
            dbg.sync_if(dbg.d.fwd_sync_return)
        ctx.save_for_backward(lse, torch.tensor([slot], dtype=torch.int64))     # slot as a saved tensor: see _FusedRingFn
        ctx.fc, ctx.ub, ctx.scale = fc, ub, scale
        return out

    @staticmethod
    def backward(ctx, do):
        lse, slot_t = ctx.saved_tensors
        fc, ub, scale = ctx.fc, ctx.ub, ctx.scale
        slot = int(slot_t.item())
        g = fc.g_uly
        uly_bwd_push(fc, ub, slot, do.contiguous())
        fc.barrier(g)
        uly_bwd_compute(fc, ub, slot, lse, scale)
        fc.barrier(g)
        dq, dk, dv = uly_bwd_pull(fc, ub)
        fc.dbg.drain(3)
        return dq, dk, dv, None, None


# ============================================================================ hybrid: the Ulysses exchange on its own
class _FusedSeqToHeadFn(torch.autograd.Function):
    """``[B, Tl, H, D]`` (this rank's tokens, all heads) -> ``[B, Tl*P, H/P, D]`` (the whole ring block, this rank's
    heads) for q, k and v at once, by peer stores into the head owners' per-layer landing buffers; the adjoint pulls
    the gradients back (the exchange that ``hybrid_attention`` wraps around ring attention,
    context_parallel/ContextParallel.h:1359-1396)."""

    @staticmethod
    def forward(ctx, q, k, v, fc: FusedComm):
        g = fc.g_uly
        ub, slot = uly_fwd_push(fc, q, k, v)
        fc.barrier(g)
        # a tensor object of its own over the landing buffer: views of the shared arena tensor would share its version
        # counter, and any later in-place copy into the arena would invalidate them for autograd
        base = fc.heap.base + ub.qkv_off + slot * ub.qkv_bytes
        land = tensor_from_ptr(base, ub.qkv_bytes, fc.device).view(torch.bfloat16).view(ub.B, ub.T, ub.hl, ub.D)
        ctx.fc, ctx.ub = fc, ub
        return land[:, :, :ub.nq], land[:, :, ub.nq:ub.nq + ub.kvl], land[:, :, ub.nq + ub.kvl:]

    @staticmethod
    def backward(ctx, dqh, dkh, dvh):
        fc, ub = ctx.fc, ctx.ub
        ub.dq.copy_(dqh)
        ub.dk.copy_(dkh)
        ub.dv.copy_(dvh)
        fc.barrier(fc.g_uly)
        dq, dk, dv = uly_bwd_pull(fc, ub)
        return dq, dk, dv, None


class _FusedHeadToSeqFn(torch.autograd.Function):
    """The reverse exchange for the attention output: ``[B, Tl*P, Hq/P, D]`` -> ``[B, Tl, Hq, D]``: the output is staged
    in the arena, and every token owner pulls its rows of every head; the adjoint pushes dO to the head owners."""

    @staticmethod
    def forward(ctx, oh, fc: FusedComm, ub: "_UlyssesBuffers"):
        g = fc.g_uly
        B, Tl, Hq, D = ub.B, ub.Tl, ub.Hq, ub.D
        ub.dq.copy_(oh)                     # the dQ staging buffer has the shape of the per-head-slice output; forward and backward never overlap
        fc.barrier(g)
        out = torch.empty((B, Tl, Hq, D), dtype=torch.bfloat16, device=fc.device)
        _a2a_pull(fc, g, [(out, Hq, ub.nq, 1, 0, ub.nq, ub.dq_off)], B, Tl, D)
        ctx.fc, ctx.ub = fc, ub
        return out

    @staticmethod
    def backward(ctx, do):
        fc, ub = ctx.fc, ctx.ub
        g = fc.g_uly
        do = do.contiguous()
        _a2a_push(fc, g, [(do, ub.nq, 1, 0)], ub.B, ub.Tl, ub.D, ub.nq, ub.do_off)
        fc.barrier(g)
        return tensor_from_ptr(fc.heap.base + ub.do_off, ub.do.numel() * 2, fc.device).view(torch.bfloat16).view(ub.do.shape), None, None


def fused_seq_to_head(fc: FusedComm, q, k, v):
    qh, kh, vh = _FusedSeqToHeadFn.apply(q, k, v, fc)
    ub = fc._uly_state[(q.shape[0], q.shape[1], q.shape[2], k.shape[2], q.shape[3])]
    return qh, kh, vh, ub


def fused_head_to_seq(fc: FusedComm, oh, ub):
    return _FusedHeadToSeqFn.apply(oh, fc, ub)
