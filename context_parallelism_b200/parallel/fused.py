"""Fused communication + compute paths over NVLink peer memory (the product path on a B200 node).

``FusedComm`` owns one symmetric arena per rank (``parallel.symm``), the flag pads and the epoch
counters, and provides:

* ``ring_attention``     – one attention kernel per direction that also moves the K/V: a few of its CTAs
  pull the other ranks' K/V blocks into a position-ordered local buffer with peer loads while the
  tcgen05 tiles consume what has already landed (local diagonal chunk first); the online-softmax
  state persists across blocks, so there is no per-step merge.  Backward re-gathers K/V the same way
  and pushes dK/dV tiles into their owners' fp32 accumulators with ``red.add`` straight from the
  gradient kernel's epilogue.
* ``ulysses_attention``  – sequence→head exchange by peer stores into per-layer landing buffers, local
  attention whose epilogue stores each output row directly into the token owner's arena, and the mirrored
  backward (dO / delta pushed to head owners, dQ/dK/dV pulled back with KV-replica summation).
* ``allreduce_avg_``     – two-shot gradient all-reduce with the bf16 cast and 1/N scale fused in.

The NCCL rotators, ``all_to_all_single`` and ``all_reduce`` (``parallel.ring``, ``parallel.ulysses``,
``parallel.ddp``) remain as the measured baseline (``CP_ROTATOR=p2p|alltoall|allgather``).
"""
from __future__ import annotations

import ctypes
import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native as nv
from ..ops import attention as A
from ..ops import attention_bwd as AB
from ..ops import permute
from .symm import SymmetricHeap, tensor_from_ptr

N_COPY_CTAS = 16
FLAG_BYTES = 4096


class _Group:
    """A sub-group of the heap's ranks with its own peer table, flag row and barrier epoch."""

    def __init__(self, heap: SymmetricHeap, ranks_in_heap: List[int], my_index: int, flag_off: int, device):
        self.heap, self.size, self.rank = heap, len(ranks_in_heap), my_index
        self.peers = torch.tensor([heap.peer_bases[r] for r in ranks_in_heap], dtype=torch.int64, device=device)
        self.flag_off = flag_off
        self.epoch = 0


class FusedComm:
    def __init__(self, cfg, ctx, device: torch.device, heap_bytes: int):
        self.cfg, self.ctx, self.device = cfg, ctx, device
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self.heap = SymmetricHeap(None, heap_bytes, device)
        flags_off = self.heap.alloc("flags", 4 * FLAG_BYTES)
        all_ranks = list(range(self.world))
        self.g_world = _Group(self.heap, all_ranks, self.rank, flags_off, device)
        mesh = ctx.mesh
        self.g_ring = self.g_uly = None
        if cfg.attn_mode == "ring":
            self.g_ring = _Group(self.heap, mesh.ranks("cp"), ctx.cp_rank, flags_off + FLAG_BYTES, device)
        elif cfg.attn_mode == "ulysses":
            self.g_uly = _Group(self.heap, mesh.ranks("cp"), ctx.cp_rank, flags_off + FLAG_BYTES, device)
        elif cfg.attn_mode == "hybrid":
            self.g_ring = _Group(self.heap, mesh.ranks("ring"), ctx.ring_rank, flags_off + FLAG_BYTES, device)
            self.g_uly = _Group(self.heap, mesh.ranks("ulysses"), ctx.ulysses_rank, flags_off + 2 * FLAG_BYTES, device)
        self.timeout_s = min(cfg.watchdog_s, 20.0)
        self._ring_state: Dict[tuple, "_RingBuffers"] = {}
        self._uly_state: Dict[tuple, "_UlyssesBuffers"] = {}
        self._layer_counter = {"ring": 0, "uly": 0}      # one slot sequence per exchange (hybrid runs both in every layer)
        self._ar_stage_off: Optional[int] = None

    # ------------------------------------------------------------------ construction
    @staticmethod
    def estimate_bytes(cfg, ctx) -> int:
        B, T, D = cfg.B, cfg.T, cfg.head_dim
        L = cfg.n_layer
        Hq, Hkv = cfg.n_head, cfg.n_kv_head
        U = ctx.ulysses_size if cfg.attn_mode != "ring" else 1
        R = ctx.ring_size
        total = 64 << 20
        if R > 1:
            hq, hkv = Hq // (U if cfg.attn_mode == "hybrid" else 1), max(1, Hkv // (U if cfg.attn_mode == "hybrid" else 1))
            tl = T // R
            total += L * 2 * B * tl * hkv * D * 2            # per-layer published K/V
            total += 2 * B * T * hkv * D * 2                 # gathered K/V (shared)
            total += 2 * B * tl * hkv * D * 4                # dK/dV fp32 accumulators
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
        n_params = cfg.n_layer * (cfg.n_embd * (Hq + 2 * Hkv) * D + Hq * D * cfg.n_embd + 3 * cfg.n_embd * cfg.ffn_hidden) \
            + 2 * cfg.vocab_padded * cfg.n_embd + (1 << 22)
        total += n_params * 2 + (64 << 20)                   # bf16 gradient staging
        return int(total * 1.05)

    @staticmethod
    def create(cfg, ctx, device) -> Optional["FusedComm"]:
        if dist.get_world_size() > torch.cuda.device_count():
            return None            # more ranks than local GPUs: not a single-node job, CUDA IPC does not apply
        return FusedComm(cfg, ctx, device, FusedComm.estimate_bytes(cfg, ctx))

    def covers_world(self) -> bool:
        return True

    def supports_ring_group(self) -> bool:
        return self.g_ring is not None

    def close(self) -> None:
        self.heap.close()

    # ------------------------------------------------------------------ primitives
    def barrier(self, g: _Group) -> None:
        g.epoch += 1
        st = nv.status_for(self.device)
        nv.call("barrier", nv.ptr(g.peers), nv.l(g.flag_off), nv.i(g.size), nv.i(g.rank), nv.i(g.epoch),
                ctypes.c_double(self.timeout_s), st.ptr(), nv.stream_ptr(self.device))

    def next_layer_slot(self, n_layers: int, kind: str = "ring") -> int:
        s = self._layer_counter[kind] % n_layers
        self._layer_counter[kind] += 1
        return s

    # ------------------------------------------------------------------ gradient all-reduce
    def grad_allreduce_for(self, flat) -> "FusedComm":
        self._ar_stage_off = self.heap.alloc("grad_stage", flat.total * 2 + 64)
        self._ar_flat = flat
        return self

    def allreduce_avg_(self, buf: torch.Tensor, offset: int) -> None:
        """In-place average of a slice of the flat fp32 gradient buffer over all ranks.
        cast(grad/N)→bf16 staging | barrier | owner reduces its slice from every peer | barrier | gather."""
        g = self.g_world
        n = buf.numel()
        stage_off = self._ar_stage_off + offset * 2
        stage = self.heap.view(stage_off, (n,), torch.bfloat16)
        s = nv.stream_ptr(self.device)
        nv.call("cast_f32_bf16", nv.ptr(buf), nv.ptr(stage), nv.l(n), nv.f(1.0 / g.size), s)
        self.barrier(g)
        ctas = max(8, min(64, n // (1 << 16)))
        nv.call("allreduce_reduce", nv.ptr(g.peers), nv.l(stage_off), nv.ptr(buf), nv.l(n), nv.i(g.size), nv.i(g.rank), nv.i(ctas), s)
        self.barrier(g)
        nv.call("allreduce_gather", nv.ptr(g.peers), nv.l(stage_off), nv.ptr(buf), nv.l(n), nv.i(g.size), nv.i(g.rank), nv.i(ctas), s)

    def allreduce_finish(self) -> None:
        """Closing barrier after the last bucket of a step: no rank may overwrite its staging slices with the
        next step's gradients while a slower rank is still gathering from them."""
        self.barrier(self.g_world)

    # ------------------------------------------------------------------ ring
    def ring_attention(self, q, k, v, pos, T: int, scale: float) -> torch.Tensor:
        return _FusedRingFn.apply(q, k, v, pos, self, T, scale)

    # ------------------------------------------------------------------ ulysses
    def ulysses_attention(self, q, k, v, scale: float) -> torch.Tensor:
        return _FusedUlyssesFn.apply(q, k, v, self, scale)


# ============================================================================ ring
class _RingBuffers:
    """Symmetric buffers and tables of the fused ring for one problem shape."""

    def __init__(self, fc: FusedComm, B: int, Tl: int, Hkv: int, D: int):
        g, heap, dev = fc.g_ring, fc.heap, fc.device
        N, r = g.size, g.rank
        L = fc.cfg.n_layer
        T = Tl * N
        self.B, self.Tl, self.Hkv, self.D, self.T, self.N = B, Tl, Hkv, D, T, N
        self.cs = Tl // 2
        tag = f"ring{B}x{Tl}x{Hkv}x{D}"
        blk_bytes = 2 * B * Tl * Hkv * D * 2
        self.pub_off = heap.alloc(tag + ".kvpub", L * blk_bytes)
        self.pub_bytes = blk_bytes
        self.gathered, _ = heap.tensor(tag + ".gathered", (2, B, T, Hkv, D), torch.bfloat16)
        self.dkv_acc, self.acc_off = heap.tensor(tag + ".dkvacc", (2, B, Tl, Hkv, D), torch.float32)
        self.ready = torch.zeros(2 * N, dtype=torch.int32, device=dev)
        self.ready_bwd = torch.zeros(2 * N, dtype=torch.int32, device=dev)
        self.gather_calls = 0
        self.peer_bases = [int(x) for x in g.peers.tolist()]
        self._segs: Dict[int, torch.Tensor] = {}
        # chunk c (of 2N, cs rows each) is owned by rank c (head) or 2N-1-c (tail) at local row 0 or cs
        cs = self.cs
        rk, rv = [], []
        row_bytes = Hkv * D * 4
        for c in range(2 * N):
            owner = c if c < N else 2 * N - 1 - c
            lrow0 = 0 if c < N else cs
            base = self.peer_bases[owner] + self.acc_off
            rk.append(base + lrow0 * row_bytes)
            rv.append(base + B * Tl * row_bytes + lrow0 * row_bytes)
        self.route = (torch.tensor(rk, dtype=torch.int64, device=dev), torch.tensor(rv, dtype=torch.int64, device=dev), cs, Tl)
        # copy order: the two local chunks first, then the others in position order
        mine = [r, 2 * N - 1 - r]
        self.chunk_order = mine + [c for c in range(2 * N) if c not in mine]

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
                owner = c if c < N else 2 * N - 1 - c
                lrow0 = 0 if c < N else cs
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


class _FusedRingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, pos, fc: FusedComm, T: int, scale: float):
        rb = _ring_buffers(fc, k)
        slot = fc.next_layer_slot(fc.cfg.n_layer)
        pub = rb.pub_view(fc, slot)
        dev = q.device
        B, Tl, Hkv, D = k.shape
        # publish this rank's K/V block where the peers can read it
        permute.kv_pack(k, v, out=pub)
        fc.barrier(fc.g_ring)
        rb.gather_calls += 1
        pos32 = pos.to(torch.int32)
        segs = rb.segs(fc, slot)
        out, lse = A.flash_fwd(q, rb.gathered[0], rb.gathered[1], scale, True, pos32, 0,
                               ready=rb.ready, ready_epoch=rb.gather_calls * N_COPY_CTAS, block_rows=rb.cs,
                               segs=segs, n_segs=segs.shape[0], n_copy=N_COPY_CTAS)
        ctx.save_for_backward(q, out, lse, pos32)
        ctx.fc, ctx.rb, ctx.slot, ctx.scale = fc, rb, slot, scale
        return out

    @staticmethod
    def backward(ctx, do):
        q, out, lse, pos32 = ctx.saved_tensors
        fc, rb, slot, scale = ctx.fc, ctx.rb, ctx.slot, ctx.scale
        dev = q.device
        B, Tl, Hq, D = q.shape
        do = do.contiguous()
        rb.dkv_acc.zero_()
        fc.barrier(fc.g_ring)                  # every accumulator is zero, every published K/V is still in place
        segs = rb.segs(fc, slot)
        nv.call("ring_gather", nv.ptr(segs), nv.i(segs.shape[0]), nv.ptr(rb.ready_bwd), nv.i(4 * N_COPY_CTAS), nv.stream_ptr(dev))
        delta, lse2 = AB.flash_bwd_prep(out, do, lse)
        qpos_pad = AB.padded_q_pos(Tl, dev, pos32)
        dq = torch.zeros((B, Tl, Hq, D), dtype=torch.float32, device=dev)
        AB.flash_bwd_core(q, rb.gathered[0], rb.gathered[1], do, lse2, delta, qpos_pad, scale, True, 0, dq, None, None, True,
                          route=rb.route)
        fc.barrier(fc.g_ring)                  # every rank's contributions have landed in the owners' accumulators
        dkv = AB.cast_to_bf16(rb.dkv_acc)
        return AB.cast_to_bf16(dq), dkv[0], dkv[1], None, None, None, None


# ============================================================================ ulysses
class _UlyssesBuffers:
    def __init__(self, fc: FusedComm, B: int, Tl: int, Hq: int, Hkv: int, D: int):
        g, heap = fc.g_uly, fc.heap
        P = g.size
        L = fc.cfg.n_layer
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


class _FusedUlyssesFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, fc: FusedComm, scale: float):
        B, Tl, Hq, D = q.shape
        Hkv = k.shape[2]
        key = (B, Tl, Hq, Hkv, D)
        ub = fc._uly_state.get(key)
        if ub is None:
            ub = fc._uly_state[key] = _UlyssesBuffers(fc, B, Tl, Hq, Hkv, D)
        g = fc.g_uly
        slot = fc.next_layer_slot(fc.cfg.n_layer, "uly")
        q, k, v = _seq_layout(q, Tl, D), _seq_layout(k, Tl, D), _seq_layout(v, Tl, D)
        # sequence -> head: peer stores straight into the head owners' landing buffers
        _a2a_push(fc, g, [(q, ub.nq, 1, 0), (k, ub.kvl, ub.rep, ub.nq), (v, ub.kvl, ub.rep, ub.nq + ub.kvl)],
                  B, Tl, D, ub.hl, ub.qkv_off + slot * ub.qkv_bytes)
        fc.barrier(g)
        land = ub.qkv_view(fc, slot)
        qh, kh, vh = land[:, :, :ub.nq], land[:, :, ub.nq:ub.nq + ub.kvl], land[:, :, ub.nq + ub.kvl:]
        # local attention over the full sequence; the epilogue stores every row into its token owner's arena
        _, lse = A.flash_fwd(qh, kh, vh, scale, True,
                             o_scatter=(g.peers, ub.o_off + slot * ub.o_bytes, Tl, g.rank * ub.nq, Hq))
        fc.barrier(g)
        out = ub.o_view(fc, slot)
        ctx.save_for_backward(lse)
        ctx.fc, ctx.ub, ctx.slot, ctx.scale = fc, ub, slot, scale
        return out

    @staticmethod
    def backward(ctx, do):
        (lse,) = ctx.saved_tensors
        fc, ub, slot, scale = ctx.fc, ctx.ub, ctx.slot, ctx.scale
        g = fc.g_uly
        B, Tl, Hq, Hkv, D = ub.B, ub.Tl, ub.Hq, ub.Hkv, ub.D
        dev = fc.device
        do = do.contiguous()
        o_local = ub.o_view(fc, slot)
        delta = AB.flash_bwd_delta(o_local, do)                     # [B,Hq,Tl_pad], computed where the tokens live
        _a2a_push(fc, g, [(do, ub.nq, 1, 0)], B, Tl, D, ub.nq, ub.do_off)
        nv.call("a2a_push_rows_f32", nv.ptr(delta), nv.i(B), nv.i(Hq), nv.i(Tl), nv.i(delta.shape[-1]), nv.i(ub.nq), nv.i(g.size),
                nv.i(g.rank), nv.l(ub.delta_off), nv.i(ub.t_pad), nv.ptr(g.peers), nv.stream_ptr(dev))
        fc.barrier(g)
        lse2 = AB.flash_bwd_lse2(lse, D)
        land = ub.qkv_view(fc, slot)
        qh, kh, vh = land[:, :, :ub.nq], land[:, :, ub.nq:ub.nq + ub.kvl], land[:, :, ub.nq + ub.kvl:]
        dq32 = torch.zeros((B, ub.T, ub.nq, D), dtype=torch.float32, device=dev)
        AB.flash_bwd_core(qh, kh, vh, ub.do, lse2, ub.delta, ub.qpos_pad, scale, True, 0, dq32, ub.dk, ub.dv, False)
        nv.call("cast_f32_bf16", nv.ptr(dq32), nv.ptr(ub.dq), nv.l(dq32.numel()), nv.f(1.0), nv.stream_ptr(dev))
        fc.barrier(g)
        # head -> sequence: pull this rank's tokens of every head from the head owners, summing KV replicas
        dqkv = torch.empty((B, Tl, Hq + 2 * Hkv, D), dtype=torch.bfloat16, device=dev)
        dq, dk, dv = dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hkv], dqkv[:, :, Hq + Hkv:]
        _a2a_pull(fc, g, [(dq, Hq, ub.nq, 1, 0, ub.nq, ub.dq_off), (dk, Hkv, ub.kvl, ub.rep, 0, ub.kvl, ub.dk_off),
                          (dv, Hkv, ub.kvl, ub.rep, 0, ub.kvl, ub.dv_off)], B, Tl, D)
        return dq, dk, dv, None, None


# ============================================================================ hybrid: the Ulysses exchange on its own
class _FusedSeqToHeadFn(torch.autograd.Function):
    """``[B, Tl, H, D]`` (this rank's tokens, all heads) -> ``[B, Tl*P, H/P, D]`` (the whole ring block, this rank's
    heads) for q, k and v at once, by peer stores into the head owners' per-layer landing buffers; the adjoint pulls
    the gradients back (the exchange that ``hybrid_attention`` wraps around ring attention,
    context_parallel/ContextParallel.h:1359-1396)."""

    @staticmethod
    def forward(ctx, q, k, v, fc: FusedComm):
        B, Tl, Hq, D = q.shape
        Hkv = k.shape[2]
        key = (B, Tl, Hq, Hkv, D)
        ub = fc._uly_state.get(key)
        if ub is None:
            ub = fc._uly_state[key] = _UlyssesBuffers(fc, B, Tl, Hq, Hkv, D)
        g = fc.g_uly
        slot = fc.next_layer_slot(fc.cfg.n_layer, "uly")
        q, k, v = _seq_layout(q, Tl, D), _seq_layout(k, Tl, D), _seq_layout(v, Tl, D)
        _a2a_push(fc, g, [(q, ub.nq, 1, 0), (k, ub.kvl, ub.rep, ub.nq), (v, ub.kvl, ub.rep, ub.nq + ub.kvl)],
                  B, Tl, D, ub.hl, ub.qkv_off + slot * ub.qkv_bytes)
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
        g = fc.g_uly
        B, Tl, Hq, Hkv, D = ub.B, ub.Tl, ub.Hq, ub.Hkv, ub.D
        ub.dq.copy_(dqh)
        ub.dk.copy_(dkh)
        ub.dv.copy_(dvh)
        fc.barrier(g)
        dqkv = torch.empty((B, Tl, Hq + 2 * Hkv, D), dtype=torch.bfloat16, device=fc.device)
        dq, dk, dv = dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hkv], dqkv[:, :, Hq + Hkv:]
        _a2a_pull(fc, g, [(dq, Hq, ub.nq, 1, 0, ub.nq, ub.dq_off), (dk, Hkv, ub.kvl, ub.rep, 0, ub.kvl, ub.dk_off),
                          (dv, Hkv, ub.kvl, ub.rep, 0, ub.kvl, ub.dv_off)], B, Tl, D)
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

