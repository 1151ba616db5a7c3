"""Runtime bisect tools for overlap races and cross-rank parity, all off by default and switched on by the
reference's environment names (parsed once into ``config.DebugConfig``).

The reference grew these while chasing real races in its overlapped ring (context_parallel/ContextParallel.h:
805-820 ``CP_DRAIN_AT``, :888-968 ``CP_SELFCHECK``, :1052-1095 ``CP_DUMP_KV_CHUNKS``; ``DUMP_CP_OUT`` /
``DUMP_CP_STEPS`` / ``DUMP_CP_MERGE`` parity dumps).  The protocol hazards here are of the same kind (flag epochs,
per-layer publish slots, copy CTAs racing compute CTAs, a side-stream gradient reduction), so the same tools exist:

* ``CP_SELFCHECK=1``     – after a fused attention forward, drain everything, recompute the same attention from the
  now complete K/V with the same tile order and diff bit-for-bit; a non-zero difference means a compute CTA consumed a
  block before it had landed.  First hit per rank is written to ``<log_dir>/cp_selfcheck_rank<r>.log``.
* ``CP_DUMP_KV_CHUNKS=1`` (+ ``CP_DUMP_KV_CALL=n``) – checksum of every K/V chunk as published by its owner versus
  as gathered by this rank.
* ``CP_DRAIN_AT=1|2|3``  – device-wide synchronisation before the attention op, after its forward, after its backward.
* ``CP_SYNC_RING=1``     – synchronise the device around every cross-rank barrier (serialises all overlap).
* ``CP_NO_OVERLAP[_FWD|_BWD]=1`` – K/V gather as a stand-alone launch before the attention kernel; gradient reduction
  on the compute stream.
* ``CP_FWD_SYNC_RECV`` / ``CP_FWD_SYNC_RETURN`` – synchronise after the K/V arrived / before the forward returns.
* ``DUMP_CP_OUT`` / ``DUMP_CP_STEPS`` / ``DUMP_CP_MERGE`` / ``DUMP_FWD`` / ``CP_DEBUG_SHAPES`` – tensor dumps
  (``<log_dir>/dump_<name>_rank<r>_call<n>.pt``) and shape prints.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch
import torch.distributed as dist


class DebugTools:
    def __init__(self, cfg, rank: int = 0):
        self.d = cfg.debug
        self.log_dir = cfg.log_dir
        self.rank = rank
        self.calls: Dict[str, int] = {}
        self.selfcheck_hits = 0
        self.kv_mismatches = 0
        self._kv_dumped = False
        self.kv_call = int(os.environ.get("CP_DUMP_KV_CALL", "0") or 0)
        self.active = any((self.d.selfcheck, self.d.drain_at, self.d.sync_ring, self.d.fwd_sync_recv, self.d.fwd_sync_return,
                           self.d.dump_cp_out, self.d.dump_cp_steps, self.d.dump_cp_merge, self.d.dump_kv_chunks,
                           self.d.debug_shapes, self.d.dump_fwd))

    # ------------------------------------------------------------------ synchronisation points
    def drain(self, point: int) -> None:
        if self.d.drain_at == point and torch.cuda.is_available():
            torch.cuda.synchronize()

    def sync_if(self, flag: bool) -> None:
        if flag and torch.cuda.is_available():
            torch.cuda.synchronize()

    # ------------------------------------------------------------------ dumps
    def next_call(self, kind: str) -> int:
        n = self.calls.get(kind, 0)
        self.calls[kind] = n + 1
        return n

    def dump(self, enabled: bool, name: str, call: int, **tensors) -> Optional[str]:
        if not enabled:
            return None
        os.makedirs(self.log_dir or ".", exist_ok=True)
        path = os.path.join(self.log_dir or ".", f"dump_{name}_rank{self.rank}_call{call}.pt")
        torch.save({k: v.detach().float().cpu() for k, v in tensors.items()}, path)
        return path

    def shapes(self, what: str, **tensors) -> None:
        if self.d.debug_shapes:
            desc = ", ".join(f"{k}={tuple(v.shape)}:{str(v.dtype).replace('torch.', '')}" for k, v in tensors.items())
            print(f"[CP_DEBUG_SHAPES] rank {self.rank} {what}: {desc}", flush=True)

    # ------------------------------------------------------------------ recompute-and-diff
    def selfcheck(self, what: str, call: int, got: Dict[str, torch.Tensor], recompute) -> float:
        """``got``: tensors produced under overlap; ``recompute()``: the same computation on settled inputs, returning
        tensors under the same keys.  The outputs are snapshotted to the host BEFORE the recompute so that its own
        allocations cannot alias what is being compared.  Returns the largest absolute difference."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        snap = {k: v.detach().float().cpu() for k, v in got.items()}
        if dist.is_initialized():
            dist.barrier()
        ref = recompute()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        worst = 0.0
        for k, h in snap.items():
            r = ref[k].detach().float().cpu()
            fin = torch.isfinite(h) & torch.isfinite(r)
            d = float((h[fin] - r[fin]).abs().max()) if bool(fin.any()) else 0.0
            if not torch.equal(torch.isfinite(h), torch.isfinite(r)):
                d = float("inf")
            worst = max(worst, d)
        if worst > 0.0:
            self.selfcheck_hits += 1
            refmax = max(float(v.detach().float().abs().max()) for v in ref.values())
            msg = f"[CP_SELFCHECK] RACE {what} call={call} rank={self.rank} maxabs_diff={worst:.3e} ref_maxabs={refmax:.3e}"
            print(msg, flush=True)
            if self.selfcheck_hits == 1:
                os.makedirs(self.log_dir or ".", exist_ok=True)
                with open(os.path.join(self.log_dir or ".", f"cp_selfcheck_rank{self.rank}.log"), "w") as f:
                    f.write("FIRST RACE HIT\n" + msg + "\n")
        return worst

    # ------------------------------------------------------------------ sent-versus-received K/V
    def want_kv_check(self, call: int) -> bool:
        if not self.d.dump_kv_chunks or self._kv_dumped or call < self.kv_call:
            return False
        self._kv_dumped = True
        return True

    @staticmethod
    def checksum(t: torch.Tensor) -> torch.Tensor:
        """Order-independent exact checksum of a bf16/fp32 tensor's bytes: sum of its 16-bit words as int64, and the
        sum of their squares (two numbers make an accidental match of different contents unlikely)."""
        w = t.contiguous().view(torch.int16).to(torch.int64)
        return torch.stack([w.sum(), (w * w).sum()])

    def compare_kv(self, call: int, sent: torch.Tensor, received: torch.Tensor, owners, group) -> int:
        """``sent``: ``[n_mine, 2]`` checksums of the chunks this rank published (in ``owners``' order of its own
        chunks); ``received``: ``[n_chunks, 2]`` checksums of every chunk as gathered here; ``owners[c] = (rank, idx)``
        names the publisher of chunk c and the index among its chunks.  Returns the number of mismatching chunks."""
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        if world > 1:
            allsent = [torch.empty_like(sent) for _ in range(world)]
            dist.all_gather(allsent, sent, group=group)
        else:
            allsent = [sent]
        bad = 0
        for c, (owner, idx) in enumerate(owners):
            if not torch.equal(allsent[owner][idx].cpu(), received[c].cpu()):
                bad += 1
                print(f"[CP_DUMP_KV_CHUNKS] MISMATCH call={call} rank={self.rank} chunk={c} owner={owner}: "
                      f"sent {allsent[owner][idx].tolist()} received {received[c].tolist()}", flush=True)
        if bad == 0:
            print(f"[CP_DUMP_KV_CHUNKS] call={call} rank={self.rank}: all {len(owners)} chunks match their owners' copies", flush=True)
        self.kv_mismatches += bad
        return bad
