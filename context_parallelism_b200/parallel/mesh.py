"""Device mesh: N-D row-major arrangement of ranks with one process group per axis.

Same coordinate semantics and mesh shapes as the reference ``DeviceMesh``
(process_group/device_mesh.h:15-75, device_mesh.cpp:64-177): ``{ws}``, ``{dp,cp}``,
``{dp,ring,ulysses}`` or ``{ring,dp,ulysses}`` when ``CP_RING_OUTER`` is set
(Scripts/Blutrain/bluscriptCP.cpp:904-942).  The coordinate math is the native
``csrc/runtime/mesh.cpp``; communicators are ``torch.distributed`` groups (NCCL on GPUs, gloo on CPU),
created for every slice on every rank, as ``new_group`` requires.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import _native as nv


def _carr(vals: Sequence[int]):
    return (ctypes.c_int * len(vals))(*vals)


def mesh_coords(shape: Sequence[int], rank: int) -> List[int]:
    out = (ctypes.c_int * len(shape))()
    nv.check(nv.lib().cpb_mesh_coords(_carr(shape), len(shape), rank, out), "mesh_coords")
    return list(out)


def mesh_rank(shape: Sequence[int], coords: Sequence[int]) -> int:
    return nv.lib().cpb_mesh_rank(_carr(shape), len(shape), _carr(coords))


def mesh_group_ranks(shape: Sequence[int], rank: int, axis: int) -> List[int]:
    out = (ctypes.c_int * shape[axis])()
    nv.check(nv.lib().cpb_mesh_group_ranks(_carr(shape), len(shape), rank, axis, out), "mesh_group_ranks")
    return list(out)


class DeviceMesh:
    """``DeviceMesh((dp, cp), ("dp", "cp"))`` → ``mesh.group("cp")``, ``mesh.coord("cp")``, ``mesh.ranks("cp")``."""

    def __init__(self, shape: Sequence[int], names: Sequence[str], rank: Optional[int] = None,
                 world_size: Optional[int] = None, create_groups: bool = True):
        self.shape = tuple(int(s) for s in shape)
        self.names = tuple(names)
        assert len(self.shape) == len(self.names)
        self.world_size = world_size if world_size is not None else (dist.get_world_size() if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0)
        total = 1
        for s in self.shape:
            total *= s
        if total != self.world_size:
            raise ValueError(f"mesh {self.shape} does not cover world size {self.world_size}")
        self.coords = mesh_coords(self.shape, self.rank)
        self._groups: Dict[str, Optional[dist.ProcessGroup]] = {}
        self._ranks: Dict[str, List[int]] = {}
        for ax, name in enumerate(self.names):
            self._ranks[name] = mesh_group_ranks(self.shape, self.rank, ax)
        if create_groups and dist.is_initialized() and self.world_size > 1:
            for ax, name in enumerate(self.names):
                mine = None
                seen = set()
                for r in range(self.world_size):
                    members = tuple(mesh_group_ranks(self.shape, r, ax))
                    if members in seen:
                        continue
                    seen.add(members)
                    g = dist.new_group(list(members)) if len(members) > 1 else None
                    if self.rank in members:
                        mine = g
                self._groups[name] = mine
        else:
            for name in self.names:
                self._groups[name] = None

    def size(self, name: str) -> int:
        return self.shape[self.names.index(name)]

    def coord(self, name: str) -> int:
        return self.coords[self.names.index(name)]

    def ranks(self, name: str) -> List[int]:
        return self._ranks[name]

    def group(self, name: str):
        return self._groups[name]

    def has(self, name: str) -> bool:
        return name in self.names

    @staticmethod
    def for_config(cfg, rank: Optional[int] = None, world_size: Optional[int] = None, create_groups: bool = True) -> "DeviceMesh":
        dp = cfg.world_size // cfg.cp_size
        if cfg.attn_mode == "hybrid":
            r, u = cfg.cp_size // cfg.ulysses_size, cfg.ulysses_size
            if cfg.ring_outer:
                return DeviceMesh((r, dp, u), ("ring", "dp", "ulysses"), rank, world_size, create_groups)
            return DeviceMesh((dp, r, u), ("dp", "ring", "ulysses"), rank, world_size, create_groups)
        return DeviceMesh((dp, cfg.cp_size), ("dp", "cp"), rank, world_size, create_groups)


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> tuple:
    """Initialise ``torch.distributed`` from the ``torchrun`` environment; returns ``(rank, world, local_rank)``."""
    import datetime
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # without a launcher-provided LOCAL_RANK the device is rank % NO_GPUS_PER_NODE, as in the reference
    # (process_group/device_mesh.cpp:126-133)
    gpn = int(os.environ.get("NO_GPUS_PER_NODE", "0") or 0) or (torch.cuda.device_count() if torch.cuda.is_available() else 1) or 1
    local = int(os.environ["LOCAL_RANK"]) if "LOCAL_RANK" in os.environ else rank % gpn
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    elif torch.cuda.is_available():
        torch.cuda.set_device(local)
    return rank, world, local
