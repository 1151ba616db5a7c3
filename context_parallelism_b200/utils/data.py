"""Batch sources: the native mmap token-shard loader (``csrc/runtime/dataloader.cpp``) and synthetic
uniform-random tokens.  Both hand out FULL sequences ``(x, y)`` of shape ``[B, T]`` in pinned host memory;
all ranks of a context-parallel group read the same batch and only the data-parallel coordinate selects the
stream (Scripts/Blutrain/bluscriptCP.cpp:1022-1025; gpt2_cp_test.cpp:957-960)."""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from .. import _native as nv


def _pinned(shape):
    t = torch.empty(shape, dtype=torch.int64)
    if torch.cuda.is_available():
        try:
            t = t.pin_memory()
        except RuntimeError:
            pass
    return t


class ShardLoader:
    """uint16 ``*.bin`` shards under ``root`` whose names contain ``split``."""

    def __init__(self, root: str, split: str, B: int, T: int, rank: int = 0, world: int = 1):
        self.B, self.T = B, T
        self._h = ctypes.c_void_p()
        nv.check(nv.lib().cpb_dl_open(root.encode(), split.encode(), B, T, rank, world, ctypes.byref(self._h)), "dl_open")
        self._x = [_pinned((B, T)) for _ in range(2)]
        self._y = [_pinned((B, T)) for _ in range(2)]
        self._i = 0

    def next_batch(self) -> Tuple[torch.Tensor, torch.Tensor]:
        x, y = self._x[self._i], self._y[self._i]
        self._i ^= 1
        nv.check(nv.lib().cpb_dl_next(self._h, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr())), "dl_next")
        return x, y

    def skip_batches(self, n: int) -> None:
        nv.check(nv.lib().cpb_dl_skip(self._h, ctypes.c_long(n)), "dl_skip")

    def reset(self) -> None:
        nv.check(nv.lib().cpb_dl_reset(self._h), "dl_reset")

    @property
    def num_shards(self) -> int:
        return nv.lib().cpb_dl_num_shards(self._h)

    @property
    def position(self) -> int:
        nv.lib().cpb_dl_position.restype = ctypes.c_long
        return nv.lib().cpb_dl_position(self._h)

    def close(self) -> None:
        if self._h:
            nv.lib().cpb_dl_close.restype = None
            nv.lib().cpb_dl_close(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class SyntheticLoader:
    """Uniform random tokens in ``[0, vocab)`` from a seeded generator; the stream depends on ``(seed, rank)`` only,
    so a resumed run can fast-forward with ``skip_batches``."""

    def __init__(self, vocab: int, B: int, T: int, rank: int = 0, world: int = 1, seed: int = 0):
        self.vocab, self.B, self.T = vocab, B, T
        self.gen = torch.Generator().manual_seed(seed * 1000003 + rank)
        self._buf = [_pinned((B, T + 1)) for _ in range(2)]
        self._i = 0

    def next_batch(self) -> Tuple[torch.Tensor, torch.Tensor]:
        b = self._buf[self._i]
        self._i ^= 1
        b.copy_(torch.randint(0, self.vocab, (self.B, self.T + 1), generator=self.gen))
        return b[:, :-1], b[:, 1:]

    def skip_batches(self, n: int) -> None:
        for _ in range(n):
            torch.randint(0, self.vocab, (self.B, self.T + 1), generator=self.gen)

    def reset(self) -> None:
        pass

    def close(self) -> None:
        pass


def make_loader(cfg, split: str, dp_rank: int, dp_size: int):
    if cfg.synthetic or not cfg.data_root:
        return SyntheticLoader(cfg.vocab_size, cfg.B, cfg.T, dp_rank, dp_size, 0 if split == "train" else 7919)   # data seed 0, independent of the weight-init seed
    return ShardLoader(cfg.data_root, split, cfg.B, cfg.T, dp_rank, dp_size)
