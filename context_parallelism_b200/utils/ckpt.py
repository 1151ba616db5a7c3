"""Named-record weight files and run-numbered checkpoints with auto-resume.

Record format (byte-compatible with the reference's named-init files,
Scripts/Pytorch/gpt2_cp_attnstyle_fp32.py:752-767, reader Scripts/Blutrain/gpt2_cp_test.cpp:851-933):
repeated ``int32 name_len | name bytes | int32 ndim | int64 dims[ndim] | float32 data`` in PyTorch layout
(Linear weights ``[out, in]``), little endian, no header.

Checkpoints reuse the same record stream: the model tensors under their reference names, then
``opt.m.<name>`` / ``opt.v.<name>`` Adam moments, then a ``__meta__`` record ``[step, loss, run]``.  Files are
``<dir>/<prefix>_run<N>_step_<S>.ckpt`` directly inside the checkpoint directory; rank 0 saves, every rank
loads, the newest ``keep`` files of a run are kept, and the run to resume is chosen like the reference does
(Scripts/Blutrain/bluscriptCP.cpp:1049-1088): ``CP_CKPT_RESUME=<N>`` forces a run (a new one if it has no
file), ``CP_CKPT_NEW_RUN=1`` forces a fresh one, otherwise ONLY the highest run number is looked at: it is
resumed when its last step is below ``max_steps``, and a new run starts when it is complete (older
incomplete runs are never picked up).  Checkpoints do not depend on sequence length or world size.
"""
from __future__ import annotations

import os
import re
import struct
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch


def write_named(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> int:
    n = 0
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        for name, t in tensors:
            arr = t.detach().to(torch.float32).cpu().contiguous().numpy()
            nm = name.encode()
            f.write(struct.pack("<i", len(nm)))
            f.write(nm)
            f.write(struct.pack("<i", arr.ndim))
            for d in arr.shape:
                f.write(struct.pack("<q", int(d)))
            f.write(arr.tobytes())
            n += 1
    os.replace(tmp, path)
    return n


def read_named(path: str) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        data = f.read()
    off, size = 0, len(data)
    while off < size:
        (nl,) = struct.unpack_from("<i", data, off); off += 4
        if nl <= 0 or nl > 4096:
            raise ValueError(f"{path}: corrupt record at byte {off - 4}")
        name = data[off:off + nl].decode(); off += nl
        (nd,) = struct.unpack_from("<i", data, off); off += 4
        dims = struct.unpack_from(f"<{nd}q", data, off); off += 8 * nd
        cnt = int(np.prod(dims)) if nd else 1
        arr = np.frombuffer(data, dtype="<f4", count=cnt, offset=off).reshape(dims)
        off += 4 * cnt
        out[name] = torch.from_numpy(arr.copy())
    return out


def _split_fused(model, flat) -> List[Tuple[str, torch.Tensor]]:
    """Model tensors under reference names, taken from the fp32 masters."""
    masters = flat.named_master()
    by_param = {id(p): masters[name] for name, p, _, _ in flat.entries}
    out = []
    for name, view in model.named_tensors().items():
        base = view._base if view._base is not None else view
        m = by_param.get(id(base))
        if m is None:      # e.g. tied lm_head alias
            continue
        if view._base is not None:
            off = view.storage_offset() - base.storage_offset()
            rows = off // base.shape[1]
            m = m[rows:rows + view.shape[0]]
        out.append((name, m))
    return out


def save_named_init(path: str, model, flat, rank: int = 0) -> int:
    """Every rank calls this (collective when the optimiser state is sharded); rank 0 writes."""
    recs = _split_fused(model, flat)
    return write_named(path, recs) if rank == 0 else len(recs)


def load_named_into(model, flat, tensors: Dict[str, torch.Tensor], strict: bool = True) -> int:
    """Copy records into the fp32 masters (and refresh the bf16 compute copies).  Vocabulary rows beyond the
    file's row count stay zero (padding).  ``strict``: every model tensor must be in the file.  Either way a file
    record that matches no model tensor is an error (optimiser ``opt.*`` and ``__meta__`` records excepted, and
    ``lm_head.weight`` of an untied file loaded into a tied model): a silently skipped record leaves a parameter at
    its initial value, which a name mismatch between writer and reader would otherwise hide."""
    known = set(model.named_tensors())
    stray = [k for k in tensors if k not in known and not k.startswith("opt.") and k != "__meta__"
             and k not in ("lm_head.weight", "lm_head")]
    if stray:
        raise KeyError(f"weight file has records that match no model tensor: {stray[:6]}{' ...' if len(stray) > 6 else ''}")
    by_param = {id(p): (name, p) for name, p, _, _ in flat.entries}
    n = 0
    for name, view in model.named_tensors().items():
        if name not in tensors:
            if strict:
                raise KeyError(f"missing tensor {name!r} in weight file")
            continue
        src = tensors[name]
        base = view._base if view._base is not None else view
        ent = by_param.get(id(base))
        if ent is None:
            continue
        row0 = 0
        if view._base is not None:
            off = view.storage_offset() - base.storage_offset()
            row0 = off // base.shape[1]
        want = tuple(view.shape)
        if src.dim() == 2 and len(want) == 2 and src.shape[0] < want[0] and src.shape[1] == want[1]:
            pass                                   # fewer vocabulary rows than the padded table: the rest stays zero
        elif tuple(src.shape) != want:
            raise ValueError(f"{name}: file shape {tuple(src.shape)} != model shape {want}")
        flat.load_master_rows(ent[0], row0, src)
        n += 1
    flat.sync_compute_copy()
    return n


# ------------------------------------------------------------------ run-numbered checkpoints


class CheckpointManager:
    def __init__(self, root: str, prefix: str, keep: int = 6, rank: int = 0):
        self.root, self.prefix, self.keep, self.rank = root, prefix, keep, rank
        self.run: Optional[int] = None
        self._file_re = re.compile(re.escape(prefix) + r"_run(\d+)_step_(\d+)\.ckpt$")

    def list_runs(self) -> Dict[int, List[int]]:
        """``{run: sorted steps}`` from the flat ``<prefix>_run<K>_step_<S>.ckpt`` files of the directory."""
        runs: Dict[int, List[int]] = {}
        if not os.path.isdir(self.root):
            return runs
        for f in os.listdir(self.root):
            m = self._file_re.match(f)
            if m and os.path.isfile(os.path.join(self.root, f)):
                runs.setdefault(int(m.group(1)), []).append(int(m.group(2)))
        return {r: sorted(s) for r, s in runs.items()}

    def resolve_run(self, max_steps: int, new_run: bool = False, resume: int = -1) -> Tuple[int, bool]:
        """Returns ``(run_number, resuming)``.  Call on rank 0 and broadcast the result."""
        runs = self.list_runs()
        fresh = max(runs) + 1 if runs else 0
        if new_run:
            return fresh, False
        if resume >= 0:
            return (resume, True) if runs.get(resume) else (fresh, False)
        if runs:
            last = max(runs)
            if runs[last][-1] < max_steps:
                return last, True
        return fresh, False

    def path(self, run: int, step: int) -> str:
        return os.path.join(self.root, f"{self.prefix}_run{run}_step_{step}.ckpt")

    def save(self, run: int, step: int, model, flat, opt, loss: float) -> Optional[str]:
        """Every rank calls this (assembling the masters and moments of a sharded optimiser is a collective); rank 0
        writes."""
        recs = _split_fused(model, flat)
        state = opt.state_dict()
        if self.rank != 0:
            return None
        os.makedirs(self.root, exist_ok=True)
        for name, t in state.items():
            recs.append(("opt." + name, t))
        recs.append(("__meta__", torch.tensor([float(step), float(loss), float(run)])))
        p = self.path(run, step)
        write_named(p, recs)
        steps = self.list_runs().get(run, [])
        for s in steps[:-self.keep] if self.keep > 0 else []:
            try:
                os.remove(self.path(run, s))
            except OSError:
                pass
        return p

    def seed_run_from(self, src_run: int, dst_run: int) -> int:
        """Start ``dst_run`` from the newest checkpoint of ``src_run``: the file is copied under the new run's name
        (same step), so that resuming ``dst_run`` continues training from those weights and optimiser moments.  Does
        nothing if ``dst_run`` already has a checkpoint.  Returns the step of ``dst_run``'s newest checkpoint."""
        import shutil
        runs = self.list_runs()
        if runs.get(dst_run):
            return runs[dst_run][-1]
        if not runs.get(src_run):
            raise FileNotFoundError(f"run {src_run} has no checkpoint under {self.root}")
        step = runs[src_run][-1]
        tmp = self.path(dst_run, step) + ".tmp"
        shutil.copyfile(self.path(src_run, step), tmp)
        os.replace(tmp, self.path(dst_run, step))
        return step

    def load_latest(self, run: int, model, flat, opt) -> Tuple[int, float]:
        """Load the newest checkpoint of ``run`` on every rank; returns ``(step, loss)`` or ``(0, nan)``."""
        steps = self.list_runs().get(run, [])
        if not steps:
            return 0, float("nan")
        recs = read_named(self.path(run, steps[-1]))
        load_named_into(model, flat, recs, strict=True)
        opt.load_state_dict({k[4:]: v for k, v in recs.items() if k.startswith("opt.")})
        meta = recs.get("__meta__")
        return (int(meta[0]), float(meta[1])) if meta is not None else (steps[-1], float("nan"))
