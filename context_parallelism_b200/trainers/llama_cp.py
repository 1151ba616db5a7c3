"""Llama-style Ring / Ulysses / Hybrid context-parallel trainer — the counterpart of ``bluscriptCP``
(Scripts/Blutrain/bluscriptCP.cpp:579-1902), configured by the same ``CP_*`` / ``YARN_*`` environment variables.

    torchrun --nproc-per-node 8 -m context_parallelism_b200.trainers.llama_cp          # CP_SIZE defaults to world

Modes (first match wins, as in the reference, bluscriptCP.cpp:1252-1649):
  ``CP_DUMP_ROPE=<file>``        write the active cos/sin cache (``CP_DUMP_ROPE_SEQLEN`` rows) as a named record
  ``CP_DUMP_NAMED=<file>``       write the weights under the reference names and exit
  ``CP_DUMP_ACTS=<file>``        forward one batch and write the final hidden states of the first ``CP_DUMP_ACTS_T`` tokens
  ``CP_LONGROPE_SEARCH=1``       resident evaluator: reads factor-file paths on stdin, prints ``PPL <value>`` per line
  ``CP_EVAL_PPL=1``              teacher-forced per-position NLL over ``CP_EVAL_WINDOWS`` windows → ``CP_EVAL_OUT`` CSV
  otherwise                      training (with ``CP_MEM_PROBE=1``: a short run that ends with a memory snapshot)

Context extension: YaRN through ``YARN_*``; LongRoPE through ``CP_LONGROPE_FACTORS`` (+ ``CP_LONGROPE_MSCALE``);
CREAM / PoSE / RandPos position relabelling per step through ``CP_CREAM_MODE`` (single context-parallel rank only,
bluscriptCP.cpp:717-719), optionally on top of a LongRoPE cache of length ``factor·T``.
"""
from __future__ import annotations

import math
import os
import sys
from typing import List, Optional

import torch
import torch.distributed as dist

from ..config import Config
from ..engine import TrainEngine
from ..ops import rope as R
from ..parallel.mesh import init_distributed
from ..utils import ckpt as ckpt_mod
from ..utils import cream
from ..utils import data as data_mod
from ..utils import metrics as M
from . import common


def install_context_extension(cfg: Config, eng: TrainEngine):
    """Build the RoPE cache the configuration asks for; returns the CREAM gather source (or None)."""
    dev, model = eng.device, eng.model
    factor = int(round(cfg.yarn.scale))
    source = None
    if cfg.longrope_factors:
        lam, n_hat, s, slen = R.parse_longrope_factors(cfg.longrope_factors, cfg.head_dim // 2)
        mscale = cfg.longrope_mscale
        if cfg.cream_mode != "off":
            if slen and slen != factor * cfg.T:
                raise ValueError(f"LongRoPE search length {slen} != factor*T = {factor * cfg.T} (composition with CREAM)")
            source = R.build_rope_cache_longrope(factor * cfg.T, cfg.head_dim, cfg.rope_theta, lam, n_hat, dev, mscale)
        else:
            model.set_rope_cache(R.build_rope_cache_longrope(cfg.T, cfg.head_dim, cfg.rope_theta, lam, n_hat, dev, mscale))
        M.log(f"[LongRoPE] {len(lam)} factors, n_hat={n_hat}, s={s}, mscale={mscale}")
    elif cfg.cream_mode != "off":
        source = R.build_rope_cache(factor * cfg.T, cfg.head_dim, cfg.rope_theta, dev, cfg.yarn)
    return source


def cream_relabel(cfg: Config, eng: TrainEngine, source: torch.Tensor, step: int) -> None:
    """Install this step's relabelled cache: row j of the model's cache = source[label[j]]
    (bluscriptCP.cpp:467-494,1687-1694)."""
    factor = int(round(cfg.yarn.scale))
    seed = cfg.cream_seed if cfg.cream_seed else 1000003 * (step + 1)
    labels = cream.generate_positions(cfg.cream_mode, cfg.T, factor, cfg.cream_sigma, seed)
    eng.model.set_rope_cache(R.gather_cache_rows(source, torch.tensor(labels, dtype=torch.int64)))
    if cfg.cream_log:
        M.log(f"[CREAM] step {step} mode={cfg.cream_mode} first={labels[0]} mid={labels[len(labels) // 2]} last={labels[-1]}")


def eval_windows(cfg: Config, eng: TrainEngine) -> List:
    """Evaluation windows ``(x, y)`` of length T: from ``CP_EVAL_TOKENS_BIN`` (raw uint16) or the val split."""
    n, skip = cfg.eval_windows, cfg.eval_skip_windows
    out = []
    if cfg.eval_tokens_bin:
        import numpy as np
        tok = np.fromfile(cfg.eval_tokens_bin, dtype=np.uint16).astype(np.int64)
        for w in range(skip, skip + n):
            lo = w * cfg.T
            if lo + cfg.T + 1 > tok.size:
                break
            t = torch.from_numpy(tok[lo:lo + cfg.T + 1])[None]
            out.append((t[:, :-1], t[:, 1:]))
        return out
    ld = data_mod.make_loader(cfg.replace(B=1), "val", 0, 1)
    ld.skip_batches(skip)
    for _ in range(n):
        x, y = ld.next_batch()
        out.append((x.clone(), y.clone()))
    ld.close()
    return out


@torch.no_grad()
def per_position_nll(cfg: Config, eng: TrainEngine, windows) -> torch.Tensor:
    """Mean NLL per global position ``[T]`` over the windows; identical for every CP degree and mode
    (the CP-invariance check of Tests/bluscriptcp/cp_parity.sh:46-55)."""
    T = cfg.T
    tot = torch.zeros(T, dtype=torch.float64, device=eng.device)
    for x, y in windows:
        idx, tgt, pos = eng.shard_batch(x, y)
        nll = eng.model.per_token_nll(idx, tgt, pos).double().sum(0)         # [T_local]
        tot.index_add_(0, pos, nll / x.shape[0])
    if eng.cp.cp_size > 1:
        dist.all_reduce(tot)
        tot /= eng.cp.dp_size            # every data-parallel replica evaluated the same windows
    return tot / max(1, len(windows))


def write_ppl_csv(path: str, nll: torch.Tensor, count: int) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write("pos,count,mean_nll,ppl\n")
        for p, v in enumerate(nll.tolist()):
            f.write(f"{p},{count},{v:.6f},{math.exp(min(v, 50.0)):.6f}\n")


def longrope_search_loop(cfg: Config, eng: TrainEngine) -> None:
    """Resident evaluator (bluscriptCP.cpp:1376-1460): rank 0 reads one factor-file path per line from stdin; the
    parse result is broadcast BEFORE anything else happens so that a bad candidate makes every rank skip together
    and no rank is ever left alone inside a collective."""
    windows = eval_windows(cfg, eng)
    half = cfg.head_dim // 2
    dev = eng.device
    bdev = dev if (dist.is_initialized() and dist.get_backend() == "nccl") else torch.device("cpu")
    M.log(f"[search] ready: {len(windows)} windows of T={cfg.T}")
    while True:
        msg = torch.zeros(half + 3, dtype=torch.float64)
        if eng.rank == 0:
            line = sys.stdin.readline()
            if not line or line.strip() in ("quit", "exit"):
                msg[0] = -1
            else:
                try:
                    lam, n_hat, s, _ = R.parse_longrope_factors(line.strip(), cfg.head_dim // 2)
                    from ..ops.reference import validate_longrope
                    validate_longrope(lam, cfg.head_dim, n_hat)
                    msg[0], msg[1], msg[2] = 1, n_hat, s
                    msg[3:] = torch.tensor(lam, dtype=torch.float64)
                except Exception as e:          # parse / validation error: status 0 is broadcast, all ranks continue
                    print(f"ERR {e}", flush=True)
        if dist.is_initialized() and eng.world > 1:
            t = msg.to(bdev)
            dist.broadcast(t, 0)
            msg = t.cpu()
        if msg[0] < 0:
            break
        if msg[0] == 0:
            continue
        lam, n_hat = msg[3:].tolist(), int(msg[1])
        eng.model.set_rope_cache(R.build_rope_cache_longrope(cfg.T, cfg.head_dim, cfg.rope_theta, lam, n_hat, dev, cfg.longrope_mscale))
        nll = per_position_nll(cfg, eng, windows)
        ppl = math.exp(min(float(nll.mean()), 50.0))
        if eng.rank == 0:
            print(f"PPL {ppl:.6f}", flush=True)


def main() -> None:
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    cfg = Config.from_env("llama", world)
    if dev.type == "cpu" and cfg.dtype == "bf16":
        cfg = cfg.replace(dtype="fp32")
    quiet_stdout = rank != 0
    real_stdout = sys.stdout
    if quiet_stdout:
        sys.stdout = open(os.devnull, "w")
    M.log("Llama CP trainer\n" + cfg.describe())
    eng = TrainEngine(cfg, dev)
    if cfg.load_init_named:
        ckpt_mod.load_named_into(eng.model, eng.flat, ckpt_mod.read_named(cfg.load_init_named), strict=False)
    source = install_context_extension(cfg, eng)

    def resume_weights() -> None:
        mgr = ckpt_mod.CheckpointManager(cfg.ckpt_dir, cfg.ckpt_prefix, cfg.ckpt_keep, rank)
        run = cfg.ckpt_resume if cfg.ckpt_resume >= 0 else common.broadcast_ints([mgr.resolve_run(10 ** 9)[0] if rank == 0 else 0])[0]
        step, loss = mgr.load_latest(run, eng.model, eng.flat, eng.opt)
        M.log(f"[eval] weights of run {run} step {step} (loss {loss:.4f})")

    if cfg.dump_rope:
        n = cfg.dump_rope_seqlen or cfg.T
        if rank == 0:
            ckpt_mod.write_named(cfg.dump_rope, [("rope_cache", eng.model.rope_cache[:n])])
        M.log(f"[dump] rope cache rows={n} -> {cfg.dump_rope}")
    elif cfg.dump_named:
        n = ckpt_mod.save_named_init(cfg.dump_named, eng.model, eng.flat, rank)
        M.log(f"[dump] {n} named tensors -> {cfg.dump_named}")
    elif cfg.dump_acts:
        ld = data_mod.make_loader(cfg, "val", eng.cp.dp_rank, eng.cp.dp_size)
        x, y = ld.next_batch()
        with torch.no_grad():
            idx, _, pos = eng.shard_batch(x, None)
            h = eng.model.hidden(idx, pos)
        n = cfg.dump_acts_t or h.shape[1]
        if rank == 0:
            ckpt_mod.write_named(cfg.dump_acts, [("hidden", h[:, :n].float()), ("positions", pos[:n].float())])
        M.log(f"[dump] activations of {n} local tokens -> {cfg.dump_acts}")
    elif cfg.longrope_search:
        if cfg.checkpointing:
            resume_weights()
        sys.stdout = real_stdout if rank == 0 else sys.stdout
        longrope_search_loop(cfg, eng)
    elif cfg.eval_ppl:
        if cfg.checkpointing:
            resume_weights()
        windows = eval_windows(cfg, eng)
        nll = per_position_nll(cfg, eng, windows)
        if rank == 0:
            write_ppl_csv(cfg.eval_out, nll, len(windows))
        M.log(f"[eval] {len(windows)} windows, mean NLL {float(nll.mean()):.6f}, PPL {math.exp(min(float(nll.mean()), 50)):.4f} -> {cfg.eval_out}")
    else:
        on_step = (lambda s: cream_relabel(cfg, eng, source, s)) if (cfg.cream_mode != "off" and source is not None) else None
        common.train(cfg, eng, "B200", M.LLAMA_CSV, on_step_begin=on_step)
    eng.close()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
