"""GPT-2 context-parallel trainer — the counterpart of ``gpt2_cp_test`` (Scripts/Blutrain/gpt2_cp_test.cpp:611-1908),
configured by the same ``CP_*`` environment variables.

    torchrun --nproc-per-node 2 -m context_parallelism_b200.trainers.gpt2_cp
    CP_MODEL_44M=1 CP_T=2048 CP_ATTN_MODE=ring python -m context_parallelism_b200.trainers.gpt2_cp     # single rank

Features kept: 44M / 124–161M presets, tied or untied head, named-init load (``LOAD_INIT_NAMED``) and save
(``SAVE_INIT_NAMED``), run-numbered CSV log + checkpoints with auto-resume, validation and top-k(50) sample
generation every ``CP_VAL_FREQ`` steps (``CP_GENERATE=1``), step-0 gradient dump (``DUMP_STEP0_GRADS``) for
parity against the PyTorch reference script, memory-probe mode (``CP_MEM_PROBE``).
On a GPU the model computes in bf16 (``CP_DTYPE`` defaults to fp32 only on CPU, the oracle path).
"""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

from ..config import Config
from ..engine import TrainEngine
from ..parallel.cp_attention import CPAttention, CPContext
from ..parallel.mesh import init_distributed
from ..utils import ckpt as ckpt_mod
from ..utils import metrics as M
from . import common


@torch.no_grad()
def generate(eng: TrainEngine, prompt: torch.Tensor, n_new: int = 32, top_k: int = 50, seed: int = 42) -> torch.Tensor:
    """Top-k sampling on rank 0's replica without context parallelism, tokens broadcast to every rank so all
    ranks print the same text (the reference broadcasts each sampled token, gpt2_cp_test.cpp:1237-1346)."""
    from ..ops import xent
    model = eng.model
    saved = model.attn
    model.attn = CPAttention(eng.cfg, CPContext.single(eng.cfg))
    gen = torch.Generator(device="cpu").manual_seed(seed)
    x = prompt.to(eng.device)
    try:
        for _ in range(n_new):
            T = x.shape[1]
            pad = (-T) % 8
            xp = torch.cat([x, x.new_zeros(x.shape[0], pad)], 1) if pad else x
            pos = torch.arange(xp.shape[1], device=eng.device)
            h = model.hidden(xp, pos)[:, T - 1]
            logits = xent.logits_last(h, model.head_weight())[:, : eng.cfg.vocab_size].float().cpu()
            vals, idx = torch.topk(logits, top_k, dim=-1)
            choice = torch.multinomial(torch.softmax(vals, -1), 1, generator=gen)
            nxt = idx.gather(-1, choice).to(eng.device)
            if dist.is_initialized() and dist.get_world_size() > 1:
                dist.broadcast(nxt, 0)
            x = torch.cat([x, nxt], 1)
    finally:
        model.attn = saved
    return x


def dump_step0_grads(eng: TrainEngine, path: str) -> None:
    """Per-parameter gradient L2 norms after the averaged all-reduce of the first step
    (gpt2_cp_test.cpp:1371-1487), as ``name,l2`` lines under the named-init names."""
    grad = eng.flat.full_reduced_grad()         # collective when the optimiser state is sharded
    if eng.rank != 0:
        return
    by_param = {id(p): (o, n) for _, p, o, n in eng.flat.entries}
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        for name, view in eng.model.named_tensors().items():
            base = view._base if view._base is not None else view
            if id(base) not in by_param:
                continue
            o, n = by_param[id(base)]
            f.write(f"{name},{float(grad[o:o + n].norm()):.8e}\n")


def main() -> None:
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    cfg = Config.from_env("gpt2", world)
    if dev.type == "cuda" and cfg.dtype == "fp32":
        cfg = cfg.replace(dtype="bf16")         # the CUDA kernels compute in bf16; fp32 is the CPU oracle path
    if rank != 0:
        sys.stdout = open(os.devnull, "w")      # non-master ranks are silent (bluscriptCP.cpp:586-591)
    M.log("GPT-2 CP trainer\n" + cfg.describe())
    eng = TrainEngine(cfg, dev)
    if cfg.load_init_named:
        n = ckpt_mod.load_named_into(eng.model, eng.flat, ckpt_mod.read_named(cfg.load_init_named), strict=True)
        M.log(f"loaded {n} named tensors from {cfg.load_init_named}")
    if cfg.save_init_named:
        n = ckpt_mod.save_named_init(cfg.save_init_named, eng.model, eng.flat, rank)
        M.log(f"saved {n} named tensors to {cfg.save_init_named}")

    def periodic(step: int) -> None:
        if cfg.generate and cfg.val_freq > 0 and step % cfg.val_freq == 0 and step > 0:
            out = generate(eng, torch.tensor([[15496, 11, 314, 1101]]) % cfg.vocab_size, 16)      # "Hello, I'm" in GPT-2 BPE
            M.log("sample tokens: " + " ".join(map(str, out[0].tolist())))

    if cfg.debug.dump_step0_grads:
        from ..utils import data as data_mod
        ld = data_mod.make_loader(cfg, "train", eng.cp.dp_rank, eng.cp.dp_size)
        x, y = ld.next_batch()
        eng.forward_backward(x, y, 1, True)
        dump_step0_grads(eng, os.path.join(cfg.log_dir, "step0_grads_b200.csv"))
        eng.opt.zero_grad()
        ld.close()
    common.train(cfg, eng, "B200", M.GPT2_CSV, periodic=periodic)
    eng.close()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
