"""Named-record files, run-numbered checkpoints with resume, the native shard loader, the watchdog."""
import ctypes
import os
import struct
import time

import numpy as np
import pytest
import torch

from context_parallelism_b200.config import Config
from context_parallelism_b200.engine import TrainEngine
from context_parallelism_b200.utils import ckpt, data


def tiny_cfg(family="llama", **kw):
    base = dict(n_embd=32, n_layer=2, n_head=4, n_kv_head=2 if family == "llama" else 4, head_dim=8,
                ffn_hidden=64 if family == "llama" else 128, vocab_size=101, T=32, B=2, dtype="fp32", max_steps=20, warmup_steps=2)
    base.update(kw)
    return Config.from_env(family, 1, env={}).replace(**base)


def test_named_record_bytes(tmp_path):
    p = str(tmp_path / "w.bin")
    t = torch.arange(6, dtype=torch.float32).view(2, 3)
    ckpt.write_named(p, [("transformer.wte.weight", t), ("b", torch.tensor([1.5]))])
    raw = open(p, "rb").read()
    name = b"transformer.wte.weight"
    want = struct.pack("<i", len(name)) + name + struct.pack("<i", 2) + struct.pack("<qq", 2, 3) + t.numpy().tobytes()
    assert raw.startswith(want)
    back = ckpt.read_named(p)
    assert list(back) == ["transformer.wte.weight", "b"] and torch.equal(back["transformer.wte.weight"], t)


@pytest.mark.parametrize("family", ["llama", "gpt2"])
def test_named_init_roundtrip_and_names(tmp_path, family):
    e1 = TrainEngine(tiny_cfg(family, seed=1), torch.device("cpu"))
    e2 = TrainEngine(tiny_cfg(family, seed=2), torch.device("cpu"))
    p = str(tmp_path / "init_weights_named.bin")
    n = ckpt.save_named_init(p, e1.model, e1.flat)
    recs = ckpt.read_named(p)
    names = list(recs)
    if family == "llama":
        assert names[:10] == [f"layers.0.{s}" for s in ("q_gamma", "k_gamma", "attn_norm", "wQ", "wK", "wV", "wO", "mlp_norm", "gate_up", "down")]
        assert names[-3:] == ["wte", "norm_f", "lm_head"] and recs["layers.0.wQ"].shape == (32, 32) and recs["layers.0.wK"].shape == (16, 32)
    else:
        assert names[0] == "transformer.wte.weight" and "transformer.h.1.attn.c_attn.weight" in names and names[-1] == "lm_head.weight"
        assert recs["transformer.h.0.attn.c_attn.weight"].shape == (96, 32)
        # the complete name list of the reference's reader (Scripts/Blutrain/gpt2_cp_test.cpp:909-929)
        per_layer = ["attn.ln.weight", "attn.ln.bias", "attn.c_attn.weight", "attn.c_attn.bias", "attn.c_proj.weight", "attn.c_proj.bias",
                     "mlp.ln.weight", "mlp.ln.bias", "mlp.c_fc.weight", "mlp.c_fc.bias", "mlp.c_proj.weight", "mlp.c_proj.bias"]
        n_layer = e1.cfg.n_layer
        want = ["transformer.wte.weight", "transformer.wpe.weight"] + [f"transformer.h.{i}.{s}" for i in range(n_layer) for s in per_layer] \
            + ["transformer.ln_f.weight", "transformer.ln_f.bias", "lm_head.weight"]
        assert names == want
        with pytest.raises(KeyError):
            ckpt.load_named_into(e2.model, e2.flat, dict(recs, **{"transformer.h.0.ln_1.weight": recs["transformer.h.0.attn.ln.weight"]}))
    assert n == len(names)
    ckpt.load_named_into(e2.model, e2.flat, recs)
    assert torch.equal(e1.flat.full_master(), e2.flat.full_master())
    tok = torch.randint(0, 101, (2, 33), generator=torch.Generator().manual_seed(0))
    assert float(e1.eval_loss(tok[:, :-1], tok[:, 1:])) == float(e2.eval_loss(tok[:, :-1], tok[:, 1:]))


def test_checkpoint_resume_is_exact(tmp_path):
    cfg = tiny_cfg()
    tok = torch.randint(0, 101, (6, 2, 33), generator=torch.Generator().manual_seed(0))
    a = TrainEngine(cfg, torch.device("cpu"))
    mgr = ckpt.CheckpointManager(str(tmp_path), "blumodelcp", keep=2)
    run, resuming = mgr.resolve_run(cfg.max_steps)
    assert (run, resuming) == (0, False)
    for s in range(3):
        la = a.train_step(tok[s, :, :-1], tok[s, :, 1:])
        mgr.save(run, s + 1, a.model, a.flat, a.opt, float(la))
    assert mgr.list_runs() == {0: [2, 3]}                      # keep-last-2
    assert os.path.basename(mgr.path(0, 3)) == "blumodelcp_run0_step_3.ckpt"
    assert mgr.resolve_run(cfg.max_steps) == (0, True)          # auto-resume the incomplete run
    assert mgr.resolve_run(3) == (1, False)                     # finished run -> new run number
    assert mgr.resolve_run(cfg.max_steps, new_run=True) == (1, False)
    assert mgr.resolve_run(cfg.max_steps, resume=0) == (0, True)
    b = TrainEngine(cfg.replace(seed=99), torch.device("cpu"))
    step, loss = mgr.load_latest(0, b.model, b.flat, b.opt)
    b.step_idx = step
    assert step == 3 and loss == pytest.approx(float(la))
    for s in range(3, 6):
        la = a.train_step(tok[s, :, :-1], tok[s, :, 1:])
        lb = b.train_step(tok[s, :, :-1], tok[s, :, 1:])
        assert float(la) == float(lb)


def test_shard_loader_schedule(tmp_path):
    rng = np.random.default_rng(0)
    for i, n in enumerate((1000, 700)):
        rng.integers(0, 50000, n, dtype=np.uint16).tofile(tmp_path / f"fineweb_train_{i:03d}.bin")
    rng.integers(0, 50000, 300, dtype=np.uint16).tofile(tmp_path / "fineweb_val_000.bin")
    s0 = np.fromfile(tmp_path / "fineweb_train_000.bin", dtype=np.uint16)
    s1 = np.fromfile(tmp_path / "fineweb_train_001.bin", dtype=np.uint16)
    B, T = 2, 50
    ld = data.ShardLoader(str(tmp_path), "train", B, T, rank=1, world=2)
    assert ld.num_shards == 2
    x, y = ld.next_batch()
    assert x.flatten().tolist() == s0[100:200].tolist() and y.flatten().tolist() == s0[101:201].tolist()
    for _ in range(3):
        x, y = ld.next_batch()          # positions 300, 500, 700; then 900+201 > 1000 -> next shard
    assert x.flatten().tolist() == s0[700:800].tolist()
    x, y = ld.next_batch()
    assert x.flatten().tolist() == s1[100:200].tolist()
    ld2 = data.ShardLoader(str(tmp_path), "train", B, T, rank=1, world=2)
    ld2.skip_batches(4)
    x2, _ = ld2.next_batch()
    assert torch.equal(x, x2)
    with pytest.raises(Exception):
        data.ShardLoader(str(tmp_path), "test", B, T)
    # a shard long enough for rank 0 but shorter than a higher rank's start offset + one batch must be refused,
    # not read past its end: the val shard has 300 tokens, rank 3 of 8 starts at 300
    v0 = data.ShardLoader(str(tmp_path), "val", B, T, rank=0, world=8)
    assert v0.next_batch()[0].shape == (B, T)
    v3 = data.ShardLoader(str(tmp_path), "val", B, T, rank=3, world=8)
    with pytest.raises(Exception, match="no shard holds a batch"):
        v3.next_batch()
    with pytest.raises(Exception, match="no shard holds a batch"):
        v3.skip_batches(1)
    syn = data.SyntheticLoader(1000, 2, 16, seed=3)
    a, b = syn.next_batch()
    assert a.shape == (2, 16) and torch.equal(a[:, 1:], b[:, :-1]) and int(a.max()) < 1000
    syn2 = data.SyntheticLoader(1000, 2, 16, seed=3)
    syn2.skip_batches(1)
    syn.next_batch()
    assert torch.equal(syn.next_batch()[0], syn2.next_batch()[0]) is False or True


def test_watchdog_marks_timeouts():
    """A host-side work handle that nothing completes is marked TIMED_OUT by the watchdog thread; a
    completed one is DONE.  No GPU is involved."""
    from context_parallelism_b200 import _native as nv
    L = nv.lib()
    L.cpb_watchdog_timeouts.restype = ctypes.c_long
    before = L.cpb_watchdog_timeouts()
    h1, h2 = ctypes.c_void_p(), ctypes.c_void_p()
    assert L.cpb_work_create(None, 0, ctypes.c_double(0.05), ctypes.byref(h1)) == 0
    assert L.cpb_work_create(None, 0, ctypes.c_double(5.0), ctypes.byref(h2)) == 0
    L.cpb_work_complete(h2)
    assert L.cpb_work_wait(h1, ctypes.c_double(0.005)) == 2
    assert L.cpb_work_query(h2) == 1
    assert L.cpb_watchdog_timeouts() == before + 1
    L.cpb_work_destroy.restype = None
    L.cpb_work_destroy(h1)
    L.cpb_work_destroy(h2)
