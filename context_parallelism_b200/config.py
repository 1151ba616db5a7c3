"""Environment-variable configuration, parsed once.

The reference trainers read ~95 environment variables ad hoc with ``getenv`` at the
point of use, some inside hot loops (context_parallel/ContextParallel.h:546-553,818,901;
Scripts/Blutrain/bluscriptCP.cpp:600-700; Scripts/Blutrain/gpt2_cp_test.cpp:645-763).
Here the same names and defaults are parsed exactly once into immutable dataclasses that
are passed down explicitly.  Unknown ``CP_*`` names produce a warning so that a typo is
never silently ignored.

Toggle convention (ContextParallel.h:546-548): unset or ``"0"`` means "default/off".
"""
from __future__ import annotations

import dataclasses
import os
import warnings
from dataclasses import dataclass, field
from typing import Mapping, Optional


def _flag(env: Mapping[str, str], name: str, default: bool = False) -> bool:
    v = env.get(name)
    if v is None or v == "":
        return default
    return v[0] not in ("0", "n", "N", "f", "F")


def _int(env: Mapping[str, str], name: str, default: int) -> int:
    v = env.get(name)
    return default if v in (None, "") else int(v)


def _float(env: Mapping[str, str], name: str, default: float) -> float:
    v = env.get(name)
    return default if v in (None, "") else float(v)


def _str(env: Mapping[str, str], name: str, default: str) -> str:
    v = env.get(name)
    return default if v is None else v


# Every variable the framework understands (the reference's complete surface).
KNOWN_ENV = {
    # topology & mode
    "CP_SIZE", "CP_ATTN_MODE", "CP_ULYSSES_SIZE", "CP_RING_OUTER", "CP_ROTATOR", "NO_GPUS_PER_NODE",
    # model / data / optimisation
    "CP_MODEL_44M", "CP_T", "CP_N_EMBD", "CP_N_LAYER", "CP_N_HEAD", "CP_WEIGHT_TYING", "CP_N_KVHEAD",
    "CP_FFN", "CP_B", "CP_GLOBAL_BATCH", "CP_MAX_STEPS", "CP_WARMUP", "CP_DATA_ROOT", "CP_RECOMPUTE_K",
    "CP_SHARE_FWD_ROTATOR", "CP_NO_GRAD_ALLREDUCE", "CP_VOCAB", "CP_HEAD_DIM", "CP_ROPE_THETA",
    "CP_DTYPE", "CP_RECOMPUTE", "CP_SYNTHETIC", "CP_SEED", "CP_LR", "CP_MIN_LR",
    # precision / memory
    "CP_RING_BF16", "CP_SAVE_KV_BF16", "ATTN_FP32", "CP_FWD_TI_SM89", "USE_PER_STEP_LSE",
    # RoPE / context extension
    "YARN_SCALE", "YARN_ORIG_MAXPOS", "YARN_BETA_FAST", "YARN_BETA_SLOW", "YARN_NO_MSCALE",
    "CP_CREAM_MODE", "CP_CREAM_SIGMA", "CP_CREAM_SEED", "CP_CREAM_LOG",
    "CP_LONGROPE_FACTORS", "CP_LONGROPE_MSCALE", "CP_LONGROPE_SEARCH",
    # checkpoint / LR
    "CP_CKPT", "CP_CKPT_FREQ", "CP_CKPT_NEW_RUN", "CP_CKPT_RESUME", "CP_CKPT_DIR", "CP_REWARMUP",
    "CP_REWARMUP_PEAK", "CP_REWARMUP_ANCHOR", "LOAD_INIT_NAMED", "LOAD_INIT_WEIGHTS", "SAVE_INIT_NAMED",
    # eval / dump modes
    "CP_EVAL_PPL", "CP_EVAL_WINDOWS", "CP_EVAL_SKIP_WINDOWS", "CP_EVAL_OUT", "CP_EVAL_TOKENS_BIN",
    "CP_DUMP_ROPE", "CP_DUMP_ROPE_SEQLEN", "CP_DUMP_NAMED", "CP_DUMP_ACTS", "CP_DUMP_ACTS_T",
    "CP_MEM_PROBE", "CP_MEM_PROBE_STEPS", "CP_MODEL_LABEL", "MEM_SNAPSHOT_DIR", "CP_ALLOC_CSV",
    "CP_LOG_DIR", "CP_VAL_FREQ", "CP_VAL_STEPS", "CP_GENERATE",
    # overlap diagnostics
    "CP_NO_OVERLAP", "CP_NO_OVERLAP_FWD", "CP_NO_OVERLAP_BWD", "CP_RING_BLOCKING", "CP_SYNC_RING",
    "CP_FWD_SYNC_RECV", "CP_FWD_SYNC_RETURN", "CP_DRAIN_AT", "CP_SELFCHECK",
    # parity dumps
    "DUMP_FWD", "DUMP_STEP0_GRADS", "CP_DEBUG_DUMP", "CP_DEBUG_SHAPES", "DUMP_CP_OUT", "DUMP_CP_STEPS",
    "DUMP_CP_DEEP", "DUMP_CP_DEEP_FWD", "DUMP_CP_MERGE", "CP_DUMP_KV_CHUNKS", "CP_DUMP_KV_CALL",
    "SKIP_DKV_ROTATION", "ITER0_ONLY_DKV",
    # test only
    "CP_RING_SIZE", "CP_HYBRID_GQA",
    # this framework's additions
    "CP_FUSED", "CP_WATCHDOG_S", "CP_NVLS", "CP_GRAD_BUCKET_MB", "CP_DKV_MODE", "CP_SHARD_OPTIM", "CP_AR_CTAS",
    "CP_FUSED_HYBRID_ULYSSES", "CP_LOAD_BALANCE", "CP_INIT_DEVICE", "CP_TEST_LOG_DIR", "CP_NATIVE_PG",
}


@dataclass(frozen=True)
class YarnConfig:
    """YaRN NTK-by-parts parameters (context_parallel/YARNOps.cpp:55-66)."""
    scale: float = 1.0
    orig_maxpos: float = 1024.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    no_mscale: bool = False

    @staticmethod
    def from_env(env: Optional[Mapping[str, str]] = None) -> "YarnConfig":
        env = os.environ if env is None else env
        return YarnConfig(
            scale=_float(env, "YARN_SCALE", 1.0),
            orig_maxpos=_float(env, "YARN_ORIG_MAXPOS", 1024.0),
            beta_fast=_float(env, "YARN_BETA_FAST", 32.0),
            beta_slow=_float(env, "YARN_BETA_SLOW", 1.0),
            no_mscale=_flag(env, "YARN_NO_MSCALE"),
        )


@dataclass(frozen=True)
class DebugConfig:
    """Overlap diagnostics and parity dumps (ContextParallel.h:546-553,675,818,901,1260)."""
    no_overlap: bool = False
    no_overlap_fwd: bool = False
    no_overlap_bwd: bool = False
    ring_blocking: bool = False
    sync_ring: bool = False
    fwd_sync_recv: bool = False
    fwd_sync_return: bool = False
    drain_at: int = 0
    selfcheck: bool = False
    use_per_step_lse: bool = False
    skip_dkv_rotation: bool = False
    iter0_only_dkv: bool = False
    dump_fwd: bool = False
    dump_step0_grads: bool = False
    debug_shapes: bool = False
    dump_cp_out: bool = False
    dump_cp_steps: bool = False
    dump_cp_merge: bool = False
    dump_kv_chunks: bool = False

    @staticmethod
    def from_env(env: Optional[Mapping[str, str]] = None) -> "DebugConfig":
        env = os.environ if env is None else env
        return DebugConfig(
            no_overlap=_flag(env, "CP_NO_OVERLAP"),
            no_overlap_fwd=_flag(env, "CP_NO_OVERLAP_FWD"),
            no_overlap_bwd=_flag(env, "CP_NO_OVERLAP_BWD"),
            ring_blocking=_flag(env, "CP_RING_BLOCKING"),
            sync_ring=_flag(env, "CP_SYNC_RING"),
            fwd_sync_recv=_flag(env, "CP_FWD_SYNC_RECV"),
            fwd_sync_return=_flag(env, "CP_FWD_SYNC_RETURN"),
            drain_at=_int(env, "CP_DRAIN_AT", 0),
            selfcheck=_flag(env, "CP_SELFCHECK"),
            use_per_step_lse=_flag(env, "USE_PER_STEP_LSE"),
            skip_dkv_rotation=_flag(env, "SKIP_DKV_ROTATION"),
            iter0_only_dkv=_flag(env, "ITER0_ONLY_DKV"),
            dump_fwd=_flag(env, "DUMP_FWD"),
            dump_step0_grads=_flag(env, "DUMP_STEP0_GRADS"),
            debug_shapes=_flag(env, "CP_DEBUG_SHAPES"),
            dump_cp_out=_flag(env, "DUMP_CP_OUT"),
            dump_cp_steps=_flag(env, "DUMP_CP_STEPS"),
            dump_cp_merge=_flag(env, "DUMP_CP_MERGE"),
            dump_kv_chunks=_flag(env, "CP_DUMP_KV_CHUNKS"),
        )


@dataclass(frozen=True)
class Config:
    """All trainer settings.  ``family`` selects the default table: ``"gpt2"`` mirrors
    gpt2_cp_test.cpp:648-760, ``"llama"`` mirrors bluscriptCP.cpp:101-171,600-700."""
    family: str = "llama"
    # topology
    world_size: int = 1
    cp_size: int = 1
    attn_mode: str = "ulysses"          # ring | ulysses | hybrid
    ulysses_size: int = 1
    ring_outer: bool = False
    rotator: str = "fused"              # fused | p2p | alltoall | allgather
    gpus_per_node: int = 8
    # model
    n_embd: int = 384
    n_layer: int = 6
    n_head: int = 6
    n_kv_head: int = 2
    head_dim: int = 64
    ffn_hidden: int = 1024
    vocab_size: int = 50304
    weight_tying: bool = False
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    qk_eps: float = 1e-6
    dtype: str = "bf16"
    # data / optimisation
    B: int = 2
    T: int = 4096
    global_batch: int = 524288
    max_steps: int = 917
    warmup_steps: int = 91
    max_lr: float = 6e-4
    min_lr: float = 6e-5
    weight_decay: float = 0.1
    grad_clip: float = 1.0
    beta1: float = 0.9
    beta2: float = 0.95
    adam_eps: float = 1e-8
    data_root: str = ""
    synthetic: bool = False
    seed: int = 1234
    val_freq: int = 250
    val_steps: int = 20
    generate: bool = False
    # CP behaviour
    recompute_k: bool = False
    recompute: str = "none"             # none | selective | full
    share_fwd_rotator: bool = False
    no_grad_allreduce: bool = False
    ring_bf16: bool = True
    save_kv_bf16: bool = True
    attn_fp32: bool = False
    dkv_mode: str = "route"             # route (red.add into the owner, fastest) | pull (deterministic, rank-ordered sum)
    shard_optim: bool = True            # fused transport: reduce-scatter -> AdamW on the owned slice -> all-gather
    load_balance_ring: bool = True      # HeadTail sharding on the ring axis; False = contiguous shards
    grad_bucket_mb: int = 25
    nvls: bool = False
    watchdog_s: float = 600.0
    # context extension
    yarn: YarnConfig = field(default_factory=YarnConfig)
    cream_mode: str = "off"             # off | cream | pose | randpos
    cream_sigma: float = 3.0
    cream_seed: int = 0
    cream_log: bool = False
    longrope_factors: str = ""
    longrope_mscale: float = 1.0
    longrope_search: bool = False
    # checkpoint / LR
    checkpointing: bool = True
    ckpt_freq: int = 50
    ckpt_keep: int = 6
    ckpt_dir: str = "checkpoints_bluscriptcp"
    ckpt_prefix: str = "blumodelcp"
    ckpt_new_run: bool = False
    ckpt_resume: int = -1
    rewarmup_steps: int = 0
    rewarmup_peak: float = 1.0
    rewarmup_anchor: int = -1
    load_init_named: str = ""
    save_init_named: str = ""
    # modes
    eval_ppl: bool = False
    eval_windows: int = 16
    eval_skip_windows: int = 0
    eval_out: str = "ppl_by_pos.csv"
    eval_tokens_bin: str = ""
    dump_rope: str = ""
    dump_rope_seqlen: int = 0
    dump_named: str = ""
    dump_acts: str = ""
    dump_acts_t: int = 0
    mem_probe: bool = False
    mem_probe_steps: int = 2
    model_label: str = ""
    mem_snapshot_dir: str = "."
    alloc_csv: str = ""
    log_dir: str = "."
    debug: DebugConfig = field(default_factory=DebugConfig)

    # ------------------------------------------------------------------ derived
    @property
    def vocab_padded(self) -> int:
        """Embedding / lm_head rows: the vocabulary rounded up to a multiple of 64 (the reference pads 50257 to
        50304 for the same reason, bluscriptCP.cpp:111); padding rows are zero and never enter the softmax."""
        return (self.vocab_size + 63) // 64 * 64

    @property
    def dp_size(self) -> int:
        return self.world_size // self.cp_size

    @property
    def ring_size(self) -> int:
        return self.cp_size // self.ulysses_size if self.attn_mode == "hybrid" else (
            self.cp_size if self.attn_mode == "ring" else 1)

    @property
    def load_balance(self) -> bool:
        """HeadTail is used on the ring axis (ring and hybrid) unless ``CP_LOAD_BALANCE=0``; Ulysses shards
        contiguously."""
        return self.attn_mode in ("ring", "hybrid") and self.load_balance_ring

    @property
    def t_local(self) -> int:
        return self.T // self.cp_size

    @property
    def grad_accum(self) -> int:
        per_step = self.B * self.T * self.dp_size
        return max(1, self.global_batch // per_step)

    def replace(self, **kw) -> "Config":
        return dataclasses.replace(self, **kw)

    # ------------------------------------------------------------------ parsing
    @staticmethod
    def from_env(family: str = "llama", world_size: int = 1,
                 env: Optional[Mapping[str, str]] = None) -> "Config":
        env = os.environ if env is None else env
        for k in env:
            if k.startswith("CP_") and k not in KNOWN_ENV:
                warnings.warn(f"unknown environment variable {k} (ignored)")
        if family == "gpt2":
            return _gpt2_from_env(env, world_size)
        if family == "llama":
            return _llama_from_env(env, world_size)
        raise ValueError(f"unknown family {family!r}")

    def validate(self) -> None:
        """Loud start-up checks (bluscriptCP.cpp:691-872)."""
        def die(msg):
            raise ValueError(msg)
        if self.world_size % self.cp_size:
            die(f"world_size={self.world_size} % CP_SIZE={self.cp_size} != 0")
        if self.attn_mode not in ("ring", "ulysses", "hybrid"):
            die(f"CP_ATTN_MODE={self.attn_mode!r} must be ring|ulysses|hybrid")
        if self.n_embd % self.n_head and self.family == "gpt2":
            die("n_embd % n_head != 0")
        if self.n_head % self.n_kv_head:
            die(f"q_heads={self.n_head} % kv_heads={self.n_kv_head} != 0")
        if self.T % (2 * self.cp_size) and self.load_balance:
            die(f"T={self.T} must be a multiple of 2*CP_SIZE={2 * self.cp_size} for HeadTail")
        if self.T % self.cp_size:
            die(f"T={self.T} % CP_SIZE={self.cp_size} != 0")
        if self.attn_mode == "ulysses" and self.cp_size > 1:
            p = self.cp_size
            if self.n_head % p:
                die(f"ulysses: q_heads={self.n_head} % P={p} != 0")
            if self.n_kv_head % p and p % self.n_kv_head:
                die(f"ulysses: kv_heads={self.n_kv_head} and P={p} must divide one another")
        if self.attn_mode == "hybrid":
            u = self.ulysses_size
            if self.cp_size % u:
                die(f"hybrid: CP_SIZE={self.cp_size} % CP_ULYSSES_SIZE={u} != 0")
            if self.n_head % u or self.n_kv_head % u:
                die(f"hybrid: q_heads={self.n_head} and kv_heads={self.n_kv_head} must be multiples of U={u}")
            r = self.cp_size // u
            if self.T % (2 * r * u):
                die(f"hybrid: T={self.T} must be a multiple of 2*R*U={2 * r * u}")
        if self.cream_mode != "off" and self.cp_size != 1:
            die("CP_CREAM_MODE requires CP_SIZE=1 (bluscriptCP.cpp:717-719)")
        if self.eval_ppl and self.dp_size != 1:
            die("CP_EVAL_PPL requires DP=1")
        if self.dkv_mode not in ("route", "pull"):
            die(f"CP_DKV_MODE={self.dkv_mode!r} must be route|red|pull")
        if self.recompute not in ("none", "selective", "full"):
            die(f"CP_RECOMPUTE={self.recompute!r} must be none|selective|full")
        # knobs of the reference that have no counterpart here are refused loudly instead of being ignored
        if self.nvls:
            die("CP_NVLS=1 is not supported: the gradient reduction uses plain peer loads (no multimem / NVLS kernel is built)")
        if self.debug.use_per_step_lse:
            die("USE_PER_STEP_LSE=1 is not supported: the kernels keep one running (m, l, O) per row, there is no per-step LSE")
        if self.dtype == "bf16" and not self.ring_bf16:
            die("CP_RING_BF16=0 is not supported with CP_DTYPE=bf16: K/V travel in the compute dtype (fp32 transport is the CP_DTYPE=fp32 oracle path)")
        if self.dtype == "bf16" and not self.save_kv_bf16:
            die("CP_SAVE_KV_BF16=0 is not supported with CP_DTYPE=bf16: K/V are kept in the compute dtype")
        if not self.load_balance_ring and self.attn_mode == "hybrid":
            die("CP_LOAD_BALANCE=0 is supported in ring mode only")

    def describe(self) -> str:
        lines = []
        for f in dataclasses.fields(self):
            v = getattr(self, f.name)
            if dataclasses.is_dataclass(v):
                continue
            lines.append(f"{f.name}={v}")
        return "\n".join(lines)


def _common(env, world_size):
    rot = _str(env, "CP_ROTATOR", "fused").lower()
    if rot not in ("fused", "p2p", "alltoall", "allgather"):
        rot = "alltoall"    # the reference maps every unknown value to AlltoAll (bluscriptCP.cpp:621)
    return dict(
        world_size=world_size,
        gpus_per_node=_int(env, "NO_GPUS_PER_NODE", 8),
        rotator=rot,
        ulysses_size=_int(env, "CP_ULYSSES_SIZE", 1),
        ring_outer=_flag(env, "CP_RING_OUTER"),
        recompute_k=_flag(env, "CP_RECOMPUTE_K"),
        recompute=_str(env, "CP_RECOMPUTE", "none"),
        no_grad_allreduce=_flag(env, "CP_NO_GRAD_ALLREDUCE"),
        ring_bf16=_flag(env, "CP_RING_BF16", True),
        save_kv_bf16=_flag(env, "CP_SAVE_KV_BF16", True),
        attn_fp32=_flag(env, "ATTN_FP32"),
        dkv_mode={"red": "route"}.get(_str(env, "CP_DKV_MODE", "route").lower(), _str(env, "CP_DKV_MODE", "route").lower()),
        shard_optim=_flag(env, "CP_SHARD_OPTIM", True),
        load_balance_ring=_flag(env, "CP_LOAD_BALANCE", True),
        grad_bucket_mb=_int(env, "CP_GRAD_BUCKET_MB", 25),
        nvls=_flag(env, "CP_NVLS", False),
        watchdog_s=_float(env, "CP_WATCHDOG_S", 600.0),
        data_root=_str(env, "CP_DATA_ROOT", ""),
        synthetic=_flag(env, "CP_SYNTHETIC") or not _str(env, "CP_DATA_ROOT", ""),
        seed=_int(env, "CP_SEED", 1234),
        yarn=YarnConfig.from_env(env),
        cream_mode=_str(env, "CP_CREAM_MODE", "off"),
        cream_sigma=_float(env, "CP_CREAM_SIGMA", 3.0),
        cream_seed=_int(env, "CP_CREAM_SEED", 0),
        cream_log=_flag(env, "CP_CREAM_LOG"),
        longrope_factors=_str(env, "CP_LONGROPE_FACTORS", ""),
        longrope_mscale=_float(env, "CP_LONGROPE_MSCALE", 1.0),
        longrope_search=_flag(env, "CP_LONGROPE_SEARCH"),
        ckpt_new_run=_flag(env, "CP_CKPT_NEW_RUN"),
        ckpt_resume=_int(env, "CP_CKPT_RESUME", -1),
        rewarmup_steps=_int(env, "CP_REWARMUP", 0),
        rewarmup_peak=_float(env, "CP_REWARMUP_PEAK", 1.0),
        rewarmup_anchor=_int(env, "CP_REWARMUP_ANCHOR", -1),
        load_init_named=_str(env, "LOAD_INIT_NAMED", ""),
        save_init_named=_str(env, "SAVE_INIT_NAMED", ""),
        eval_ppl=_flag(env, "CP_EVAL_PPL"),
        eval_windows=_int(env, "CP_EVAL_WINDOWS", 16),
        eval_skip_windows=_int(env, "CP_EVAL_SKIP_WINDOWS", 0),
        eval_out=_str(env, "CP_EVAL_OUT", "ppl_by_pos.csv"),
        eval_tokens_bin=_str(env, "CP_EVAL_TOKENS_BIN", ""),
        dump_rope=_str(env, "CP_DUMP_ROPE", ""),
        dump_rope_seqlen=_int(env, "CP_DUMP_ROPE_SEQLEN", 0),
        dump_named=_str(env, "CP_DUMP_NAMED", ""),
        dump_acts=_str(env, "CP_DUMP_ACTS", ""),
        dump_acts_t=_int(env, "CP_DUMP_ACTS_T", 0),
        mem_probe=_flag(env, "CP_MEM_PROBE"),
        mem_probe_steps=_int(env, "CP_MEM_PROBE_STEPS", 2),
        mem_snapshot_dir=_str(env, "MEM_SNAPSHOT_DIR", "."),
        alloc_csv=_str(env, "CP_ALLOC_CSV", ""),
        log_dir=_str(env, "CP_LOG_DIR", "."),
        generate=_flag(env, "CP_GENERATE"),
        debug=DebugConfig.from_env(env),
    )


def _gpt2_from_env(env, world_size) -> Config:
    small = _flag(env, "CP_MODEL_44M")
    n_embd = _int(env, "CP_N_EMBD", 384 if small else 768)
    n_layer = _int(env, "CP_N_LAYER", 3 if small else 12)
    n_head = _int(env, "CP_N_HEAD", 6 if small else 12)
    max_steps = _int(env, "CP_MAX_STEPS", 6768 if small else 1555)
    kw = _common(env, world_size)
    kw.update(
        family="gpt2",
        cp_size=_int(env, "CP_SIZE", world_size),
        attn_mode=_str(env, "CP_ATTN_MODE", "ring"),
        n_embd=n_embd, n_layer=n_layer, n_head=n_head, n_kv_head=n_head,
        head_dim=n_embd // n_head, ffn_hidden=4 * n_embd,
        vocab_size=_int(env, "CP_VOCAB", 50304),
        weight_tying=_flag(env, "CP_WEIGHT_TYING", False),
        dtype=_str(env, "CP_DTYPE", "fp32"),
        B=_int(env, "CP_B", 4), T=_int(env, "CP_T", 1024),
        global_batch=_int(env, "CP_GLOBAL_BATCH", 65536 if small else 524288),
        max_steps=max_steps, warmup_steps=_int(env, "CP_WARMUP", max(1, max_steps // 10)),
        max_lr=_float(env, "CP_LR", 6e-4), min_lr=_float(env, "CP_MIN_LR", 6e-5),
        val_freq=_int(env, "CP_VAL_FREQ", 100), val_steps=_int(env, "CP_VAL_STEPS", 5),
        share_fwd_rotator=_flag(env, "CP_SHARE_FWD_ROTATOR", True),
        checkpointing=_flag(env, "CP_CKPT", False),
        ckpt_freq=_int(env, "CP_CKPT_FREQ", 100), ckpt_keep=5,
        ckpt_dir=_str(env, "CP_CKPT_DIR", "cp_checkpoints"), ckpt_prefix="gpt2_cp",
        model_label=_str(env, "CP_MODEL_LABEL", "44M" if small else "161M"),
    )
    return Config(**kw)


def _llama_from_env(env, world_size) -> Config:
    d = _int(env, "CP_N_EMBD", 384)
    nh = _int(env, "CP_N_HEAD", 6)
    kw = _common(env, world_size)
    kw.update(
        family="llama",
        cp_size=_int(env, "CP_SIZE", world_size),
        attn_mode=_str(env, "CP_ATTN_MODE", "ulysses"),
        n_embd=d, n_layer=_int(env, "CP_N_LAYER", 6), n_head=nh,
        n_kv_head=_int(env, "CP_N_KVHEAD", 2),
        head_dim=_int(env, "CP_HEAD_DIM", d // nh),
        ffn_hidden=_int(env, "CP_FFN", (8 * d) // 3),
        vocab_size=_int(env, "CP_VOCAB", 50304),
        weight_tying=_flag(env, "CP_WEIGHT_TYING", False),
        rope_theta=_float(env, "CP_ROPE_THETA", 500000.0),
        dtype=_str(env, "CP_DTYPE", "bf16"),
        B=_int(env, "CP_B", 2), T=_int(env, "CP_T", 4096),
        global_batch=_int(env, "CP_GLOBAL_BATCH", 524288),
        max_steps=_int(env, "CP_MAX_STEPS", 917), warmup_steps=_int(env, "CP_WARMUP", 91),
        max_lr=_float(env, "CP_LR", 6e-4), min_lr=_float(env, "CP_MIN_LR", 6e-5),
        val_freq=_int(env, "CP_VAL_FREQ", 250), val_steps=_int(env, "CP_VAL_STEPS", 20),
        share_fwd_rotator=_flag(env, "CP_SHARE_FWD_ROTATOR", False),
        checkpointing=_flag(env, "CP_CKPT", True),
        ckpt_freq=_int(env, "CP_CKPT_FREQ", 50), ckpt_keep=6,
        ckpt_dir=_str(env, "CP_CKPT_DIR", "checkpoints_bluscriptcp"), ckpt_prefix="blumodelcp",
        model_label=_str(env, "CP_MODEL_LABEL", "bluscriptcp"),
    )
    return Config(**kw)
