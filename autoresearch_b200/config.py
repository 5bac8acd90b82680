"""Runtime model / schedule / training configuration.

The reference fixes every architectural number at compile time
(brain/src/config.rs:1-39) and reads the training recipe from environment
variables (brain/src/main.rs:40-93).  Here the architecture is a runtime
dataclass with named presets, while the environment-variable names, flag
names, defaults and precedence of the recipe tier are kept.
"""
from __future__ import annotations

import dataclasses
import os
from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass
class MoEConfig:
    """Mixture-of-experts block (brain/src/config.rs:28-31)."""

    n_experts: int = 8
    top_k: int = 2
    mlp_dim_e: int = 4096
    aux_coeff: float = 0.01
    # The reference never drops tokens; a capacity factor <= 0 means "no limit".
    capacity_factor: float = 0.0


@dataclass
class ModelConfig:
    """Architecture of the GPT (brain/src/config.rs:1-39)."""

    vocab: int = 8192
    seq_len: int = 2048
    d_model: int = 512
    n_head: int = 4
    head_dim: int = 128
    mlp_dim: int = 2048
    n_layer: int = 30
    ve_layers: Tuple[int, ...] = (1, 3, 5, 7)
    ve_gate_ch: int = 32
    softcap: float = 15.0
    eps: float = 1e-5
    rope_base: float = 200000.0
    init_scale: float = 0.68
    window_short: int = 256
    window_pattern: str = "SSSSL"
    ce_chunk: int = 4096
    moe: Optional[MoEConfig] = None
    name: str = "custom"

    def __post_init__(self):
        self.ve_layers = tuple(i for i in self.ve_layers if 0 <= i < self.n_layer)
        if self.n_head * self.head_dim != self.d_model:
            raise ValueError("d_model must equal n_head * head_dim")
        if self.head_dim % 2:
            raise ValueError("head_dim must be even (rotate-half RoPE)")
        if self.ve_layers and self.d_model < self.ve_gate_ch:
            raise ValueError("value-embedding gate needs d_model >= ve_gate_ch")

    # -- derived ---------------------------------------------------------
    @property
    def n_kv_head(self) -> int:
        return self.n_head

    def has_ve(self, layer: int) -> bool:
        return layer in self.ve_layers

    def is_moe_layer(self, layer: int) -> bool:
        return self.moe is not None

    def window(self, layer: int) -> int:
        """Number of keys *before* the query that stay visible (key j is seen by
        query i iff i - window <= j <= i).  A value >= seq_len means plain causal
        (brain/src/config.rs:17-24, brain/src/forward.rs:1134-1138)."""
        c = self.window_pattern[layer % len(self.window_pattern)]
        return self.window_short if c == "S" else self.seq_len

    def num_params(self) -> dict:
        D, V, L = self.d_model, self.vocab, self.n_layer
        attn = 4 * D * D * L
        if self.moe is None:
            mlp = 2 * D * self.mlp_dim * L
            router = 0
        else:
            mlp = 2 * D * self.moe.mlp_dim_e * self.moe.n_experts * L
            router = self.moe.n_experts * D * L
        ve = len(self.ve_layers) * V * D
        gate = len(self.ve_layers) * self.n_kv_head * self.ve_gate_ch
        scalars = 2 * L
        out = dict(wte=V * D, lm_head=V * D, attn=attn, mlp=mlp, router=router,
                   ve=ve, ve_gate=gate, scalars=scalars)
        out["total"] = sum(out.values())
        return out

    def flops_per_token(self) -> float:
        """6*(params - wte - ve - scalars) + sum_layers 12*H*hd*min(window, T)
        (brain/src/train.rs:152-188).  For MoE only the top_k active experts count."""
        p = self.num_params()
        dense = p["total"] - p["wte"] - p["ve"] - p["scalars"]
        if self.moe is not None:
            active = 2 * self.d_model * self.moe.mlp_dim_e * self.moe.top_k * self.n_layer
            dense = dense - p["mlp"] + active
        attn = 0
        for l in range(self.n_layer):
            attn += 12 * self.n_head * self.head_dim * min(self.window(l), self.seq_len)
        return 6.0 * dense + attn


def _preset(name: str) -> ModelConfig:
    if name == "tiny":
        return ModelConfig(vocab=256, seq_len=128, d_model=64, n_head=2, head_dim=32,
                           mlp_dim=256, n_layer=2, ce_chunk=128, name="tiny")
    if name == "tiny_moe":
        return ModelConfig(vocab=256, seq_len=128, d_model=64, n_head=2, head_dim=32,
                           mlp_dim=256, n_layer=2, ce_chunk=128, name="tiny_moe",
                           moe=MoEConfig(n_experts=4, top_k=2, mlp_dim_e=128))
    if name == "small":  # GPU smoke size: head_dim 128 so the tensor-core kernels apply
        return ModelConfig(vocab=1024, seq_len=512, d_model=256, n_head=2, head_dim=128,
                           mlp_dim=1024, n_layer=4, ce_chunk=1024, name="small")
    if name == "small_moe":
        return ModelConfig(vocab=1024, seq_len=256, d_model=256, n_head=2, head_dim=128,
                           mlp_dim=1024, n_layer=2, ce_chunk=1024, name="small_moe",
                           moe=MoEConfig(n_experts=4, top_k=2, mlp_dim_e=512, capacity_factor=2.0))
    if name == "phase1":
        return ModelConfig(vocab=8192, seq_len=2048, d_model=512, n_head=4, head_dim=128,
                           mlp_dim=2048, n_layer=30, name="phase1")
    if name == "phase2":
        return ModelConfig(vocab=8192, seq_len=32768, d_model=1024, n_head=8, head_dim=128,
                           mlp_dim=4096, n_layer=30, name="phase2")
    if name == "moe":
        return ModelConfig(vocab=8192, seq_len=8192, d_model=1024, n_head=8, head_dim=128,
                           mlp_dim=4096, n_layer=30, name="moe",
                           moe=MoEConfig(n_experts=8, top_k=2, mlp_dim_e=4096,
                                         capacity_factor=1.25))
    if name == "wide":
        return ModelConfig(vocab=8192, seq_len=8192, d_model=2048, n_head=16, head_dim=128,
                           mlp_dim=8192, n_layer=30, name="wide")
    raise KeyError(f"unknown model preset {name!r}")


PRESETS = ("tiny", "tiny_moe", "small", "small_moe", "phase1", "phase2", "moe", "wide")


def model_preset(name: str, **overrides) -> ModelConfig:
    cfg = _preset(name)
    if overrides:
        cfg = dataclasses.replace(cfg, **overrides)
    return cfg


@dataclass
class ScheduleConfig:
    """Optimizer recipe (brain/src/optim.rs:23-43,87-101)."""

    peak_lr: float = 0.04
    embedding_lr: float = 0.9
    unembedding_lr: float = 0.005
    scalar_lr: float = 0.5
    weight_decay: float = 0.2
    warmup_ratio: float = 0.0
    warmdown_ratio: float = 0.75
    final_lr_frac: float = 0.05
    schedule: str = "linear"  # or "cosine"
    adam_beta1: float = 0.8
    adam_beta2: float = 0.95
    adam_eps: float = 1e-10
    wd_wte: float = 0.001
    wd_lm_head: float = 0.01
    wd_ve: float = 0.003
    wd_router: float = 0.01
    muon_momentum_start: float = 0.85
    muon_momentum_end: float = 0.95
    muon_momentum_warmup_steps: int = 200
    muon_beta2: float = 0.95
    ns_steps: int = 5

    @staticmethod
    def from_env(env=None) -> "ScheduleConfig":
        """PEAK_LR rescales the embedding / unembedding / scalar learning rates by
        PEAK_LR / 0.04 (brain/src/main.rs:68-79)."""
        env = os.environ if env is None else env
        d = ScheduleConfig()

        def f(name, default):
            try:
                return float(env[name])
            except (KeyError, ValueError):
                return default

        peak = f("PEAK_LR", d.peak_lr)
        scale = peak / d.peak_lr
        sched = str(env.get("SCHEDULE", d.schedule)).lower()
        if sched not in ("linear", "cosine"):
            sched = "linear"
        return ScheduleConfig(
            peak_lr=peak,
            embedding_lr=d.embedding_lr * scale,
            unembedding_lr=d.unembedding_lr * scale,
            scalar_lr=d.scalar_lr * scale,
            weight_decay=f("WEIGHT_DECAY", d.weight_decay),
            warmup_ratio=f("WARMUP_RATIO", 0.0),
            warmdown_ratio=f("WARMDOWN_RATIO", d.warmdown_ratio),
            final_lr_frac=f("FINAL_LR_FRAC", d.final_lr_frac),
            schedule=sched,
        )


@dataclass
class ParallelConfig:
    dp: int = 1
    tp: int = 1
    ep: int = 1
    pp: int = 1
    # "fused" = peer-memory kernels, "nccl" = library collectives (the measured baseline)
    comm: str = "fused"
    # gradient buckets by depth for the fused data-parallel exchange: > 1 starts the reduce-scatter and the owner
    # update of the upper layers while the backward pass is still working on the lower ones; 1 = after the backward pass
    dp_buckets: int = 3

    @property
    def world(self) -> int:
        return self.dp * self.tp * self.pp

    def describe(self) -> str:
        parts = []
        for k in ("dp", "tp", "ep", "pp"):
            v = getattr(self, k)
            if v > 1:
                parts.append(f"{k}{v}")
        return "x".join(parts) if parts else "dp1"


@dataclass
class TrainConfig:
    """Driver configuration (brain/src/train.rs:629-681)."""

    device_batch_size: int = 32
    total_batch_size: int = 524288
    max_steps: Optional[int] = None
    cooldown_steps: int = 500
    data_dir: str = ""
    tokenizer_dir: str = ""
    checkpoint_dir: str = ""
    eval_interval: int = 25
    checkpoint_interval: int = 100
    load_checkpoint: Optional[str] = None
    init_weights_path: Optional[str] = None
    diagnostic_steps: Optional[int] = None
    num_train_shards: Optional[int] = None
    stream_input: bool = False
    synthetic_data: bool = False
    synthetic_kind: str = "lcg"  # "lcg" (reference stream) or "zipf"
    n_pipeline_stages: int = 1
    distributed: bool = False
    schedule_cfg: ScheduleConfig = field(default_factory=ScheduleConfig)
    impl: str = "auto"  # "oracle" | "baseline" | "sm100" | "auto"
    seed: int = 42
    log_interval: int = 5
    cooldown_trigger_file: str = "/tmp/autoresearch_cooldown"
    metrics_jsonl: Optional[str] = None
    resume: bool = False
    heartbeat_timeout_s: float = 0.0  # > 0: watch peer liveness through the process group's store
    peak_flops: Optional[float] = None  # MFU denominator per GPU; None = ARB_PEAK_TFLOPS or the nominal B200 peak
    parallel: ParallelConfig = field(default_factory=ParallelConfig)

    @staticmethod
    def from_env(env=None) -> "TrainConfig":
        env = os.environ if env is None else env

        def i(name, default):
            try:
                return int(env[name])
            except (KeyError, ValueError):
                return default

        home = env.get("HOME", "/root")
        ms = i("MAX_STEPS", 0)
        return TrainConfig(
            device_batch_size=i("BATCH_SIZE", 32),
            total_batch_size=i("TOTAL_BATCH", 524288),
            max_steps=ms if ms > 0 else None,
            cooldown_steps=i("COOLDOWN_STEPS", 500),
            data_dir=f"{home}/.cache/autoresearch/shards",
            tokenizer_dir=f"{home}/.cache/autoresearch/tokenizer",
            checkpoint_dir=env.get("CHECKPOINT_DIR", f"{home}/.cache/autoresearch/checkpoints"),
            eval_interval=i("EVAL_EVERY", 25),
            checkpoint_interval=i("CHECKPOINT_EVERY", 100),
            init_weights_path=env.get("INIT_WEIGHTS_PATH") or None,
            num_train_shards=(i("NUM_TRAIN_SHARDS", -1) if i("NUM_TRAIN_SHARDS", -1) >= 0 else None),
            synthetic_data=env.get("SYNTHETIC", "") in ("1", "true"),
            heartbeat_timeout_s=float(env.get("HEARTBEAT_TIMEOUT", "0") or 0),
            schedule_cfg=ScheduleConfig.from_env(env),
        )


def derive_accumulation(total_batch: int, device_batch: int, seq_len: int, dp: int) -> Tuple[int, int]:
    """(micro_batch_per_rank, accumulation steps) such that
    micro_batch * seq_len * dp * accum == total_batch.

    The reference floors silently (brain/src/train.rs:747-749); a combination that does
    not divide is refused here.  When one micro-step of `device_batch` sequences on every
    rank already exceeds the budget, the per-rank micro-batch shrinks (8 GPUs at T=32768:
    micro-batch 2, one accumulation step)."""
    if total_batch % seq_len:
        raise ValueError(f"TOTAL_BATCH={total_batch} is not a multiple of seq_len={seq_len}")
    seqs = total_batch // seq_len
    if seqs % dp:
        raise ValueError(f"{seqs} sequences per step do not divide over dp={dp}")
    per_rank = seqs // dp
    mb = min(device_batch, per_rank)
    while per_rank % mb:
        mb -= 1
    return mb, per_rank // mb
