"""TOML configuration schema: ``[model]``, ``[optim]``, ``[parallel]``, ``[train]``, ``[data]``, ``[ckpt]``.

The ``[model]`` and ``[optim]`` tables accept exactly the key names of the
reference's axis files (config/model/minicpm4_0.5b.toml:22-56,
config/optim/default.toml) and of its rendered gate products, whose ``[cli]``
table carries the run shape (workload/src/config/long-train.toml:4-30).  HF-style
aliases (``scale_emb``, ``dim_model_base``, ``scale_depth``) map onto the muP keys
(ref/reference/minicpm4_8b_hf_singlecard/hf_model/config.json:37-40).  Unknown keys
are rejected, as harness/config_runtime.py:191-234 does.  The ``[parallel]`` table is
new: the reference only has ``tensor_parallel_size`` as a product key.
"""
from __future__ import annotations

import dataclasses
import math
import os
import tomllib
from dataclasses import dataclass, field
from typing import Any

_MODEL_ALIASES = {
    "scale_emb": "mup_emb_scale",
    "dim_model_base": "mup_base_hidden_size",
    "scale_depth": "mup_depth_scale",
    "num_hidden_layers": "num_layers",
    "intermediate_size": "ffn_hidden_size",
    "num_key_value_heads": "num_query_groups",
    "vocab_size": "padded_vocab_size",
    "rms_norm_eps": "norm_epsilon",
    "rope_theta": "rotary_base",
    "tie_word_embeddings": "tie_embeddings",
    "initializer_range": "init_method_std",
}


@dataclass(frozen=True)
class ModelConfig:
    name: str = "custom"
    num_layers: int = 2
    hidden_size: int = 256
    ffn_hidden_size: int = 1024
    num_attention_heads: int = 4
    num_query_groups: int = 2
    head_dim: int = 64
    seq_length: int = 256
    max_position_embeddings: int = 0  # 0 -> seq_length
    padded_vocab_size: int = 8192
    rotary_base: float = 10000.0
    norm_epsilon: float = 1e-6
    init_method_std: float = 0.02
    mup_base_hidden_size: int = 256
    mup_emb_scale: float = 12.0
    mup_depth_scale: float = 1.4
    mtp_num_layers: int = 0
    mtp_loss_weight: float = 0.0
    tie_embeddings: bool = False
    qk_norm: bool = False  # Qwen3-style per-head RMSNorm on q and k (model_qwen3.py:102-156)
    use_mup: bool = True

    def __post_init__(self):
        if self.num_attention_heads % self.num_query_groups:
            raise ValueError("num_attention_heads must be a multiple of num_query_groups")
        if self.max_position_embeddings == 0:
            object.__setattr__(self, "max_position_embeddings", self.seq_length)

    # derived geometry -----------------------------------------------------
    @property
    def q_per_kv(self) -> int:
        return self.num_attention_heads // self.num_query_groups

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_query_groups * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    @property
    def width_mult(self) -> float:
        if not self.use_mup:
            return 1.0
        return self.hidden_size / float(self.mup_base_hidden_size)

    @property
    def emb_scale(self) -> float:
        return self.mup_emb_scale if self.use_mup else 1.0

    def depth_scale(self, extra_layers: int = 0) -> float:
        """Residual-branch multiplier ``mup_depth_scale / sqrt(L)`` (train_loop.py:1562-1567)."""
        if not self.use_mup:
            return 1.0
        return self.mup_depth_scale / math.sqrt(self.num_layers + extra_layers)

    def flops_per_token(self, with_mtp: bool | None = None) -> float:
        """Training FLOPs per token by GEMM enumeration, times 3 (train_loop.py:724-747)."""
        H, Hq, Hkv = float(self.hidden_size), float(self.q_dim), float(self.kv_dim)
        S, F, V = float(self.seq_length), float(self.ffn_hidden_size), float(self.padded_vocab_size)
        per_layer = 2.0 * H * (Hq + 2.0 * Hkv) + 2.0 * Hq * H + 2.0 * S * Hq + 6.0 * H * F
        head = 2.0 * H * V
        n_mtp = float(self.mtp_num_layers if with_mtp is None or with_mtp else 0)
        mtp = n_mtp * (per_layer + 2.0 * (2.0 * H) * H + head)
        return 3.0 * (self.num_layers * per_layer + head + mtp)


@dataclass(frozen=True)
class OptimConfig:
    lr: float = 1e-3
    min_lr: float = 0.0
    lr_warmup_iters: int = 0
    lr_decay_iters: int = 0
    lr_wsd_decay_iters: int = 0
    weight_decay: float = 0.1
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8
    clip_grad: float = 1.0
    lr_schedule: str = "wsd"  # "wsd" (train_loop.py:173-186) | "cosine" | "constant"


@dataclass(frozen=True)
class ParallelConfig:
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    virtual_pipeline_stages: int = 1
    sequence_parallel: bool = False
    context_parallel_size: int = 1
    use_distributed_optimizer: bool = False
    ddp_bucket_elems: int = 40_000_000
    overlap_grad_reduce: bool = True
    fused_comm: bool = True  # in-kernel NVLink collectives where available
    fp8: str = "off"  # "off" | "mxfp8"
    # Layers per pipeline model chunk, in chunk order (chunk v*pp + p lives on stage p); empty = an even split.  The last
    # chunk also runs the final norm, the LM head and the loss (about 2.6 layers' worth of work at the 0.5B shape), so an
    # even split leaves the last stage the slowest: e.g. (7, 6, 6, 5) for 24 layers on pp = 2 x 2 virtual stages
    # (Megatron: --decoder-first/last-pipeline-num-layers).
    pipeline_layer_split: tuple = ()
    # "global": the clip norm is the L2 norm of the whole model's gradient (every model-parallel shard once), Megatron's rule.
    # "tp_local": every TP rank clips by the norm of ITS OWN shards (replicated weights counted on every rank), which is what
    # the hand-written DP x TP reference does (ref/reference/train_minicpm4_8b_tp.py:321) and what its dptp gate compares.
    clip_norm_scope: str = "global"

    def __post_init__(self):
        if self.clip_norm_scope not in ("global", "tp_local"):
            raise ValueError("clip_norm_scope must be 'global' or 'tp_local'")
        if self.clip_norm_scope == "tp_local" and self.pipeline_parallel_size > 1:
            raise ValueError("clip_norm_scope = 'tp_local' mirrors a reference without pipeline parallelism")
        object.__setattr__(self, "pipeline_layer_split", tuple(int(x) for x in self.pipeline_layer_split))
        if self.fp8 not in ("off", "mxfp8"):
            raise ValueError("fp8 must be 'off' or 'mxfp8'")
        if self.context_parallel_size != 1:
            raise ValueError("context parallelism is not implemented (context_parallel_size must be 1)")
        if self.sequence_parallel and self.tensor_parallel_size == 1:
            object.__setattr__(self, "sequence_parallel", False)

    def data_parallel_size(self, world_size: int) -> int:
        mp = self.tensor_parallel_size * self.pipeline_parallel_size
        if world_size % mp:
            raise ValueError(f"world size {world_size} not divisible by TP*PP={mp}")
        return world_size // mp


@dataclass(frozen=True)
class TrainConfig:
    num_steps: int = 20
    micro_batch_size: int = 2
    global_batch_size: int = 0  # 0 -> micro_batch_size * dp * grad_accum_steps
    grad_accum_steps: int = 1
    seed: int = 0
    deterministic: bool = False
    dtype: str = "bf16"  # "bf16" | "fp32"
    start_step: int = 0
    save_path: str | None = None
    save_interval: int = 0
    resume_from: str | None = None
    init_weights_only: bool = False
    phase_name: str | None = None
    forge_init_ones: bool = True
    # "reference": every full tensor drawn from one CPU generator in the reference's parameter order (bit-identical start
    # for the gates; minutes of host time at 8B).  "device": each shard drawn on its GPU (throughput runs).
    init_mode: str = "reference"
    debug_checks: bool = False       # validate token ids / labels against the vocabulary every micro-batch (also FORGE_DEBUG_CHECKS=1)
    cuda_graph: bool = True
    hash_capture_level: int = 0
    hash_output: str | None = None
    loss_tag: str = "LOSS"
    metrics_jsonl: str | None = None
    recompute: bool = False          # drop the SwiGLU intermediate of every layer and rebuild it in backward
    # Activation recompute of whole layers: the LAST n layers of every model chunk keep only their input and are run again
    # in the backward pass (-1 = every layer); the first layers keep their activations (ref/reference/model_pure_mup_mtp.py:
    # 363-391, --recompute-num-layers).  Trades one extra forward of those layers for their activation memory.
    recompute_num_layers: int = 0


@dataclass(frozen=True)
class DataConfig:
    data_loader: str = "synthetic"  # "synthetic" | "megatron_binary" | "hf" (streaming parquet / JSON-lines packer) | "modelbest"
    data_path: str = ""
    prefetch_size: int = 8
    synthetic_seed: int = 0


@dataclass(frozen=True)
class CkptConfig:
    format: str = "megatron_dist"  # "megatron_dist" | "legacy"
    checkpoint_root: str = ""  # directory holding canonical_state_fp32.pt, if any


@dataclass(frozen=True)
class RunConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    optim: OptimConfig = field(default_factory=OptimConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    train: TrainConfig = field(default_factory=TrainConfig)
    data: DataConfig = field(default_factory=DataConfig)
    ckpt: CkptConfig = field(default_factory=CkptConfig)

    def __post_init__(self):
        # cross-table checks that would otherwise only fail when the model is built on every rank
        split = self.parallel.pipeline_layer_split
        if split:
            chunks = self.parallel.pipeline_parallel_size * max(1, self.parallel.virtual_pipeline_stages)
            if len(split) != chunks or any(int(x) <= 0 for x in split) or sum(int(x) for x in split) != self.model.num_layers:
                raise ValueError(f"pipeline_layer_split {tuple(split)} needs {chunks} positive entries that sum to "
                                 f"num_layers = {self.model.num_layers}")

    def replace(self, **tables: dict[str, Any]) -> "RunConfig":
        """Return a copy with per-table field overrides, e.g. ``replace(train={"num_steps": 3})``."""
        out = {}
        for f in dataclasses.fields(self):
            cur = getattr(self, f.name)
            out[f.name] = dataclasses.replace(cur, **tables[f.name]) if f.name in tables else cur
        return RunConfig(**out)

    def grad_accum(self, dp_size: int) -> int:
        t = self.train
        if t.global_batch_size:
            denom = t.micro_batch_size * dp_size
            if t.global_batch_size % denom:
                raise ValueError("global_batch_size must be a multiple of micro_batch_size * DP")
            return t.global_batch_size // denom
        return t.grad_accum_steps


def _build(cls, table: dict[str, Any], aliases: dict[str, str] | None = None, where: str = ""):
    names = {f.name: f for f in dataclasses.fields(cls)}
    kwargs = {}
    for k, v in table.items():
        k = (aliases or {}).get(k, k)
        if k not in names:
            raise KeyError(f"unknown key {k!r} in [{where}]")
        ftype = names[k].type
        if ftype in ("int", int) and isinstance(v, float) and v == int(v):
            v = int(v)
        if ftype in ("float", float) and isinstance(v, int):
            v = float(v)
        if ftype in ("bool", bool) and isinstance(v, int):
            v = bool(v)
        kwargs[k] = v
    return cls(**kwargs)


_CLI_TO_TABLE = {
    # keys of a rendered gate product's [cli] table (tools/render_gate_configs.py:68-81)
    "num_steps": "train", "micro_batch_size": "train", "global_batch_size": "train",
    "grad_accum_steps": "train", "seed": "train", "deterministic": "train",
    "forge_init_ones": "train", "tensor_parallel_size": "parallel",
}


def from_dict(doc: dict[str, Any]) -> RunConfig:
    doc = {k: dict(v) if isinstance(v, dict) else v for k, v in doc.items()}
    # A gate product keeps the run shape in [cli]; fold the keys we understand.
    cli = doc.pop("cli", None)
    doc.pop("env", None)
    if cli:
        for k, v in cli.items():
            tbl = _CLI_TO_TABLE.get(k)
            if tbl:
                doc.setdefault(tbl, {}).setdefault(k, v)
            elif k in {f.name for f in dataclasses.fields(OptimConfig)}:
                doc.setdefault("optim", {}).setdefault(k, v)
            elif k in {f.name for f in dataclasses.fields(ModelConfig)} or k in _MODEL_ALIASES:
                doc.setdefault("model", {}).setdefault(k, v)
    known = {"model", "optim", "parallel", "train", "data", "ckpt"}
    extra = set(doc) - known
    if extra:
        raise KeyError(f"unknown tables: {sorted(extra)}")
    return RunConfig(
        model=_build(ModelConfig, doc.get("model", {}), _MODEL_ALIASES, "model"),
        optim=_build(OptimConfig, doc.get("optim", {}), None, "optim"),
        parallel=_build(ParallelConfig, doc.get("parallel", {}), None, "parallel"),
        train=_build(TrainConfig, doc.get("train", {}), None, "train"),
        data=_build(DataConfig, doc.get("data", {}), None, "data"),
        ckpt=_build(CkptConfig, doc.get("ckpt", {}), None, "ckpt"),
    )


def load(path: str) -> RunConfig:
    with open(path, "rb") as f:
        return from_dict(tomllib.load(f))


def load_gate_product() -> RunConfig:
    """Resolve ``$FORGE_OURS_CONFIG_DIR/$FORGE_GATE.toml`` as runtime_config.py:84-139 does."""
    d, g = os.environ["FORGE_OURS_CONFIG_DIR"], os.environ["FORGE_GATE"]
    return load(os.path.join(d, f"{g}.toml"))


# ---------------------------------------------------------------------------
# Presets: the five benchmark shapes plus the reference's model axis files.
# ---------------------------------------------------------------------------

def preset(name: str) -> ModelConfig:
    if name == "tiny":
        return ModelConfig(name="tiny", num_layers=2, hidden_size=256, ffn_hidden_size=1024,
                           num_attention_heads=4, num_query_groups=2, head_dim=64, seq_length=256,
                           padded_vocab_size=8192, norm_epsilon=1e-5, init_method_std=0.02,
                           tie_embeddings=True)
    if name == "minicpm4_0.5b":
        return ModelConfig(name=name, num_layers=24, hidden_size=1024, ffn_hidden_size=4096,
                           num_attention_heads=16, num_query_groups=2, head_dim=64, seq_length=4096,
                           padded_vocab_size=73448, norm_epsilon=1e-6, init_method_std=0.1,
                           tie_embeddings=True)
    if name == "minicpm4_8b":
        return ModelConfig(name=name, num_layers=32, hidden_size=4096, ffn_hidden_size=16384,
                           num_attention_heads=32, num_query_groups=2, head_dim=128, seq_length=4096,
                           padded_vocab_size=73448, norm_epsilon=1e-6, init_method_std=0.1)
    if name == "minicpm5_1b":
        return ModelConfig(name=name, num_layers=24, hidden_size=1536, ffn_hidden_size=4608,
                           num_attention_heads=16, num_query_groups=2, head_dim=128, seq_length=4096,
                           padded_vocab_size=130560, norm_epsilon=1e-6, init_method_std=0.02,
                           mtp_num_layers=1, mtp_loss_weight=0.3)
    if name == "qwen3_0.6b":
        return ModelConfig(name=name, num_layers=28, hidden_size=1024, ffn_hidden_size=3072,
                           num_attention_heads=16, num_query_groups=8, head_dim=128, seq_length=4096,
                           padded_vocab_size=151936, rotary_base=1e6, norm_epsilon=1e-6,
                           init_method_std=0.02, tie_embeddings=True, qk_norm=True, use_mup=False)
    raise KeyError(name)
