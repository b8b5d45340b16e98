"""The reference engine's environment-variable surface, mapped onto this engine's configuration.

The reference engine takes its geometry, hyper-parameters and feature switches from upper-case environment variables (a
rendered gate product's ``[env]`` table exported by ``tools/product_env.py``, or a launcher's ``export`` lines):
geometry ``NUM_LAYERS ... ROTARY_BASE`` (config.py:16-28), ``INIT_METHOD_STD`` / ``MTP_*`` / ``MUP_*`` (train_loop.py:1549-1555),
optimizer ``LR ... CLIP_GRAD`` (1675-1686), and the switches ``DETERMINISTIC`` (1519), ``FORGE_INIT_ONES`` (1543),
``ENABLE_ZERO_OPTIMIZER`` (1726), ``ENABLE_DL_PREFETCH`` / ``DL_PREFETCH_SIZE`` (1790-1792), ``MTP_LOSS_WEIGHT`` (1832),
``ENABLE_CUDA_GRAPH`` (1891), ``ENABLE_TRITON_{RMSNORM,SWIGLU,ROPE}_{FWD,BWD}``, ``ENABLE_TRITON_CE_BWD`` (forward.py:59,135;
backward.py:43,151,233,307,595).  A launch environment written for the reference therefore drives this engine unchanged:

    cfg = apply_reference_env(schema.load("run.toml"), os.environ)     # or: python -m ...train --config run.toml --reference-env

Every variable that is present overrides the file; absent ones leave it alone.  The reference's per-kernel Triton switches map
onto this engine's op router: ``ENABLE_TRITON_RMSNORM_FWD=0`` selects the plain-PyTorch version of that op
(``OP_RMSNORM_FWD=baseline``), ``=1`` the hand-written one.  Variables that have no meaning here (NCCL tuning of the
reference's collectives, ``CUDA_DEVICE_MAX_CONNECTIONS``) are left to the process environment as they are.
"""
from __future__ import annotations

from typing import Any, Mapping

from .schema import RunConfig

_MODEL_INT = {"NUM_LAYERS": "num_layers", "HIDDEN_SIZE": "hidden_size", "FFN_HIDDEN_SIZE": "ffn_hidden_size",
              "NUM_ATTENTION_HEADS": "num_attention_heads", "NUM_QUERY_GROUPS": "num_query_groups", "HEAD_DIM": "head_dim",
              "SEQ_LENGTH": "seq_length", "MAX_POSITION_EMBEDDINGS": "max_position_embeddings", "PADDED_VOCAB_SIZE": "padded_vocab_size",
              "MTP_NUM_LAYERS": "mtp_num_layers", "MUP_BASE_HIDDEN_SIZE": "mup_base_hidden_size"}
_MODEL_FLOAT = {"NORM_EPSILON": "norm_epsilon", "ROTARY_BASE": "rotary_base", "INIT_METHOD_STD": "init_method_std",
                "MUP_EMB_SCALE": "mup_emb_scale", "MUP_DEPTH_SCALE": "mup_depth_scale", "MTP_LOSS_WEIGHT": "mtp_loss_weight"}
_OPTIM_FLOAT = {"LR": "lr", "MIN_LR": "min_lr", "WEIGHT_DECAY": "weight_decay", "ADAM_BETA1": "adam_beta1", "ADAM_BETA2": "adam_beta2",
                "CLIP_GRAD": "clip_grad"}
_OPTIM_INT = {"LR_WARMUP_ITERS": "lr_warmup_iters", "LR_DECAY_ITERS": "lr_decay_iters", "LR_WSD_DECAY_ITERS": "lr_wsd_decay_iters"}
_TRAIN_INT = {"MICRO_BATCH_SIZE": "micro_batch_size", "GLOBAL_BATCH_SIZE": "global_batch_size", "NUM_STEPS": "num_steps", "SEED": "seed"}
_TRITON_TO_OP = {"ENABLE_TRITON_RMSNORM_FWD": ("OP_RMSNORM_FWD", "OP_RESIDUAL_RMSNORM_FWD"), "ENABLE_TRITON_RMSNORM_BWD": ("OP_RMSNORM_BWD",),
                 "ENABLE_TRITON_SWIGLU_FWD": ("OP_SWIGLU_FWD",), "ENABLE_TRITON_SWIGLU_BWD": ("OP_SWIGLU_BWD",),
                 "ENABLE_TRITON_ROPE_FWD": ("OP_ROPE_FWD",), "ENABLE_TRITON_ROPE_BWD": ("OP_ROPE_BWD",),
                 "ENABLE_TRITON_CE_BWD": ("OP_CROSS_ENTROPY_FWD_BWD",)}


def _flag(v: str) -> bool:
    return str(v).strip().lower() in ("1", "true", "yes", "on")


def apply_reference_env(cfg: RunConfig, env: Mapping[str, str]) -> RunConfig:
    """``cfg`` with every reference variable present in ``env`` applied.  A value that does not parse raises ``ValueError``
    naming the variable (the reference fails fast on a missing or malformed key, config.py:16-28)."""
    tables: dict[str, dict[str, Any]] = {}

    def put(table: str, field: str, var: str, conv):
        if var in env and str(env[var]).strip() != "":
            try:
                tables.setdefault(table, {})[field] = conv(env[var])
            except (TypeError, ValueError) as e:
                raise ValueError(f"environment variable {var}={env[var]!r} does not parse: {e}") from e

    for var, f in _MODEL_INT.items():
        put("model", f, var, lambda v: int(float(v)))
    for var, f in _MODEL_FLOAT.items():
        put("model", f, var, float)
    for var, f in _OPTIM_FLOAT.items():
        put("optim", f, var, float)
    for var, f in _OPTIM_INT.items():
        put("optim", f, var, lambda v: int(float(v)))
    for var, f in _TRAIN_INT.items():
        put("train", f, var, lambda v: int(float(v)))
    put("train", "deterministic", "DETERMINISTIC", _flag)
    put("train", "forge_init_ones", "FORGE_INIT_ONES", _flag)
    put("train", "cuda_graph", "ENABLE_CUDA_GRAPH", _flag)
    put("parallel", "use_distributed_optimizer", "ENABLE_ZERO_OPTIMIZER", _flag)
    put("data", "prefetch_size", "DL_PREFETCH_SIZE", lambda v: int(float(v)))
    if "ENABLE_DL_PREFETCH" in env and not _flag(env["ENABLE_DL_PREFETCH"]):
        tables.setdefault("data", {})["prefetch_size"] = 0
    if tables.get("model", {}).get("mtp_num_layers") == 0:
        tables["model"].setdefault("mtp_loss_weight", 0.0)
    return cfg.replace(**tables) if tables else cfg


def op_env_from_reference(env: Mapping[str, str]) -> dict[str, str]:
    """``OP_<NAME>`` selectors implied by the reference's ``ENABLE_TRITON_*`` switches that are present in ``env``."""
    out = {}
    for var, ops in _TRITON_TO_OP.items():
        if var in env and str(env[var]).strip() != "":
            for op in ops:
                out[op] = "sm100" if _flag(env[var]) else "baseline"
    return out
