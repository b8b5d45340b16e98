"""Parameter inventory, tensor-parallel sharding rules and initialisation.

Parameters are bare tensors that are views into flat buffers (no ``nn.Module``), named
with the reference's FQNs (workload/src/training_engine_tensor/parameters.py:111-143):
``tok_embeddings.weight``, ``layers.<i>.{attention_norm,wqkv,wo,ffn_norm,wfc1,w2}.weight``,
``norm.weight``, ``output.weight`` and ``mtp.*``.

Sharding rules follow the hand-written TP reference (ref/reference/model_minicpm4_8b_tp.py:239-347):
QKV is column-split by whole KV groups, FC1 column-split with gate and up halves kept
paired, out-proj / FC2 row-split, embedding and LM head vocabulary-split.  Beyond that
reference (which asserts ``NUM_KV_HEADS % tp == 0`` at :444), a TP degree larger than the
number of KV heads is supported by replicating each KV head over ``tp / n_kv`` ranks; the
replicated rows' gradients are summed over those ranks before the optimizer step.

Initialisation draws every FULL logical tensor from one seeded CPU generator in the
reference's parameter order and then slices the local shard, so any (TP, PP) layout starts
from the same weights (model_minicpm4_8b_tp.py:552-601; std rules model_pure_mup_mtp.py:436-477).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..config.schema import ModelConfig


@dataclass(frozen=True)
class ParamSpec:
    name: str
    full_shape: tuple[int, ...]
    kind: str  # "replicated" | "qkv" | "col_pair" | "row" | "vocab"
    is_matrix: bool  # muP matrix weight: lr / width_mult
    init: str  # "norm" | "std" | "scaled_std"
    layer: int  # global layer index, -1 for embedding, 10**6 for head side

    @property
    def weight_decay(self) -> bool:
        return len(self.full_shape) >= 2


def is_head_partial(spec: ParamSpec) -> bool:
    """Replicated weights applied per attention head (the q / k norms of the Qwen3 variant): under tensor parallelism a
    rank sees only its own heads, so its gradient is a partial sum that must be added over the TP group."""
    return spec.kind == "replicated" and spec.name.endswith(("q_norm.weight", "k_norm.weight"))


def full_param_specs(cfg: ModelConfig) -> list[ParamSpec]:
    """Every logical parameter in the reference's ``named_parameters`` order."""
    H, F, V = cfg.hidden_size, cfg.ffn_hidden_size, cfg.padded_vocab_size
    out = [ParamSpec("tok_embeddings.weight", (V, H), "vocab", False, "std", -1)]

    def layer(prefix: str, li: int):
        ps = [ParamSpec(f"{prefix}attention_norm.weight", (H,), "replicated", False, "norm", li),
              ParamSpec(f"{prefix}wqkv.weight", (cfg.qkv_dim, H), "qkv", True, "scaled_std", li)]
        if cfg.qk_norm:
            ps += [ParamSpec(f"{prefix}q_norm.weight", (cfg.head_dim,), "replicated", False, "norm", li),
                   ParamSpec(f"{prefix}k_norm.weight", (cfg.head_dim,), "replicated", False, "norm", li)]
        ps += [ParamSpec(f"{prefix}wo.weight", (H, cfg.q_dim), "row", True, "scaled_std", li),
               ParamSpec(f"{prefix}ffn_norm.weight", (H,), "replicated", False, "norm", li),
               ParamSpec(f"{prefix}wfc1.weight", (2 * F, H), "col_pair", True, "scaled_std", li),
               ParamSpec(f"{prefix}w2.weight", (H, F), "row", True, "scaled_std", li)]
        return ps

    for li in range(cfg.num_layers):
        out += layer(f"layers.{li}.", li)
    big = 10 ** 6
    out.append(ParamSpec("norm.weight", (H,), "replicated", False, "norm", big))
    if not cfg.tie_embeddings:
        out.append(ParamSpec("output.weight", (V, H), "vocab", False, "std", big))
    if cfg.mtp_num_layers:
        out += [ParamSpec("mtp.emb_input_layernorm.weight", (H,), "replicated", False, "norm", big),
                ParamSpec("mtp.hidden_input_layernorm.weight", (H,), "replicated", False, "norm", big),
                ParamSpec("mtp.eagle_fc.weight", (H, 2 * H), "replicated", True, "scaled_std", big)]
        out += [ParamSpec(p.name, p.full_shape, p.kind, p.is_matrix, p.init, big) for p in layer("mtp.layer.", big)]
        out.append(ParamSpec("mtp.final_layernorm.weight", (H,), "replicated", False, "norm", big))
    return out


# ---------------------------------------------------------------------------
# Tensor-parallel geometry
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class TPGeometry:
    """Local attention / MLP / vocabulary extents of one TP rank."""
    tp: int
    rank: int
    n_kv_local: int  # KV heads held by this rank (each possibly a replica)
    g_local: int  # query heads per local KV head
    kv_replicas: int  # ranks sharing one KV head (1 = no replication)
    head_dim: int
    ffn_local: int
    vocab_start: int
    vocab_local: int

    @property
    def q_dim_local(self) -> int:
        return self.n_kv_local * self.g_local * self.head_dim

    @property
    def qkv_dim_local(self) -> int:
        return self.n_kv_local * (self.g_local + 2) * self.head_dim


def tp_geometry(cfg: ModelConfig, tp: int, rank: int) -> TPGeometry:
    nkv, g = cfg.num_query_groups, cfg.q_per_kv
    if tp <= nkv:
        if nkv % tp:
            raise ValueError("num_query_groups must be divisible by TP when TP <= num_query_groups")
        n_kv_local, g_local, rep = nkv // tp, g, 1
    else:
        if tp % nkv or g % (tp // nkv):
            raise ValueError("TP must be a multiple of num_query_groups and divide the query heads evenly")
        rep = tp // nkv
        n_kv_local, g_local = 1, g // rep
    if cfg.ffn_hidden_size % tp:
        raise ValueError("ffn_hidden_size must be divisible by TP")
    V = cfg.padded_vocab_size
    per = (V + tp - 1) // tp
    vs = min(rank * per, V)
    return TPGeometry(tp, rank, n_kv_local, g_local, rep, cfg.head_dim, cfg.ffn_hidden_size // tp,
                      vs, min(per, V - vs))


def shard_rows(spec: ParamSpec, cfg: ModelConfig, tp: int, rank: int) -> tuple[int, torch.Tensor | None]:
    """``(dim, index)``: which indices of ``dim`` of the full tensor this rank holds (None = all)."""
    if tp == 1 or spec.kind == "replicated":
        return 0, None
    geo = tp_geometry(cfg, tp, rank)
    d, g = cfg.head_dim, cfg.q_per_kv
    if spec.kind == "qkv":
        idx = []
        for j in range(geo.n_kv_local):
            if geo.kv_replicas == 1:
                kvh, q0 = rank * geo.n_kv_local + j, 0
            else:
                kvh, q0 = rank // geo.kv_replicas, (rank % geo.kv_replicas) * geo.g_local
            base = kvh * (g + 2) * d
            idx.append(torch.arange(base + q0 * d, base + (q0 + geo.g_local) * d))
            idx.append(torch.arange(base + g * d, base + (g + 2) * d))
        return 0, torch.cat(idx)
    if spec.kind == "row":
        n = spec.full_shape[1]
        if n == cfg.q_dim:  # out-proj: columns follow the local query heads
            per = geo.q_dim_local
        else:
            per = n // tp
        return 1, torch.arange(rank * per, (rank + 1) * per)
    if spec.kind == "col_pair":
        F = spec.full_shape[0] // 2
        per = F // tp
        a = torch.arange(rank * per, (rank + 1) * per)
        return 0, torch.cat([a, a + F])
    if spec.kind == "vocab":
        return 0, torch.arange(geo.vocab_start, geo.vocab_start + geo.vocab_local)
    raise ValueError(spec.kind)


def local_shape(spec: ParamSpec, cfg: ModelConfig, tp: int, rank: int) -> tuple[int, ...]:
    dim, idx = shard_rows(spec, cfg, tp, rank)
    if idx is None:
        return spec.full_shape
    s = list(spec.full_shape)
    s[dim] = idx.numel()
    return tuple(s)


def kv_replicated_rows(cfg: ModelConfig, tp: int, rank: int) -> torch.Tensor | None:
    """Local row indices of ``wqkv`` that are replicas shared with other TP ranks (k and v rows)."""
    geo = tp_geometry(cfg, tp, rank)
    if geo.kv_replicas == 1:
        return None
    d = cfg.head_dim
    return torch.arange(geo.g_local * d, (geo.g_local + 2) * d)


# ---------------------------------------------------------------------------
# Initialisation
# ---------------------------------------------------------------------------

def init_std(spec: ParamSpec, cfg: ModelConfig) -> float:
    if spec.init == "std":
        return cfg.init_method_std
    return cfg.init_method_std / math.sqrt(cfg.width_mult)


def iter_full_init(cfg: ModelConfig, seed: int, init_ones: bool = True, wanted: set[str] | None = None):
    """Yield ``(spec, full fp32 tensor)`` in reference order from ONE generator.

    Tensors not in ``wanted`` are still drawn (to keep the stream position) but yielded as None."""
    gen = torch.Generator().manual_seed(seed)
    for spec in full_param_specs(cfg):
        if spec.init == "norm":
            t = torch.full(spec.full_shape, 1.0 if init_ones else 0.97, dtype=torch.float32)
        elif spec.kind == "qkv" and cfg.qk_norm and not cfg.use_mup:
            # the Qwen3 reference keeps q / k / v as three matrices and draws them one after the other, heads in plain order
            # (model_qwen3.py:112-115, 232-249); same draws here, then interleaved per KV group into the fused layout
            nkv, g, d, H = cfg.num_query_groups, cfg.q_per_kv, cfg.head_dim, spec.full_shape[1]
            q, k, v = (torch.randn((rows, H), generator=gen, dtype=torch.float32).mul_(init_std(spec, cfg))
                       for rows in (nkv * g * d, nkv * d, nkv * d))
            t = torch.cat([q.view(nkv, g, d, H), k.view(nkv, 1, d, H), v.view(nkv, 1, d, H)], 1).reshape(spec.full_shape)
        else:
            t = torch.randn(spec.full_shape, generator=gen, dtype=torch.float32).mul_(init_std(spec, cfg))
        yield spec, (t if wanted is None or spec.name in wanted else None)


def device_init_(tensor: torch.Tensor, spec: ParamSpec, cfg: ModelConfig, seed: int, index: int,
                 init_ones: bool = True) -> None:
    """Fast per-parameter init on the tensor's own device (benchmarks; not layout-invariant)."""
    if spec.init == "norm":
        tensor.fill_(1.0 if init_ones else 0.97)
        return
    gen = torch.Generator(device=tensor.device).manual_seed(seed * 100003 + index)
    tensor.normal_(0.0, init_std(spec, cfg), generator=gen)
