"""Start this engine from weights written by other stacks: Megatron-LM's legacy per-rank checkpoints, or a Hugging Face state
dict.  Both are rewritten as ``canonical_state_fp32.pt`` (``{engine FQN: full fp32 tensor}``), the hand-off file the engine
loads at start-up when ``[ckpt].checkpoint_root`` names its directory (``Trainer._init_weights``; the reference's own
hand-off file, workload/src/training_engine_tensor/parameters.py:146-190).

    python -m forge_train_harness_b200.ckpt.import_weights megatron <root or iter dir> --model minicpm4_0.5b --out <ckpt_root> [--impl te|local]
    python -m forge_train_harness_b200.ckpt.import_weights hf <state.pt> --model minicpm4_8b --out <ckpt_root> [--layers N]

Megatron side: ``iter_<N>/mp_rank_<tp>[_<pp>]/model_optim_rng.pt`` at any TP x PP (the layout ``ckpt/export_megatron.py`` writes
and Megatron-LM's ``--ckpt-format torch`` uses, ref/reference/train_minicpm4_0.5b_gsm8k.sh:307-320).  Tensor-parallel shards
are merged by the inverse of ``models/params.py::shard_rows`` (whole KV groups of the QKV weight, paired gate / up rows of
FC1, columns of the row-parallel weights, vocabulary rows), pipeline stages by their local layer index.  HF side: the name /
layout map of ``ckpt/hf_names.py``.  Every parameter of the target model must be found, with the right shape.
"""
from __future__ import annotations

import argparse
import dataclasses
import os
import re
import sys

import torch

from ..config.schema import ModelConfig, preset
from ..models import params as P
from . import hf_names
from .export_megatron import megatron_name

_MP = re.compile(r"^mp_rank_(\d+)(?:_(\d+))?$")


def _iter_dir(path: str) -> str:
    if os.path.isdir(path) and any(_MP.match(d) for d in os.listdir(path)):
        return path
    tracker = os.path.join(path, "latest_checkpointed_iteration.txt")
    if os.path.isfile(tracker):
        it = open(tracker).read().strip()
        cand = os.path.join(path, "release" if it == "release" else f"iter_{int(it):07d}")
        if os.path.isdir(cand):
            return cand
    its = sorted(d for d in os.listdir(path) if d.startswith("iter_"))
    if not its:
        raise FileNotFoundError(f"no mp_rank_* directories or iter_* checkpoints under {path}")
    return os.path.join(path, its[-1])


def from_megatron(path: str, cfg: ModelConfig, impl: str = "te") -> dict:
    """``{engine FQN: full fp32 tensor}`` from a legacy-layout Megatron checkpoint."""
    d = _iter_dir(path)
    shards: dict[tuple[int, int], dict] = {}
    for name in sorted(os.listdir(d)):
        m = _MP.match(name)
        if m:
            sd = torch.load(os.path.join(d, name, "model_optim_rng.pt"), map_location="cpu", weights_only=False)
            shards[(int(m[1]), int(m[2] or 0))] = sd["model"] if "model" in sd else sd
    if not shards:
        raise FileNotFoundError(f"no mp_rank_* directories in {d}")
    tp = max(t for t, _ in shards) + 1
    pp = max(p for _, p in shards) + 1
    if cfg.num_layers % pp:
        raise ValueError(f"{cfg.num_layers} layers do not divide over the checkpoint's {pp} pipeline stages")
    per = cfg.num_layers // pp
    out = {}
    for spec in P.full_param_specs(cfg):
        if spec.name.startswith("mtp."):
            raise ValueError("the MTP branch has no counterpart in the Megatron name map")
        if spec.layer == -1:
            stage, local = 0, None
        elif spec.layer == 10 ** 6:
            stage, local = pp - 1, None
        else:
            stage, local = spec.layer // per, spec.layer % per
        key = megatron_name(spec.name, local, impl)
        full = torch.zeros(spec.full_shape, dtype=torch.float32)
        for t in range(tp):
            sd = shards.get((t, stage))
            if sd is None or key not in sd:
                raise KeyError(f"{key} (for {spec.name}) not found in mp_rank_{t:02d}" + (f"_{stage:03d}" if pp > 1 else ""))
            dim, idx = P.shard_rows(spec, cfg, tp, t)
            piece = sd[key].float()
            if idx is None:
                if tuple(piece.shape) != tuple(spec.full_shape):
                    raise ValueError(f"{key}: shape {tuple(piece.shape)}, model wants {tuple(spec.full_shape)}")
                full.copy_(piece)
            else:
                if piece.shape[dim] != idx.numel():
                    raise ValueError(f"{key}: shard has {piece.shape[dim]} entries along dim {dim}, TP {tp} of this model has {idx.numel()}")
                full.index_copy_(dim, idx, piece)
        out[spec.name] = full
    return out


def from_hf(state: dict, cfg: ModelConfig) -> dict:
    eng = {k: v.float() for k, v in hf_names.hf_to_engine(state, cfg).items()}
    want = {s.name: s for s in P.full_param_specs(cfg) if not s.name.startswith("mtp.")}
    missing = sorted(set(want) - set(eng))
    if missing:
        raise KeyError(f"the HF state lacks: {missing[:6]}{' ...' if len(missing) > 6 else ''}")
    for name, spec in want.items():
        if tuple(eng[name].shape) != tuple(spec.full_shape):
            raise ValueError(f"{name}: shape {tuple(eng[name].shape)}, model wants {tuple(spec.full_shape)}")
    return {k: eng[k].contiguous() for k in want}


def write_canonical(state: dict, out_root: str) -> str:
    os.makedirs(out_root, exist_ok=True)
    path = os.path.join(out_root, "canonical_state_fp32.pt")
    torch.save(state, path + ".tmp")
    os.replace(path + ".tmp", path)
    return path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["megatron", "hf"])
    ap.add_argument("src")
    ap.add_argument("--model", required=True, help="a preset name (the checkpoint's model shape)")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--out", required=True)
    ap.add_argument("--impl", default="te", choices=["te", "local"])
    ap.add_argument("--untied", action="store_true", help="the checkpoint has a separate output layer")
    a = ap.parse_args(argv)
    cfg = preset(a.model)
    if a.layers:
        cfg = dataclasses.replace(cfg, num_layers=a.layers)
    cfg = dataclasses.replace(cfg, mtp_num_layers=0, mtp_loss_weight=0.0, tie_embeddings=cfg.tie_embeddings and not a.untied)
    if a.kind == "megatron":
        state = from_megatron(a.src, cfg, a.impl)
    else:
        state = from_hf(torch.load(a.src, map_location="cpu", weights_only=True), cfg)
    print(write_canonical(state, a.out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
