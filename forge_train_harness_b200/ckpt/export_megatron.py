"""Rewrite a ``megatron_dist`` checkpoint of this engine under Megatron-LM (mcore ``GPTModel``) state-dict names, in
Megatron's legacy per-rank layout ``iter_<N>/mp_rank_<tp>[_<pp>]/model_optim_rng.pt`` at any target TP x PP.

    python -m forge_train_harness_b200.ckpt.export_megatron <checkpoint root or iter dir> <out root> [--tp 2 --pp 1] [--impl te|local]
        [--dtype bf16|fp32]

Name map (this engine's FQNs are the reference's, workload/src/training_engine_tensor/parameters.py:111-143):

    tok_embeddings.weight               embedding.word_embeddings.weight
    layers.<i>.attention_norm.weight    decoder.layers.<j>.self_attention.linear_qkv.layer_norm_weight   (te)
                                        decoder.layers.<j>.input_layernorm.weight                        (local)
    layers.<i>.wqkv.weight              decoder.layers.<j>.self_attention.linear_qkv.weight
    layers.<i>.wo.weight                decoder.layers.<j>.self_attention.linear_proj.weight
    layers.<i>.ffn_norm.weight          decoder.layers.<j>.mlp.linear_fc1.layer_norm_weight              (te)
                                        decoder.layers.<j>.pre_mlp_layernorm.weight                      (local)
    layers.<i>.wfc1.weight              decoder.layers.<j>.mlp.linear_fc1.weight
    layers.<i>.w2.weight                decoder.layers.<j>.mlp.linear_fc2.weight
    norm.weight                         decoder.final_layernorm.weight
    output.weight                       output_layer.weight

``j`` is the layer's index inside its pipeline stage, as Megatron numbers them.  The tensor layouts already agree: the QKV
weight is grouped by KV head (``[n_kv, (g + 2) * d, H]``, Megatron's ``linear_qkv``), FC1 holds the gate rows then the up rows
of the local shard, and TP shards are cut exactly as ``models/params.py::shard_rows`` cuts them (whole KV groups, paired
gate / up rows, row-parallel columns, vocabulary rows).  The weights are the fp32 MASTER values (assembled from the ZeRO-1
shards, whatever layout wrote them), cast to the requested dtype.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys

import torch

from ..config.schema import ModelConfig
from ..models import params as P
from . import manager as M

_LAYER = re.compile(r"^layers\.(\d+)\.(\w+)\.weight$")


def megatron_name(fqn: str, local_index: int | None, impl: str = "te") -> str:
    top = {"tok_embeddings.weight": "embedding.word_embeddings.weight", "norm.weight": "decoder.final_layernorm.weight",
           "output.weight": "output_layer.weight"}
    if fqn in top:
        return top[fqn]
    m = _LAYER.match(fqn)
    if not m:
        raise KeyError(f"no Megatron name for {fqn}")
    j = int(m[1]) if local_index is None else local_index
    sub = {"wqkv": "self_attention.linear_qkv.weight", "wo": "self_attention.linear_proj.weight", "wfc1": "mlp.linear_fc1.weight",
           "w2": "mlp.linear_fc2.weight",
           "attention_norm": "self_attention.linear_qkv.layer_norm_weight" if impl == "te" else "input_layernorm.weight",
           "ffn_norm": "mlp.linear_fc1.layer_norm_weight" if impl == "te" else "pre_mlp_layernorm.weight",
           "q_norm": "self_attention.q_layernorm.weight", "k_norm": "self_attention.k_layernorm.weight"}[m[2]]
    return f"decoder.layers.{j}.{sub}"


def export(src: str, dst_root: str, tp: int = 1, pp: int = 1, impl: str = "te", dtype: str = "bf16") -> str:
    fmt, concrete = M._resolve(src)
    if fmt != "megatron_dist":
        raise ValueError("export reads the distributed format only")
    meta = json.load(open(os.path.join(concrete, "metadata.json")))
    cfg = ModelConfig(**meta["model"])
    if cfg.num_layers % pp:
        raise ValueError("num_layers must be divisible by the target pipeline size")
    if cfg.mtp_num_layers:
        raise ValueError("the MTP branch has no counterpart in this name map")
    per = cfg.num_layers // pp
    reader = M.ShardReader(concrete, meta)
    out_dt = {"bf16": torch.bfloat16, "fp32": torch.float32}[dtype]
    it = int(meta["iteration"])
    out_dir = os.path.join(dst_root, f"iter_{it:07d}")
    states = {(t, p): {} for t in range(tp) for p in range(pp)}
    for spec in P.full_param_specs(cfg):
        full = M.full_param_state(reader, cfg, spec.name, spec, ("master",))["master"]
        if spec.layer == -1:
            stages = [0] + ([pp - 1] if cfg.tie_embeddings and pp > 1 else [])
            local = None
        elif spec.layer == 10 ** 6:
            stages, local = [pp - 1], None
        else:
            stages, local = [spec.layer // per], spec.layer % per
        for t in range(tp):
            dim, idx = P.shard_rows(spec, cfg, tp, t)
            shard = (full if idx is None else full.index_select(dim, idx)).to(out_dt).contiguous()
            for p in stages:
                name = megatron_name(spec.name, local, impl)
                if spec.name == "tok_embeddings.weight" and p == pp - 1 and p != 0:
                    name = "output_layer.weight"          # the tied head's copy on the last stage
                states[(t, p)][name] = shard
    for (t, p), sd in states.items():
        d = os.path.join(out_dir, M._mp_dir(t, p, pp))
        os.makedirs(d, exist_ok=True)
        torch.save({"model": sd, "iteration": it, "checkpoint_version": 3.0,
                    "args": {"tensor_model_parallel_size": tp, "pipeline_model_parallel_size": pp, "num_layers": cfg.num_layers,
                             "hidden_size": cfg.hidden_size, "ffn_hidden_size": cfg.ffn_hidden_size,
                             "num_attention_heads": cfg.num_attention_heads, "num_query_groups": cfg.num_query_groups,
                             "kv_channels": cfg.head_dim, "padded_vocab_size": cfg.padded_vocab_size, "swiglu": True,
                             "group_query_attention": True, "untie_embeddings_and_output_weights": not cfg.tie_embeddings,
                             "normalization": "RMSNorm", "transformer_impl": "transformer_engine" if impl == "te" else "local"}},
                   os.path.join(d, "model_optim_rng.pt"))
    with open(os.path.join(dst_root, M.TRACKER), "w") as f:
        f.write(str(it))
    return out_dir


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--impl", default="te", choices=["te", "local"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    a = ap.parse_args(argv)
    print(export(a.src, a.dst, a.tp, a.pp, a.impl, a.dtype))


if __name__ == "__main__":
    main()
    sys.exit(0)
