"""Parameter-name and layout map between this engine and the Hugging Face MiniCPM / Llama-style decoder.

The engine keeps Megatron's fused layouts: ``wqkv`` rows are grouped per KV group (``q_per_kv`` query heads, then the key head,
then the value head), ``wfc1`` is ``[gate; up]``.  The HF modeling code (the ``MiniCPMForCausalLM`` the reference bundles for
its single-card oracle, ref/reference/minicpm4_8b_hf_singlecard/hf_model/modeling_minicpm.py) keeps ``q_proj`` / ``k_proj`` /
``v_proj`` / ``gate_proj`` / ``up_proj`` apart, heads in plain order.  Both directions are exact (row permutations only), so
a state converted there and back is bit-identical.

``python -m forge_train_harness_b200.ckpt.hf_names <checkpoint dir> <out.pt>`` writes an HF-named state dict of a saved run.
"""
from __future__ import annotations

import sys

import torch

from ..config.schema import ModelConfig

_LAYER = {"attention_norm.weight": "input_layernorm.weight", "ffn_norm.weight": "post_attention_layernorm.weight",
          "wo.weight": "self_attn.o_proj.weight", "w2.weight": "mlp.down_proj.weight",
          "q_norm.weight": "self_attn.q_norm.weight", "k_norm.weight": "self_attn.k_norm.weight"}
_TOP = {"tok_embeddings.weight": "model.embed_tokens.weight", "norm.weight": "model.norm.weight", "output.weight": "lm_head.weight"}


def split_qkv(w: torch.Tensor, cfg: ModelConfig):
    """Fused ``[nkv * (g + 2) * d, ...]`` -> (q ``[nkv*g*d, ...]``, k ``[nkv*d, ...]``, v ``[nkv*d, ...]``)."""
    nkv, g, d = cfg.num_query_groups, cfg.q_per_kv, cfg.head_dim
    v = w.reshape(nkv, g + 2, d, *w.shape[1:])
    return (v[:, :g].reshape(nkv * g * d, *w.shape[1:]), v[:, g].reshape(nkv * d, *w.shape[1:]),
            v[:, g + 1].reshape(nkv * d, *w.shape[1:]))


def fuse_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: ModelConfig) -> torch.Tensor:
    nkv, g, d = cfg.num_query_groups, cfg.q_per_kv, cfg.head_dim
    rest = q.shape[1:]
    return torch.cat([q.reshape(nkv, g, d, *rest), k.reshape(nkv, 1, d, *rest), v.reshape(nkv, 1, d, *rest)], 1) \
        .reshape(nkv * (g + 2) * d, *rest)


def engine_to_hf(state: dict, cfg: ModelConfig) -> dict:
    """``{engine FQN: full tensor}`` -> ``{HF name: tensor}`` (main decoder only; the MTP branch has no HF counterpart)."""
    out = {}
    for name, t in state.items():
        if name in _TOP:
            out[_TOP[name]] = t
        elif name.startswith("layers."):
            _, li, rest = name.split(".", 2)
            pre = f"model.layers.{li}."
            if rest == "wqkv.weight":
                q, k, v = split_qkv(t, cfg)
                out[pre + "self_attn.q_proj.weight"], out[pre + "self_attn.k_proj.weight"], out[pre + "self_attn.v_proj.weight"] = q, k, v
            elif rest == "wfc1.weight":
                gate, up = t.chunk(2, 0)
                out[pre + "mlp.gate_proj.weight"], out[pre + "mlp.up_proj.weight"] = gate, up
            elif rest in _LAYER:
                out[pre + _LAYER[rest]] = t
            else:
                raise KeyError(f"no HF name for {name}")
        elif name.startswith("mtp."):
            continue
        else:
            raise KeyError(f"no HF name for {name}")
    if cfg.tie_embeddings and "model.embed_tokens.weight" in out:
        out.setdefault("lm_head.weight", out["model.embed_tokens.weight"])
    return out


def hf_to_engine(state: dict, cfg: ModelConfig) -> dict:
    """``{HF name: tensor}`` -> ``{engine FQN: full tensor}``; every main-decoder parameter of ``cfg`` must be present."""
    inv_top = {v: k for k, v in _TOP.items()}
    inv_layer = {v: k for k, v in _LAYER.items()}
    out = {}
    for li in range(cfg.num_layers):
        pre, mine = f"model.layers.{li}.", f"layers.{li}."
        out[mine + "wqkv.weight"] = fuse_qkv(state[pre + "self_attn.q_proj.weight"], state[pre + "self_attn.k_proj.weight"],
                                             state[pre + "self_attn.v_proj.weight"], cfg)
        out[mine + "wfc1.weight"] = torch.cat([state[pre + "mlp.gate_proj.weight"], state[pre + "mlp.up_proj.weight"]], 0)
        for hf, eng in inv_layer.items():
            if pre + hf in state:
                out[mine + eng] = state[pre + hf]
    for hf, eng in inv_top.items():
        if hf in state and not (eng == "output.weight" and cfg.tie_embeddings):
            out[eng] = state[hf]
    return out


def hf_config_overrides(cfg: ModelConfig) -> dict:
    """Fields of the HF config object that carry this engine's geometry and muP constants."""
    return {"num_hidden_layers": cfg.num_layers, "hidden_size": cfg.hidden_size, "intermediate_size": cfg.ffn_hidden_size,
            "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_query_groups,
            "vocab_size": cfg.padded_vocab_size, "max_position_embeddings": cfg.max_position_embeddings or cfg.seq_length,
            "rms_norm_eps": cfg.norm_epsilon, "rope_theta": cfg.rotary_base, "scale_emb": cfg.mup_emb_scale,
            "scale_depth": cfg.mup_depth_scale, "dim_model_base": cfg.mup_base_hidden_size,
            "tie_word_embeddings": cfg.tie_embeddings, "rope_scaling": None, "use_cache": False}


def main(argv=None) -> int:
    import argparse
    from . import manager
    ap = argparse.ArgumentParser(description="write an HF-named state dict of a saved checkpoint")
    ap.add_argument("checkpoint")
    ap.add_argument("out")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    a = ap.parse_args(argv)
    import json
    import os
    from ..models import params as P
    fmt, concrete = manager._resolve(a.checkpoint)
    if fmt != "megatron_dist":
        raise ValueError("reads the distributed checkpoint format only")
    with open(os.path.join(concrete, "metadata.json")) as f:
        meta = json.load(f)
    cfg = ModelConfig(**meta["model"])
    reader = manager.ShardReader(concrete, meta)
    state = {spec.name: manager.full_param_state(reader, cfg, spec.name, spec, ("master",))["master"]
             for spec in P.full_param_specs(cfg)}
    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    torch.save({k: v.to(dt).contiguous() for k, v in engine_to_hf(state, cfg).items()}, a.out)
    print(f"wrote {a.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
