"""Reference-side capture bridge: run ONE micro-batch through the reference's own model (``MiniCPM4MupMtp`` of
ref/reference/model_pure_mup_mtp.py, imported unmodified from ``baseline/_ref``) with forward and full-backward hooks on its
modules, and save every captured tensor under the key families the alignment gates use:

    fwd.<fqn>    module output            (tok_embeddings, layers.<i>.{attention_norm, wqkv, wo, ffn_norm, wfc1, w2}, norm, output)
    bwd.<fqn>    gradient w.r.t. that output
    grad.<fqn>   fp32 parameter gradient  (the reference's ``main_grad``)
    loss.per_token / loss.sum

The reference installs such hooks from its own harness (evals/harness_hook/__init__.py:195-337, _module_hook.py:127-254) and
compares blake2b digests, which only a bit-identical engine can match.  An engine with its own GEMM and attention kernels is
held to a tolerance instead, so this bridge keeps the TENSORS; ``gates.verdicts.align_tolerance`` compares them key by key.
The loss is the plain sum of the per-token negative log-likelihoods, the same convention as this engine's backward pass.

    python baseline/ref_capture_bridge.py --model tiny --layers 2 --canonical <dir>/canonical_state_fp32.pt --out ref_capture.pt
"""
from __future__ import annotations

import argparse
import dataclasses
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--set", action="append", default=[], help="model override key=value (ints / floats)")
    ap.add_argument("--canonical", required=True)
    ap.add_argument("--mbs", type=int, default=2)
    ap.add_argument("--data-seed", type=int, default=0)
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    sys.path.insert(0, os.path.dirname(HERE))
    from forge_train_harness_b200.config.schema import preset         # shape constants
    from forge_train_harness_b200.data.sources import SyntheticTokens  # the input batch both sides read
    m = preset(a.model)
    over = {}
    for kv in a.set:
        k, v = kv.split("=", 1)
        cur = getattr(m, k)
        over[k] = type(cur)(v) if not isinstance(cur, bool) else v.lower() in ("1", "true")
    m = dataclasses.replace(m, tie_embeddings=False, mtp_num_layers=0, **over)
    os.environ.update({"NUM_LAYERS": str(m.num_layers), "HIDDEN_SIZE": str(m.hidden_size),
                       "NUM_ATTENTION_HEADS": str(m.num_attention_heads), "NUM_QUERY_GROUPS": str(m.num_query_groups),
                       "HEAD_DIM": str(m.head_dim), "FFN_HIDDEN_SIZE": str(m.ffn_hidden_size),
                       "PADDED_VOCAB_SIZE": str(m.padded_vocab_size), "MAX_POSITION_EMBEDDINGS": str(m.seq_length),
                       "NORM_EPSILON": str(m.norm_epsilon), "ROTARY_BASE": str(int(m.rotary_base))})
    sys.path.insert(0, REF)
    sys.path.insert(1, os.path.join(REF, "ref", "reference"))
    import torch
    import model_pure_mup_mtp as R
    dev = "cuda"
    model = R.MiniCPM4MupMtp(vocab_size=m.padded_vocab_size, mup_base_hidden_size=m.mup_base_hidden_size,
                             mup_emb_scale=m.mup_emb_scale, mup_depth_scale=m.mup_depth_scale, eagle_num_layers=0)
    state = torch.load(a.canonical, map_location="cpu", weights_only=True)
    missing = [n for n, _ in model.named_parameters() if n not in state]
    if missing:
        raise SystemExit(f"canonical state lacks {missing[:5]}")
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.copy_(state[n])
    model = model.to(device=dev, dtype=torch.bfloat16)
    rope = R.precompute_rope_freqs(m.seq_length, device=dev)

    rec: dict = {}
    want = {"tok_embeddings", "norm", "output"}
    for i in range(m.num_layers):
        want |= {f"layers.{i}.{s}" for s in ("attention_norm", "wqkv", "wo", "ffn_norm", "wfc1", "w2")}
    for name, mod in model.named_modules():
        if name not in want:
            continue
        mod.register_forward_hook(lambda _m, _i, out, name=name: rec.__setitem__(f"fwd.{name}", out.detach().reshape(-1, out.shape[-1]).cpu()))
        mod.register_full_backward_hook(
            lambda _m, _gi, go, name=name: rec.__setitem__(f"bwd.{name}", go[0].detach().reshape(-1, go[0].shape[-1]).cpu()))

    b = next(SyntheticTokens(m.padded_vocab_size, m.seq_length, a.mbs, 0, 1, a.data_seed))
    ids, labels = b["tokens"].to(dev), b["labels"].to(dev)
    logits, _ = model(ids, rope)
    nll = torch.nn.functional.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), labels.reshape(-1), reduction="none")
    rec["loss.per_token"] = nll.detach().cpu()
    rec["loss.sum"] = nll.detach().double().sum().cpu()
    nll.sum().backward()
    for n, p in model.named_parameters():
        g = getattr(p, "main_grad", None)
        if g is None:
            g = p.grad
        if g is not None:
            rec[f"grad.{n}"] = g.detach().float().cpu()
    torch.save(rec, a.out)
    print(f"captured {len(rec)} tensors -> {a.out}")


if __name__ == "__main__":
    main()
    sys.exit(0)
