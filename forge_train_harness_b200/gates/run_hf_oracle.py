"""Loss-trend cross-check of the 8B shape against the Hugging Face single-card oracle.

The reference keeps a second, framework-native oracle beside its hand-written 8B trainer (ref/reference/
train_minicpm4_8b_hf_singlecard.py): the official modeling code trained on one card, compared by loss TREND, not bitwise.
This runner is that check for this engine: (1) write a learnable synthetic ``.bin/.idx`` corpus; (2) run the oracle
(``baseline/hf_oracle.py``) as a child process, which also writes its initial weights under this engine's parameter names;
(3) run this engine from those weights on the same corpus with the same hyper-parameters through its public entry point;
(4) verdict from the two logs alone: first-step loss within ``--first-tol`` and mean relative loss difference over the window
below ``--threshold``.

    python -m forge_train_harness_b200.gates.run_hf_oracle --layers 4 --steps 50 --window 21 51 --out hf_oracle_out \
        [--device cuda:0] [--dtype bf16] [--hidden 256 --seq 64 --vocab 512]   # the bracketed shrink is for CPU tests
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import subprocess
import sys

import numpy as np

from ..config.schema import preset
from ..data.sources import write_megatron_binary
from ..utils import wire
from . import verdicts as V

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="minicpm4_8b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=0)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--vocab", type=int, default=0)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--window", type=int, nargs=2, default=[21, 51])
    ap.add_argument("--mbs", type=int, default=1)
    ap.add_argument("--accum", type=int, default=8)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--threshold", type=float, default=0.02)
    ap.add_argument("--first-tol", type=float, default=5e-3)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--out", default="hf_oracle_out")
    ap.add_argument("--timeout", type=float, default=1800.0)
    a = ap.parse_args(argv)
    out = os.path.abspath(a.out)
    os.makedirs(out, exist_ok=True)
    m = dataclasses.replace(preset(a.model), num_layers=a.layers, mtp_num_layers=0, mtp_loss_weight=0.0, tie_embeddings=False)
    if a.hidden:
        heads = max(2, a.hidden // m.head_dim)
        m = dataclasses.replace(m, hidden_size=heads * m.head_dim, num_attention_heads=heads, num_query_groups=2, ffn_hidden_size=2 * a.hidden)
    if a.seq:
        m = dataclasses.replace(m, seq_length=a.seq, max_position_embeddings=a.seq)
    if a.vocab:
        m = dataclasses.replace(m, padded_vocab_size=a.vocab)
    gbs = a.mbs * a.accum
    # learnable corpus: a fixed random successor map over a sub-vocabulary, followed 90 % of the time
    rng = np.random.RandomState(0)
    sub = min(4096, m.padded_vocab_size)
    succ = rng.permutation(sub)
    docs = []
    for _ in range((a.steps * gbs + 64 + 63) // 64):
        n = (m.seq_length + 1) * 64
        jump, rnd = rng.rand(n) < 0.1, rng.randint(0, sub, size=n)
        d = np.empty(n, dtype=np.int32)
        d[0] = rnd[0]
        for i in range(1, n):
            d[i] = rnd[i] if jump[i] else succ[d[i - 1]]
        docs.append(d)
    prefix = os.path.join(out, "corpus")
    write_megatron_binary(prefix, docs, np.int32)
    canon = os.path.join(out, "canonical")
    shrink = (["--hidden", str(a.hidden)] if a.hidden else []) + (["--seq", str(a.seq)] if a.seq else []) + \
             (["--vocab", str(a.vocab)] if a.vocab else [])
    ref_cmd = [sys.executable, os.path.join(ROOT, "baseline", "hf_oracle.py"), "--model", a.model, "--layers", str(a.layers),
               "--steps", str(a.steps), "--mbs", str(a.mbs), "--accum", str(a.accum), "--lr", str(a.lr), "--min-lr", str(a.lr * 0.1),
               "--warmup", str(a.warmup), "--decay-iters", "100000", "--data-prefix", prefix, "--ckpt-root", canon,
               "--device", a.device, "--dtype", a.dtype] + shrink
    r = subprocess.run(ref_cmd, cwd=out, capture_output=True, text=True, timeout=a.timeout)
    open(os.path.join(out, "ref.log"), "w").write(r.stdout + "\n--- stderr ---\n" + r.stderr[-20000:])
    if r.returncode == 3:
        res = {"passed": False, "unavailable": r.stderr.strip().splitlines()[-1] if r.stderr.strip() else "oracle unavailable"}
        print(json.dumps(res), flush=True)
        return 3
    ref_recs = wire.parse_loss_lines(r.stdout, strict=False)
    cfg_path = os.path.join(out, "ours.toml")
    with open(cfg_path, "w") as f:
        f.write("[model]\n" + "".join(f"{k} = {json.dumps(v)}\n" for k, v in dataclasses.asdict(m).items()))
        f.write(f"\n[optim]\nlr = {a.lr}\nmin_lr = {a.lr * 0.1}\nlr_warmup_iters = {a.warmup}\nlr_decay_iters = 100000\n"
                "lr_schedule = \"cosine\"\nweight_decay = 0.1\nadam_beta1 = 0.9\nadam_beta2 = 0.95\nclip_grad = 1.0\n")
        f.write(f"\n[train]\nnum_steps = {a.steps}\nmicro_batch_size = {a.mbs}\nglobal_batch_size = {gbs}\nseed = 1234\n"
                f"dtype = {json.dumps(a.dtype)}\n" + ("cuda_graph = false\n" if a.device == "cpu" else ""))
        f.write(f"\n[data]\ndata_loader = \"megatron_binary\"\ndata_path = {json.dumps(prefix)}\n")
        f.write(f"\n[ckpt]\ncheckpoint_root = {json.dumps(canon)}\n")
    env = dict(os.environ)
    if a.device == "cpu":
        env["CUDA_VISIBLE_DEVICES"] = ""
    o = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.train", "--config", cfg_path], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=a.timeout)
    open(os.path.join(out, "ours.log"), "w").write(o.stdout + "\n--- stderr ---\n" + o.stderr[-20000:])
    our_recs = wire.parse_loss_lines(o.stdout, strict=False)
    res = {"model": m.name, "layers": m.num_layers, "hidden": m.hidden_size, "global_batch": gbs, "steps": a.steps, "ref_rc": r.returncode,
           "ours_rc": o.returncode, "ref_steps": len(ref_recs), "ours_steps": len(our_recs)}
    if ref_recs and our_recs:
        res["first_step"] = {"ref": ref_recs[0].loss, "ours": our_recs[0].loss,
                             "rel_diff": abs(ref_recs[0].loss - our_recs[0].loss) / abs(ref_recs[0].loss)}
        res["grad_norm_first"] = {"ref": ref_recs[0].grad_norm, "ours": our_recs[0].grad_norm}
        res["trend"] = V.long_train(ref_recs, our_recs, tuple(a.window), a.threshold)
        res["passed"] = bool(res["trend"].get("passed")) and res["first_step"]["rel_diff"] < a.first_tol
    else:
        res["passed"] = False
    with open(os.path.join(out, "hf_oracle.json"), "w") as f:
        json.dump(res, f, indent=1)
    print(json.dumps(res), flush=True)
    return 0 if res["passed"] else 1


if __name__ == "__main__":
    sys.exit(main())
