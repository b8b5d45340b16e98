"""Alignment gate against a LIVE run of the reference: same init, same data, same hyper-parameters, compare ``[LOSS]`` lines.

    python -m forge_train_harness_b200.gates.run_alignment --model minicpm4_0.5b --steps 60 --window 21 61 \
        [--nproc 1] [--mbs 4] [--accum 2] [--layers 24] [--out gates_out] [--ref l0|engine]

``--ref engine`` puts the reference's produced ENGINE (``training_engine_tensor.run_training_loop``, through
``baseline/ref_engine_driver.py``) on the reference side instead of its L0 trainer; both sides then start from one
``canonical_state_fp32.pt`` written here (the reference's own hand-off file, parameters.py:169-190).  The reference's gate of
this name runs DP = 2, 200 steps, global batch 80, window [101, 201) (config/eval/dense_training/gate_config/long-train.toml):
``--nproc 2 --steps 200 --mbs 4 --accum 10 --window 101 201 --ref engine``.

The three steps of the reference's gate executor (evals/dispatcher.py:253-331): (1) run the reference side — its unmodified
pure-PyTorch L0 trainer (ref/reference/train_pure_mup_mtp.py, or ref/reference/train_qwen3_dense.py for a Qwen3 ``--model``)
from ``baseline/_ref`` as a child process; (2) run this
engine through its public entry point (``python -m forge_train_harness_b200.train``) as a child process; (3) a verdict
that only reads the two logs: mean |ours - ref| / |ref| over the step window below ``--threshold`` (the ``long-train``
rule, evals/verdicts/long_train.py:177-220) plus a first-step tolerance check (single-card alignment).

Both sides start from bit-identical weights without exchanging a file: the engine's ``init_reference`` draws every full
tensor from one CPU generator in the reference's parameter order with the reference's std rules
(model_pure_mup_mtp.py:436-477), then rounds to bf16 exactly as the reference does.  Both read the same synthetic
Megatron ``.bin/.idx`` corpus with the same shuffle rules.  A B200 engine with its own GEMM / attention kernels cannot be
bitwise equal to cuBLAS + flash-attn, so the rule is tolerance, not ``max_abs_diff == 0``.
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
REF = os.path.join(ROOT, "baseline", "_ref")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="minicpm4_0.5b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--window", type=int, nargs=2, default=[21, 61])
    ap.add_argument("--nproc", type=int, default=1)
    ap.add_argument("--mbs", type=int, default=4)
    ap.add_argument("--accum", type=int, default=2)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--threshold", type=float, default=0.01)
    ap.add_argument("--out", default="gates_out")
    ap.add_argument("--timeout", type=float, default=1500.0)
    ap.add_argument("--split-logs", default="", help="also write <dir>/ref/ref.log and <dir>/ours/ours.log (dispatcher layout)")
    ap.add_argument("--ref", default="l0", choices=["l0", "engine"], help="reference side: its L0 trainer or its produced engine")
    a = ap.parse_args(argv)
    m = preset(a.model)
    if a.layers:
        m = dataclasses.replace(m, num_layers=a.layers)
    qwen = m.qk_norm and not m.use_mup      # the Qwen3 family has its own L0 trainer (tied head, no MTP, no muP)
    m = dataclasses.replace(m, mtp_num_layers=0) if qwen else dataclasses.replace(m, tie_embeddings=False, mtp_num_layers=0)
    out = os.path.abspath(a.out)
    os.makedirs(out, exist_ok=True)
    gbs = a.mbs * a.accum * a.nproc

    rng = np.random.RandomState(0)
    n_windows = a.steps * gbs + 64
    # learnable synthetic corpus, so the loss actually moves and a numerical bias would show: a fixed random successor
    # map over a 4096-token sub-vocabulary, followed 90 % of the time
    sub = 4096
    succ = rng.permutation(sub)
    docs = []
    for _ in range((n_windows + 63) // 64):
        n = (m.seq_length + 1) * 64
        jump = rng.rand(n) < 0.1
        rnd = rng.randint(0, sub, size=n)
        d = np.empty(n, dtype=np.int32)
        d[0] = rnd[0]
        for i in range(1, n):
            d[i] = rnd[i] if jump[i] else succ[d[i - 1]]
        docs.append(d)
    prefix = os.path.join(out, "corpus")
    write_megatron_binary(prefix, docs, np.int32)
    with open(os.path.join(out, "data.toml"), "w") as f:
        f.write('[data]\ndata_loader = "megatron_binary"\n')
    with open(os.path.join(out, "data_path.txt"), "w") as f:
        f.write(f"1.0 {prefix}\n")

    canon_root = ""
    if a.ref == "engine":
        # one weight file for both sides: every full tensor from one seeded CPU generator in the reference's parameter order
        import torch
        from ..models import params as P
        canon_root = os.path.join(out, "canonical")
        os.makedirs(canon_root, exist_ok=True)
        state = {spec.name: full for spec, full in P.iter_full_init(m, 1234, True)}
        torch.save(state, os.path.join(canon_root, "canonical_state_fp32.pt"))
        del state
    port = 29600 + os.getpid() % 300
    # ---- (1) reference side --------------------------------------------------------------------------------
    env = dict(os.environ)
    for k, v in {"NUM_LAYERS": m.num_layers, "HIDDEN_SIZE": m.hidden_size, "NUM_ATTENTION_HEADS": m.num_attention_heads,
                 "NUM_QUERY_GROUPS": m.num_query_groups, "HEAD_DIM": m.head_dim, "FFN_HIDDEN_SIZE": m.ffn_hidden_size,
                 "PADDED_VOCAB_SIZE": m.padded_vocab_size, "MAX_POSITION_EMBEDDINGS": m.seq_length,
                 "NORM_EPSILON": m.norm_epsilon, "ROTARY_BASE": int(m.rotary_base)}.items():
        env[k] = str(v)
    env["PYTHONPATH"] = os.pathsep.join([REF, os.path.join(REF, "ref", "reference"), env.get("PYTHONPATH", "")])
    env["FORGE_DATA_TOML"] = os.path.join(out, "data.toml")
    ref_cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.nproc}", "--master-addr", "127.0.0.1",
               "--master-port", str(port), os.path.join(REF, "ref", "reference", "train_qwen3_dense.py" if qwen else "train_pure_mup_mtp.py"),
               "--data-path-file", os.path.join(out, "data_path.txt"), "--data-config", os.path.join(out, "data.toml"),
               "--train-iters", str(a.steps), "--micro-batch-size", str(a.mbs), "--global-batch-size", str(gbs),
               "--lr", str(a.lr), "--min-lr", str(a.lr * 0.1), "--lr-warmup-iters", "10", "--lr-decay-iters", "100000",
               "--weight-decay", "0.1", "--adam-beta1", "0.9", "--adam-beta2", "0.95", "--clip-grad", "1.0", "--seed", "1234",
               "--init-method-std", str(m.init_method_std), "--out-dir", os.path.join(out, "ref_out"), "--no-deterministic"]
    if not qwen:
        ref_cmd += ["--init-ones", "1", "--eagle-num-layers", "0"]
    if a.ref == "engine":
        ref_cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.nproc}", "--master-addr",
                   "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "baseline", "ref_engine_driver.py"),
                   "--model", a.model, "--layers", str(m.num_layers), "--steps", str(a.steps), "--mbs", str(a.mbs),
                   "--accum", str(a.accum), "--data-prefix", prefix, "--ckpt-root", canon_root, "--lr", str(a.lr)]
        env = dict(os.environ)
    r = subprocess.run(ref_cmd, env=env, cwd=out, capture_output=True, text=True, timeout=a.timeout)
    open(os.path.join(out, "ref.log"), "w").write(r.stdout + "\n--- stderr ---\n" + r.stderr[-20000:])
    ref_recs = wire.parse_loss_lines(r.stdout, strict=False)
    # ---- (2) this engine --------------------------------------------------------------------------------------
    cfg_path = os.path.join(out, "ours.toml")
    md = dataclasses.asdict(m)
    with open(cfg_path, "w") as f:
        f.write("[model]\n" + "".join(f"{k} = {json.dumps(v)}\n" for k, v in md.items()))
        f.write(f"\n[optim]\nlr = {a.lr}\nmin_lr = {a.lr * 0.1}\nlr_warmup_iters = 10\nlr_decay_iters = 100000\nlr_wsd_decay_iters = 0\n"
                "lr_schedule = \"wsd\"\nweight_decay = 0.1\nadam_beta1 = 0.9\nadam_beta2 = 0.95\nclip_grad = 1.0\n")
        f.write(f"\n[train]\nnum_steps = {a.steps}\nmicro_batch_size = {a.mbs}\nglobal_batch_size = {gbs}\nseed = 1234\ndtype = \"bf16\"\n")
        f.write(f"\n[data]\ndata_loader = \"megatron_binary\"\ndata_path = {json.dumps(prefix)}\n")
        if canon_root:
            f.write(f"\n[ckpt]\ncheckpoint_root = {json.dumps(canon_root)}\n")
    ours_cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.nproc}", "--master-addr", "127.0.0.1",
                "--master-port", str(port + 1), "-m", "forge_train_harness_b200.train", "--config", cfg_path]
    o = subprocess.run(ours_cmd, cwd=ROOT, capture_output=True, text=True, timeout=a.timeout)
    open(os.path.join(out, "ours.log"), "w").write(o.stdout + "\n--- stderr ---\n" + o.stderr[-20000:])
    our_recs = wire.parse_loss_lines(o.stdout, strict=False)
    if a.split_logs:
        for side, text in (("ref", r.stdout), ("ours", o.stdout)):
            os.makedirs(os.path.join(a.split_logs, side), exist_ok=True)
            if side == "ref" or not os.path.isfile(os.path.join(a.split_logs, side, "ours.log")):
                open(os.path.join(a.split_logs, side, f"{side}.log"), "w").write(text)
    # ---- (3) verdict ---------------------------------------------------------------------------------------------
    res = {"model": m.name, "layers": m.num_layers, "nproc": a.nproc, "reference_side": a.ref, "global_batch": gbs, "steps": a.steps,
           "ref_rc": r.returncode, "ours_rc": o.returncode, "ref_steps": len(ref_recs), "ours_steps": len(our_recs)}
    if ref_recs and our_recs:
        res["first_step"] = {"ref": ref_recs[0].loss, "ours": our_recs[0].loss,
                             "rel_diff": abs(ref_recs[0].loss - our_recs[0].loss) / abs(ref_recs[0].loss)}
        res["long_train"] = V.long_train(ref_recs, our_recs, tuple(a.window), a.threshold)
        res["grad_norm_first"] = {"ref": ref_recs[0].grad_norm, "ours": our_recs[0].grad_norm}
        res["ref_ms_per_step"] = 1e3 * float(np.median([x.time_s for x in ref_recs[5:] if x.time_s])) if len(ref_recs) > 6 else None
        res["ours_ms_per_step"] = 1e3 * float(np.median([x.time_s for x in our_recs[5:] if x.time_s])) if len(our_recs) > 6 else None
        res["passed"] = bool(res["long_train"].get("passed")) and res["first_step"]["rel_diff"] < 5e-3
    else:
        res["passed"] = False
    with open(os.path.join(out, "alignment.json"), "w") as f:
        json.dump(res, f, indent=1)
    print(json.dumps(res), flush=True)
    return 0 if res["passed"] else 1


if __name__ == "__main__":
    sys.exit(main())
