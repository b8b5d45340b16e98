"""The DP x TP gate against the reference's hand-written tensor-parallel trainer (``ref/reference/train_minicpm4_8b_tp.py``).

    python -m forge_train_harness_b200.gates.run_dptp --out dptp_out [--nproc 4 --tp 2 --layers 4 --steps 8]

The reference's gate of this name (config/eval/dense_training_8b/gate_config/dptp.toml): 4 GPUs = DP 2 x TP 2, the 8B shape cut
to 4 layers, micro-batch 2, global batch 16, 8 steps, no warm-up, bitwise on loss and gradient norm.  Here: (1) the
UNMODIFIED reference trainer runs as a child process from ``baseline/_ref`` (its geometry and muP knobs come from the
environment, model_minicpm4_8b_tp.py:29-43); (2) this engine runs the same shape, data and seed at TP 2 x DP 2 with
``parallel.clip_norm_scope = "tp_local"``, because the reference clips every TP rank by the norm of its own shards
(train_minicpm4_8b_tp.py:321) and prints rank 0's; (3) ``verdicts.trajectory`` with a relative tolerance on loss and
gradient norm (a tcgen05 GEMM and this attention kernel are not bit-equal to cuBLAS and flash-attn).  Both sides draw
every full tensor from one seeded CPU generator in the same parameter order and slice their shard, so they start from
identical weights without exchanging a file (model_minicpm4_8b_tp.py:552-601).
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
    ap.add_argument("--model", default="minicpm4_8b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--nproc", type=int, default=4)
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--mbs", type=int, default=2)
    ap.add_argument("--gbs", type=int, default=16)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--loss-rtol", type=float, default=5e-3)
    ap.add_argument("--sp", type=int, default=1, help="run this engine with sequence parallelism (the fused TP kernels)")
    ap.add_argument("--out", default="dptp_out")
    ap.add_argument("--timeout", type=float, default=1500.0)
    ap.add_argument("--split-logs", default="")
    a = ap.parse_args(argv)
    m = dataclasses.replace(preset(a.model), num_layers=a.layers, tie_embeddings=False, mtp_num_layers=0)
    out = os.path.abspath(a.out)
    os.makedirs(out, exist_ok=True)
    rng = np.random.RandomState(0)
    sub, n_docs = 4096, (a.steps * a.gbs + 63) // 64 + 1
    succ = rng.permutation(sub)
    docs = []
    for _ in range(n_docs):
        n = (m.seq_length + 1) * 64
        jump, rnd = rng.rand(n) < 0.1, rng.randint(0, sub, size=n)
        d = np.empty(n, dtype=np.int32)
        d[0] = rnd[0]
        for i in range(1, n):
            d[i] = rnd[i] if jump[i] else succ[d[i - 1]]
        docs.append(d)
    prefix = os.path.join(out, "corpus")
    write_megatron_binary(prefix, docs, np.int32)
    open(os.path.join(out, "data.toml"), "w").write('[data]\ndata_loader = "megatron_binary"\n')
    open(os.path.join(out, "data_path.txt"), "w").write(f"1.0 {prefix}\n")
    port = 29800 + os.getpid() % 150
    # ---- (1) the reference's DP x TP trainer -------------------------------------------------------------------------
    env = dict(os.environ)
    env.update({"NUM_LAYERS": str(m.num_layers), "HIDDEN_SIZE": str(m.hidden_size), "NUM_ATTENTION_HEADS": str(m.num_attention_heads),
                "NUM_QUERY_GROUPS": str(m.num_query_groups), "HEAD_DIM": str(m.head_dim), "FFN_HIDDEN_SIZE": str(m.ffn_hidden_size),
                "PADDED_VOCAB_SIZE": str(m.padded_vocab_size), "MAX_POSITION_EMBEDDINGS": str(m.seq_length),
                "NORM_EPSILON": str(m.norm_epsilon), "ROTARY_BASE": str(int(m.rotary_base)),
                "MUP_BASE_HIDDEN_SIZE": str(m.mup_base_hidden_size), "MUP_EMB_SCALE": str(m.mup_emb_scale),
                "MUP_DEPTH_SCALE": str(m.mup_depth_scale), "TENSOR_PARALLEL_SIZE": str(a.tp),
                "FORGE_DATA_TOML": os.path.join(out, "data.toml")})
    env["PYTHONPATH"] = os.pathsep.join([REF, os.path.join(REF, "ref", "reference"), env.get("PYTHONPATH", "")])
    ref_cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.nproc}", "--master-addr", "127.0.0.1",
               "--master-port", str(port), os.path.join(REF, "ref", "reference", "train_minicpm4_8b_tp.py"),
               "--data-path-file", os.path.join(out, "data_path.txt"), "--data-config", os.path.join(out, "data.toml"),
               "--train-iters", str(a.steps), "--micro-batch-size", str(a.mbs), "--global-batch-size", str(a.gbs),
               "--lr", str(a.lr), "--min-lr", str(a.lr * 0.1), "--lr-warmup-iters", "0", "--lr-decay-iters", "100000",
               "--weight-decay", "0.1", "--adam-beta1", "0.9", "--adam-beta2", "0.95", "--clip-grad", "1.0", "--seed", "1234",
               "--init-method-std", str(m.init_method_std), "--tensor-parallel-size", str(a.tp),
               "--out-dir", os.path.join(out, "ref_out"), "--no-deterministic"]
    r = subprocess.run(ref_cmd, env=env, cwd=out, capture_output=True, text=True, timeout=a.timeout)
    open(os.path.join(out, "ref.log"), "w").write(r.stdout + "\n--- stderr ---\n" + r.stderr[-20000:])
    ref_recs = wire.parse_loss_lines(r.stdout, strict=False)
    # ---- (2) this engine ----------------------------------------------------------------------------------------------------
    cfg_path = os.path.join(out, "ours.toml")
    with open(cfg_path, "w") as f:
        f.write("[model]\n" + "".join(f"{k} = {json.dumps(v)}\n" for k, v in dataclasses.asdict(m).items()))
        f.write(f"\n[optim]\nlr = {a.lr}\nmin_lr = {a.lr * 0.1}\nlr_warmup_iters = 0\nlr_decay_iters = 100000\nlr_wsd_decay_iters = 0\n"
                "lr_schedule = \"wsd\"\nweight_decay = 0.1\nadam_beta1 = 0.9\nadam_beta2 = 0.95\nclip_grad = 1.0\n")
        f.write(f"\n[train]\nnum_steps = {a.steps}\nmicro_batch_size = {a.mbs}\nglobal_batch_size = {a.gbs}\nseed = 1234\ndtype = \"bf16\"\n"
                "forge_init_ones = true\n")
        f.write(f"\n[data]\ndata_loader = \"megatron_binary\"\ndata_path = {json.dumps(prefix)}\n")
        f.write(f"\n[parallel]\ntensor_parallel_size = {a.tp}\nsequence_parallel = {'true' if a.sp else 'false'}\n"
                "clip_norm_scope = \"tp_local\"\n")
    ours_cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.nproc}", "--master-addr", "127.0.0.1",
                "--master-port", str(port + 1), "-m", "forge_train_harness_b200.train", "--config", cfg_path]
    o = subprocess.run(ours_cmd, cwd=ROOT, capture_output=True, text=True, timeout=a.timeout)
    open(os.path.join(out, "ours.log"), "w").write(o.stdout + "\n--- stderr ---\n" + o.stderr[-20000:])
    our_recs = wire.parse_loss_lines(o.stdout, strict=False)
    if a.split_logs:
        for side, text in (("ref", r.stdout), ("ours", o.stdout)):
            os.makedirs(os.path.join(a.split_logs, side), exist_ok=True)
            open(os.path.join(a.split_logs, side, f"{side}.log"), "w").write(text)
    # ---- (3) verdict --------------------------------------------------------------------------------------------------------
    res = {"model": m.name, "layers": m.num_layers, "nproc": a.nproc, "tp": a.tp, "ref_rc": r.returncode, "ours_rc": o.returncode,
           "ref_steps": len(ref_recs), "ours_steps": len(our_recs)}
    if ref_recs and our_recs:
        t = V.trajectory(ref_recs, our_recs, (1, a.steps + 1), rtol=a.loss_rtol, check_grad_norm=False)
        gn = V.trajectory(ref_recs, our_recs, (1, a.steps + 1), rtol=4 * a.loss_rtol)
        res["loss_trajectory"], res["with_grad_norm"] = t, gn
        res["first_step"] = {"ref": [ref_recs[0].loss, ref_recs[0].grad_norm], "ours": [our_recs[0].loss, our_recs[0].grad_norm]}
        res["passed"] = bool(t["passed"]) and bool(gn["passed"]) and r.returncode == 0 and o.returncode == 0
    else:
        res["passed"] = False
        res["failure_class"] = V.classify_failure(r.stdout + r.stderr if not ref_recs else o.stdout + o.stderr)
    with open(os.path.join(out, "dptp.json"), "w") as f:
        json.dump(res, f, indent=1)
    print(json.dumps(res), flush=True)
    return 0 if res["passed"] else 1


if __name__ == "__main__":
    sys.exit(main())
