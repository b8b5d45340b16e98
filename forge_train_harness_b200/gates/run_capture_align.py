"""forward-align / backward-align against the LIVE reference model, in tolerance mode.

    python -m forge_train_harness_b200.gates.run_capture_align --out align_out [--model tiny --set num_layers=2 ...]

Three steps, as every gate (evals/dispatcher.py:253-331): (1) the reference side — ``baseline/ref_capture_bridge.py`` runs one
micro-batch through the reference's unmodified ``MiniCPM4MupMtp`` with forward / full-backward hooks and keeps the tensors;
(2) this engine runs the same micro-batch from the same ``canonical_state_fp32.pt`` with ``CaptureSession(level=2,
mode="tensor")``; (3) ``verdicts.align_tolerance`` per key family: ``fwd`` and ``loss`` and ``grad`` compared as they are,
``bwd`` (gradients w.r.t. module outputs) after removing one scalar per key, because the two stacks apply the residual
scale on different sides of the hook point.  The reference's own forward-align / backward-align gates demand equal blake2b
digests (evals/verdicts/align.py:1-20), which only an engine running the same cuBLAS / flash-attn kernels can meet.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import subprocess
import sys

import torch

from ..config.schema import DataConfig, OptimConfig, RunConfig, TrainConfig, CkptConfig, preset
from ..models import params as P
from . import verdicts as V
from .capture import CaptureSession

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--set", action="append", default=["num_layers=2", "hidden_size=256", "ffn_hidden_size=512", "num_attention_heads=4",
                                                       "num_query_groups=2", "head_dim=64", "seq_length=256", "padded_vocab_size=4096"])
    ap.add_argument("--mbs", type=int, default=2)
    ap.add_argument("--out", default="align_out")
    ap.add_argument("--fwd-tol", type=float, default=1e-2, help="relative L2 error per module output")
    ap.add_argument("--bwd-tol", type=float, default=3e-2)
    ap.add_argument("--grad-tol", type=float, default=3e-2)
    a = ap.parse_args(argv)
    out = os.path.abspath(a.out)
    os.makedirs(out, exist_ok=True)
    m = preset(a.model)
    over = {}
    for kv in a.set:
        k, v = kv.split("=", 1)
        cur = getattr(m, k)
        over[k] = type(cur)(v) if not isinstance(cur, bool) else v.lower() in ("1", "true")
    m = dataclasses.replace(m, tie_embeddings=False, mtp_num_layers=0, **over)
    canon = os.path.join(out, "canonical_state_fp32.pt")
    torch.save({spec.name: full for spec, full in P.iter_full_init(m, 1234, True)}, canon)
    # (1) reference side
    ref_pt = os.path.join(out, "ref_capture.pt")
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "ref_capture_bridge.py"), "--model", a.model, "--canonical", canon,
           "--mbs", str(a.mbs), "--out", ref_pt] + [x for kv in a.set for x in ("--set", kv)]
    r = subprocess.run(cmd, cwd=out, capture_output=True, text=True, timeout=900)
    open(os.path.join(out, "ref.log"), "w").write(r.stdout + "\n--- stderr ---\n" + r.stderr[-20000:])
    res = {"ref_rc": r.returncode}
    if r.returncode != 0:
        res.update(passed=False, reason="reference capture failed", failure_class=V.classify_failure(r.stdout + r.stderr))
        print(json.dumps(res))
        return 1
    # (2) this engine, one micro-batch, tensors kept
    from ..engine import Trainer
    our_pt = os.path.join(out, "ours_capture.pt")
    cfg = RunConfig(model=m, optim=OptimConfig(lr=1e-3, lr_schedule="constant"),
                    train=TrainConfig(num_steps=1, micro_batch_size=a.mbs, grad_accum_steps=1, seed=1234, dtype="bf16", cuda_graph=False),
                    data=DataConfig(data_loader="synthetic", synthetic_seed=0, prefetch_size=0), ckpt=CkptConfig(checkpoint_root=out))
    sess = CaptureSession(our_pt, level=2, rank=0, mode="tensor")
    tr = Trainer(cfg, capture=sess, quiet=True)
    tr.train_step()
    sess.dump()
    tr.close()
    # (3) verdicts
    # this engine folds the muP embedding scale into the lookup, the reference multiplies after its embedding module
    scales = {"fwd.tok_embeddings": 1.0 / m.emb_scale}
    with open(os.path.join(out, "scales.json"), "w") as f:
        json.dump(scales, f)
    res["forward_align"] = V.align_tolerance(ref_pt, our_pt, "fwd", a.fwd_tol, scales=scales)
    res["backward_align"] = V.align_tolerance(ref_pt, our_pt, "bwd", a.bwd_tol, fit_scale=True)
    res["grad_align"] = V.align_tolerance(ref_pt, our_pt, "grad", a.grad_tol)
    res["loss_align"] = V.align_tolerance(ref_pt, our_pt, "loss", 1e-2)
    res["passed"] = all(res[k]["passed"] for k in ("forward_align", "backward_align", "grad_align", "loss_align"))
    with open(os.path.join(out, "capture_align.json"), "w") as f:
        json.dump(res, f, indent=1)
    print(json.dumps({k: (v if not isinstance(v, dict) else {x: v[x] for x in ("passed", "checks_total", "worst_rel_err") if x in v})
                      for k, v in res.items()}), flush=True)
    return 0 if res["passed"] else 1


if __name__ == "__main__":
    sys.exit(main())
