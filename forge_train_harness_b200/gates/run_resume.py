"""Resume self-compare in one process: Phase R (uninterrupted, ``[LOSS_REF]``), Phase A (train to ``--save-step``, save),
Phase B (load, continue, ``[LOSS_RES]``) — the in-process variant of the reference's resume gate
(evals/scripts/eval_resume_train.py:161-214); ``gates.verdicts.resume`` then demands max abs diff == 0 over the window."""
from __future__ import annotations

import argparse
import os
import sys

from ..config import schema
from ..engine import run_training_loop


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--save-step", type=int, default=3)
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    cfg = schema.load(a.config)
    cfg = cfg.replace(parallel={"use_distributed_optimizer": False}) if int(os.environ.get("WORLD_SIZE", "1")) == 1 else cfg
    ck = os.path.join(a.out, "ckpt")
    run_training_loop(cfg.replace(train={"num_steps": a.steps}), loss_tag="LOSS_REF")
    run_training_loop(cfg.replace(train={"num_steps": a.save_step, "save_path": ck}), loss_tag="LOSS")
    run_training_loop(cfg.replace(train={"num_steps": a.steps - a.save_step, "resume_from": ck, "start_step": a.save_step}),
                      loss_tag="LOSS_RES")


if __name__ == "__main__":
    main()
    sys.exit(0)
