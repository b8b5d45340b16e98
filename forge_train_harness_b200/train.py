"""Training entry point.

    python -m forge_train_harness_b200.train --config run.toml [--set train.num_steps=100 ...]
    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m forge_train_harness_b200.train --config run.toml
    python -m forge_train_harness_b200.runtime.launcher --nproc 8 -- python -m forge_train_harness_b200.train --config run.toml

Reads the layered TOML (``[model]`` / ``[optim]`` / ``[parallel]`` / ``[train]`` / ``[data]`` / ``[ckpt]``, or a rendered gate
product with ``[cli]``), optionally a multi-phase recipe (``--recipe``; stable -> decay -> sft, the reference's three-phase
WSD + SFT driver, evals/scripts/train_ours_al.sh:251-311), and runs the engine.  Phases are checkpoint-driven: a phase
whose final checkpoint exists is skipped, a phase with a partial checkpoint resumes from it, a fresh phase starts from
the previous phase's weights (``init_weights_only`` for the SFT hand-off).
"""
from __future__ import annotations

import argparse
import os
import sys
import tomllib

from .config import schema
from .engine import ordered_teardown, run_training_loop
from .parallel.topology import init_distributed


def _apply_sets(cfg, sets):
    """``table.field=value`` overrides, all applied in ONE step (so a set of overrides that is only valid together, such as a
    new pipeline size with a new layer split, does not trip the cross-table checks half-way)."""
    tables: dict = {}
    for item in sets or []:
        key, val = item.split("=", 1)
        table, field = key.split(".", 1)
        cur = getattr(getattr(cfg, table), field)
        if isinstance(cur, bool):
            v = val.lower() in ("1", "true", "yes")
        elif isinstance(cur, int):
            v = int(val)
        elif isinstance(cur, float):
            v = float(val)
        elif isinstance(cur, (list, tuple)):   # e.g. parallel.pipeline_layer_split=17,15 ; "" or "none" empties it
            v = tuple(int(x) for x in val.split(",") if x.strip()) if val not in ("", "none", "None") else ()
        else:
            v = None if val in ("", "none", "None") else val
        tables.setdefault(table, {})[field] = v
    return cfg.replace(**tables) if tables else cfg


def run_phases(cfg, recipe: dict, out=None):
    """``recipe``: {"phases": {"stable": {...}, "decay": {...}, "sft": {...}}, "order": [...], "save_root": ...}."""
    from .ckpt.manager import latest_iteration
    order = recipe.get("order") or list(recipe["phases"])
    root = recipe["save_root"]
    prev_dir, start = None, 0
    all_records = []
    for name in order:
        ph = dict(recipe["phases"][name])
        steps = int(ph.pop("num_steps"))
        phase_dir = os.path.join(root, name)
        end = start + steps
        done = latest_iteration(phase_dir) if os.path.isdir(phase_dir) else None
        tr_over = {"phase_name": name, "save_path": phase_dir, "save_interval": int(ph.pop("save_interval", 0))}
        init_only = bool(ph.pop("init_weights_only", False))
        data_over = {k[5:]: ph.pop(k) for k in list(ph) if k.startswith("data_")}
        if done is not None and done >= end:
            prev_dir, start = phase_dir, end
            continue
        if done is not None and done > start:  # crash-restart inside the phase
            tr_over.update(start_step=done, num_steps=end - done, resume_from=phase_dir, init_weights_only=False)
        else:
            tr_over.update(start_step=start, num_steps=steps, resume_from=prev_dir, init_weights_only=init_only and prev_dir is not None)
        c = cfg.replace(train=tr_over, optim=ph, data=data_over) if data_over else cfg.replace(train=tr_over, optim=ph)
        if prev_dir is not None and tr_over["resume_from"] == prev_dir and not tr_over["init_weights_only"]:
            # continue from the previous phase's optimizer state and step counter
            pass
        all_records += run_training_loop(c, out=out)
        prev_dir, start = phase_dir, end
    return all_records


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--recipe", default="")
    ap.add_argument("--set", action="append", default=[])
    ap.add_argument("--loss-tag", default=None)
    ap.add_argument("--reference-env", action="store_true",
                    help="apply the reference engine's environment variables (NUM_LAYERS ... LR ... ENABLE_CUDA_GRAPH, "
                         "ENABLE_TRITON_*) on top of the config file: a launch environment written for the reference drives this engine")
    a = ap.parse_args(argv)
    cfg = schema.load(a.config)
    if a.reference_env:
        from .config.ref_env import apply_reference_env, op_env_from_reference
        cfg = apply_reference_env(cfg, os.environ)
        for k, v in op_env_from_reference(os.environ).items():
            os.environ.setdefault(k, v)          # an explicit OP_<NAME> still wins
            if v == "baseline":
                os.environ.setdefault("FORGE_ALLOW_BASELINE", "1")
    cfg = _apply_sets(cfg, a.set)
    created = init_distributed()
    if a.recipe:
        with open(a.recipe, "rb") as f:
            run_phases(cfg, tomllib.load(f))
    else:
        run_training_loop(cfg, loss_tag=a.loss_tag)
    ordered_teardown(created)


if __name__ == "__main__":
    main()
    sys.exit(0)
