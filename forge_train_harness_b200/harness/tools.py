"""Small operator tools of the control plane.

* ``canonical``  — write ``canonical_state_fp32.pt`` for a model shape: every full tensor from one seeded CPU generator in the
  reference's parameter order, the hand-off file both sides of a gate can start from (tools/bootstrap_canonical.py; the
  reference keeps two, ``ones/`` with norm weights 1 and ``no1/`` with 0.97, chosen by a gate's ``forge_init_ones``).
* ``canonical-preflight`` — before a gate spends GPU time: the canonical file exists, holds exactly the model's parameters with
  the right shapes in fp32, is finite, and (when a ``.sha256`` file sits beside it) has the recorded digest
  (tools/canonical_preflight.sh, evals/canonical_preflight.py).
* ``recipe-env`` — project a training recipe TOML into shell lines ``export VAR="${VAR:-value}"``: the environment wins, the
  recipe supplies defaults; an unknown top-level table is an error, so no key silently never reaches the shell
  (tools/train_recipe_to_env.py).
* ``data-check`` — build a data source twice from fresh instances, hash the first N micro-batches of every DP rank, and
  require identical streams: same seed, same bytes (tools/hf_data_bitwise_check.py).  Works for every ``data_loader``.
* ``capture-batch`` — save one micro-batch ``{tokens, labels, loss_mask}`` of the configured data source to a file inside the
  workspace, so that profiling runs a fixed input and needs nothing from outside the tree (tools/capture_profile_batch.py).

    python -m forge_train_harness_b200.harness.tools canonical --model minicpm4_0.5b --out ckpt_root [--init-ones 0|1] [--layers N]
    python -m forge_train_harness_b200.harness.tools canonical-preflight --model minicpm4_0.5b --file ckpt_root/ones/canonical_state_fp32.pt
    python -m forge_train_harness_b200.harness.tools recipe-env configs/eval/recipe_wsd_sft_tiny.toml
    python -m forge_train_harness_b200.harness.tools data-check --config run.toml [--dp 2] [--batches 16]
    python -m forge_train_harness_b200.harness.tools capture-batch --config run.toml --out profiles_in/captured_batch.pt
"""
from __future__ import annotations

import argparse
import dataclasses
import hashlib
import json
import os
import sys
import tomllib

RECIPE_TABLES = ("launch", "common", "train", "phases")


def write_canonical(model_cfg, out_root: str, seed: int = 1234, init_ones: bool = True) -> str:
    import torch

    from ..models import params as P
    sub = os.path.join(out_root, "ones" if init_ones else "no1")
    os.makedirs(sub, exist_ok=True)
    path = os.path.join(sub, "canonical_state_fp32.pt")
    state = {spec.name: full for spec, full in P.iter_full_init(model_cfg, seed, init_ones)}
    tmp = path + ".tmp"
    torch.save(state, tmp)
    os.replace(tmp, path)
    return path


def canonical_preflight(model_cfg, path: str) -> dict:
    import torch

    from ..models import params as P
    problems = []
    if not os.path.isfile(path):
        return {"passed": False, "problems": [f"{path} does not exist"]}
    side = path + ".sha256"
    digest = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 24), b""):
            digest.update(chunk)
    if os.path.isfile(side):
        want = open(side).read().split()[0].strip()
        if want != digest.hexdigest():
            problems.append(f"sha256 {digest.hexdigest()[:16]}... differs from the recorded {want[:16]}...")
    state = torch.load(path, map_location="cpu", weights_only=True, mmap=True)
    specs = {s.name: s for s in P.full_param_specs(model_cfg)}
    for name in sorted(set(specs) - set(state)):
        problems.append(f"missing {name}")
    for name in sorted(set(state) - set(specs)):
        problems.append(f"unexpected {name}")
    for name, spec in specs.items():
        t = state.get(name)
        if t is None:
            continue
        if tuple(t.shape) != tuple(spec.full_shape):
            problems.append(f"{name}: shape {tuple(t.shape)}, model wants {tuple(spec.full_shape)}")
        elif t.dtype != torch.float32:
            problems.append(f"{name}: dtype {t.dtype}, want float32")
        elif not bool(torch.isfinite(t).all()):
            problems.append(f"{name}: not finite")
    return {"passed": not problems, "problems": problems[:20], "sha256": digest.hexdigest(), "tensors": len(state)}


def recipe_env_lines(recipe: dict) -> list[str]:
    """``export KEY="${KEY:-value}"`` per recipe key: [launch] / [common] / [train] keys upper-cased as they are, phase keys
    prefixed with the phase name; top-level scalars (``save_root``, ``order``) likewise."""
    lines = []

    def emit(name: str, value) -> None:
        if isinstance(value, bool):
            value = "1" if value else "0"
        elif isinstance(value, (list, tuple)):
            value = " ".join(str(v) for v in value)
        text = "".join("\\" + ch if ch in '"$`\\}' else ch for ch in str(value))   # literal inside "${VAR:-...}"
        lines.append(f'export {name}="${{{name}:-{text}}}"')

    for key, val in recipe.items():
        if isinstance(val, dict):
            if key not in RECIPE_TABLES:
                raise ValueError(f"unknown recipe table [{key}] (known: {', '.join(RECIPE_TABLES)})")
            if key == "phases":
                for phase, table in val.items():
                    if not isinstance(table, dict):
                        raise ValueError(f"[phases.{phase}] must be a table")
                    for k, v in table.items():
                        emit(f"{phase.upper()}_{k.upper()}", v)
            else:
                for k, v in val.items():
                    emit(k.upper(), v)
        else:
            emit(key.upper(), val)
    return lines


def batch_hashes(data_cfg, model_cfg, micro_batch: int, dp: int, seed: int, n: int) -> list[list[str]]:
    from ..data.sources import build_source
    out = []
    for rank in range(dp):
        src = build_source(data_cfg, model_cfg, micro_batch, rank, dp, seed)
        hs = []
        for _ in range(n):
            b = next(src)
            h = hashlib.sha256()
            for k in ("tokens", "labels"):
                h.update(b[k].contiguous().numpy().tobytes())
            hs.append(h.hexdigest())
        if hasattr(src, "close"):
            src.close()
        out.append(hs)
    return out


def data_check(cfg, dp: int, n: int) -> dict:
    a = batch_hashes(cfg.data, cfg.model, cfg.train.micro_batch_size, dp, cfg.train.seed, n)
    b = batch_hashes(cfg.data, cfg.model, cfg.train.micro_batch_size, dp, cfg.train.seed, n)
    bad = [(r, i) for r in range(dp) for i in range(n) if a[r][i] != b[r][i]]
    dup = dp > 1 and any(a[0][i] == a[r][i] for r in range(1, dp) for i in range(n))   # ranks must not read the same samples
    return {"passed": not bad and not dup, "ranks": dp, "batches": n, "mismatched": bad[:10], "ranks_share_samples": bool(dup),
            "first_hash": a[0][0] if a and a[0] else ""}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="tools")
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("canonical")
    c.add_argument("--model", required=True)
    c.add_argument("--out", required=True)
    c.add_argument("--seed", type=int, default=1234)
    c.add_argument("--init-ones", type=int, choices=[0, 1], required=True)
    c.add_argument("--layers", type=int, default=0)
    cp = sub.add_parser("canonical-preflight")
    cp.add_argument("--model", required=True)
    cp.add_argument("--file", required=True)
    cp.add_argument("--layers", type=int, default=0)
    r = sub.add_parser("recipe-env")
    r.add_argument("recipe")
    d = sub.add_parser("data-check")
    d.add_argument("--config", required=True)
    d.add_argument("--dp", type=int, default=1)
    d.add_argument("--batches", type=int, default=16)
    cb = sub.add_parser("capture-batch")
    cb.add_argument("--config", required=True)
    cb.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    from ..config import schema
    if a.cmd == "canonical":
        m = schema.preset(a.model)
        if a.layers:
            m = dataclasses.replace(m, num_layers=a.layers)
        print(write_canonical(m, a.out, a.seed, bool(a.init_ones)))
        return 0
    if a.cmd == "canonical-preflight":
        m = schema.preset(a.model)
        if a.layers:
            m = dataclasses.replace(m, num_layers=a.layers)
        res = canonical_preflight(m, a.file)
        print(json.dumps(res, indent=1))
        return 0 if res["passed"] else 1
    if a.cmd == "recipe-env":
        with open(a.recipe, "rb") as f:
            try:
                print("\n".join(recipe_env_lines(tomllib.load(f))))
            except ValueError as e:
                print(f"recipe-env: {e}", file=sys.stderr)
                return 1
        return 0
    cfg = schema.load(a.config)
    if a.cmd == "data-check":
        res = data_check(cfg, a.dp, a.batches)
        print(json.dumps(res))
        return 0 if res["passed"] else 1
    import torch

    from ..data.sources import build_source
    src = build_source(cfg.data, cfg.model, cfg.train.micro_batch_size, 0, 1, cfg.train.seed)
    b = next(src)
    os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
    torch.save({k: b[k] for k in ("tokens", "labels", "loss_mask")}, a.out)
    print(json.dumps({"out": a.out, "tokens": list(b["tokens"].shape), "data_loader": cfg.data.data_loader}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
