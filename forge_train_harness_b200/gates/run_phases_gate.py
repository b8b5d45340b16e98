"""Three-phase (stable -> decay -> sft) production run with host-side crash injection, for the ``wsd-sft`` and
``production-resume`` gates.

    python -m forge_train_harness_b200.gates.run_phases_gate --config run.toml --recipe recipe.toml --out <dir> --kill-at 3,7,10

Two passes of ``python -m forge_train_harness_b200.train --recipe``: a CLEAN one (``<out>/ref/ref.log``) and a MAIN one
(``<out>/ours/ours.log``) that is killed from outside — this process watches the child's output and sends SIGKILL to exactly
that child as soon as it has printed the ``[LOSS]`` line of each step in ``--kill-at`` — and restarted until it completes.
The faults are made on the host, between steps; nothing is injected on the device.  ``verdicts.wsd_sft`` then demands the
same phase order and banners and per-phase trajectory equality, ``verdicts.production`` that every expected checkpoint is
complete.  The reference's versions: evals/scripts/train_ours_al.sh:251-311 (driver), train_ours_al_resume.sh:61-117 (kill
injector), evals/verdicts/wsd_sft.py and production.py.
"""
from __future__ import annotations

import argparse
import os
import re
import signal
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run_until(argv, kill_at: int | None, timeout_s: float, env=None) -> tuple[int, str]:
    """Run ``argv``; if ``kill_at`` is set, SIGKILL the child (its PID, nothing else) once it printed that step's loss line."""
    p = subprocess.Popen(argv, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    lines = []
    pat = re.compile(r"^\[LOSS\] step=(\d+) ")
    try:
        for ln in p.stdout:
            lines.append(ln)
            m = pat.match(ln)
            if kill_at is not None and m and int(m[1]) == kill_at:
                os.kill(p.pid, signal.SIGKILL)
                break
        rc = p.wait(timeout=timeout_s)
    except subprocess.TimeoutExpired:
        p.kill()
        rc = p.wait()
    return rc, "".join(lines)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--recipe", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--kill-at", default="", help="comma-separated absolute steps after which the main run is killed")
    ap.add_argument("--timeout", type=float, default=1200.0)
    ap.add_argument("--set", action="append", default=[])
    a = ap.parse_args(argv)
    out = os.path.abspath(a.out)
    sets = [x for s in a.set for x in ("--set", s)]
    import tomllib
    with open(a.recipe, "rb") as f:
        recipe = tomllib.load(f)
    logs = {}
    for side, kills in (("ref", []), ("ours", [int(k) for k in a.kill_at.split(",") if k.strip()])):
        d = os.path.join(out, side)
        os.makedirs(d, exist_ok=True)
        # the recipe's save_root is redirected under this side's directory
        rpath = os.path.join(d, "recipe.toml")
        body = open(a.recipe).read()
        body = re.sub(r'(?m)^save_root\s*=.*$', f'save_root = "{os.path.join(d, "ckpt")}"', body)
        if "save_root" not in body:
            body = f'save_root = "{os.path.join(d, "ckpt")}"\n' + body
        open(rpath, "w").write(body)
        cmd = [sys.executable, "-m", "forge_train_harness_b200.train", "--config", a.config, "--recipe", rpath] + sets
        text = ""
        for k in kills + [None]:
            rc, t = run_until(cmd, k, a.timeout)
            text += t
            if k is None and rc != 0:
                open(os.path.join(d, f"{side}.log"), "w").write(text)
                print(f"{side} run failed with status {rc}", file=sys.stderr)
                return 1
            if k is not None and rc != -signal.SIGKILL:
                text += f"\n[gate] expected the run to be killed after step {k}, it exited with status {rc}\n"
        open(os.path.join(d, f"{side}.log"), "w").write(text)
        logs[side] = text
    print(logs["ours"], end="")
    print(f"[gate] phases: {recipe.get('order') or list(recipe['phases'])}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
