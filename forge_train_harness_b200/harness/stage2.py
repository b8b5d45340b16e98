"""Per-operator workflow: inventory, status and the ``op-long`` gate (swap exactly one op, train, compare the loss window).

The reference's stage-2 dispatcher (evals/dispatcher_stage2.py) has three suites:

* ``op-inventory`` (:210-410)  artefact / wiring validation: every registered op names its selector variable, its default and
  available versions, its kernel source and its contract test, and all of them exist and agree with the op router;
* ``op-long <name>`` (:459-475, 525-536)  the only hard gate of an op: train with that op at its hand-written version and
  everything else at the plain-PyTorch version, against a run with EVERY op at the plain-PyTorch version, same seed and
  data; mean |relative loss diff| over the window at most ``rel_diff_threshold`` (1 %).  Swapping one op at a time is what
  localises a biased kernel that per-op tolerance tests let through;
* ``op-status`` (:690-808)  per op: ``merged`` (default is the hand-written version and its last op-long passed), ``failed``,
  ``not_started`` (no hand-written version), ``inconsistent`` (registry and router disagree, or the default was switched
  without a passing op-long on record).

GPU sharing follows the reference's protocol (:81-110): runs that need the whole device (``op-long``) take an EXCLUSIVE lock
on ``.artifacts/locks/stage2-gpu.lock``, per-op tests a SHARED one, so several workers can share one box.
"""
from __future__ import annotations

import contextlib
import fcntl
import json
import os
import re
import subprocess
import sys
import tomllib

from ..ops import OP_NAMES
from ..utils import wire
from . import run_schema as RS

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REGISTRY = os.path.join(ROOT, "configs", "ops", "register.toml")


def load_registry(path: str = REGISTRY) -> dict:
    with open(path, "rb") as f:
        return tomllib.load(f)


@contextlib.contextmanager
def gpu_lock(exclusive: bool, lock_dir: str | None = None):
    d = lock_dir or os.path.join(ROOT, ".artifacts", "locks")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "stage2-gpu.lock"), "a+") as f:
        fcntl.flock(f, fcntl.LOCK_EX if exclusive else fcntl.LOCK_SH)
        try:
            yield
        finally:
            fcntl.flock(f, fcntl.LOCK_UN)


def _exists(ref: str) -> tuple[bool, str]:
    """``path::symbol``: the file exists and mentions the symbol."""
    if not ref:
        return True, ""
    path, _, sym = ref.partition("::")
    full = os.path.join(ROOT, path)
    if not os.path.isfile(full):
        return False, f"{path} does not exist"
    if sym and not re.search(r"\b" + re.escape(sym) + r"\b", open(full, errors="replace").read()):
        return False, f"{path} does not define {sym}"
    return True, ""


def op_inventory(registry: dict | None = None) -> dict:
    reg = registry or load_registry()
    ops = reg.get("ops", {})
    rows, problems = {}, []
    for name in OP_NAMES:
        ent = ops.get(name)
        if ent is None:
            problems.append(f"{name}: not in the registry")
            continue
        row = {"env_var": ent.get("env_var"), "default": ent.get("default"), "available": ent.get("available", [])}
        want_env = "OP_" + name.upper().rstrip("_")
        if row["env_var"] != want_env:
            problems.append(f"{name}: env_var {row['env_var']!r} is not what the router reads ({want_env})")
        if row["default"] not in row["available"] or "baseline" not in row["available"]:
            problems.append(f"{name}: default / baseline missing from available {row['available']}")
        if row["default"] != "baseline" and not ent.get("kernel"):
            problems.append(f"{name}: a hand-written default needs a kernel source")
        for key in ("kernel", "test"):
            ok, why = _exists(ent.get(key, ""))
            if not ok:
                problems.append(f"{name}: {key}: {why}")
        rows[name] = row
    for extra in sorted(set(ops) - set(OP_NAMES)):
        problems.append(f"{extra}: registered but not an engine op")
    return {"passed": not problems, "ops_total": len(OP_NAMES), "ops_registered": len(rows), "problems": problems, "ops": rows}


def _results_dir() -> str:
    return os.path.join(ROOT, ".artifacts", "op_long")


def op_status(registry: dict | None = None, results_dir: str | None = None) -> dict:
    reg = registry or load_registry()
    inv = op_inventory(reg)
    rd = results_dir or _results_dir()
    out, counts = {}, {"merged": 0, "failed": 0, "not_started": 0, "inconsistent": 0, "unverified": 0}
    bad = {p.split(":", 1)[0] for p in inv["problems"]}
    for name, row in inv["ops"].items():
        last = None
        path = os.path.join(rd, f"{name}.json")
        if os.path.isfile(path):
            with open(path) as f:
                last = json.load(f)
        if name in bad:
            st = "inconsistent"
        elif row["default"] == "baseline":
            st = "not_started"
        elif last is None:
            st = "unverified"        # hand-written default with no op-long on record on this machine
        elif last.get("passed"):
            st = "merged"
        else:
            st = "failed"
        out[name] = {"state": st, "default": row["default"], "last_op_long": last and {k: last.get(k) for k in ("passed", "mean_rel_diff", "steps")}}
        counts[st] += 1
    return {"passed": counts["inconsistent"] == 0 and counts["failed"] == 0, "counts": counts, "ops": out}


def op_long(name: str, config: str, steps: int = 200, window: tuple[int, int] = (101, 201), threshold: float | None = None,
            nproc: int = 1, out_dir: str | None = None, version: str | None = None, timeout_s: float = 3600.0,
            extra_sets: list[str] | None = None) -> dict:
    """Two child runs of the training entry point: candidate = ``OP_<NAME>=<version>`` with every other op at ``baseline``;
    reference = every op at ``baseline``.  The verdict reads only the two logs."""
    from ..gates import verdicts as V
    reg = load_registry()
    ent = reg.get("ops", {}).get(name)
    if ent is None:
        return {"passed": False, "reason": f"unknown op {name!r}"}
    version = version or ent["default"]
    if version not in ent["available"]:
        return {"passed": False, "reason": f"op {name!r} has no version {version!r}"}
    threshold = threshold if threshold is not None else reg.get("automation", {}).get("rel_diff_threshold", 0.01)
    out_dir = out_dir or os.path.join(ROOT, ".artifacts", "runs", f"op-long-{name}")
    os.makedirs(out_dir, exist_ok=True)
    base_env = dict(os.environ, FORGE_ALLOW_BASELINE="1")
    for n in OP_NAMES:
        base_env["OP_" + n.upper().rstrip("_")] = "baseline"
    cand_env = dict(base_env)
    cand_env[ent["env_var"]] = version
    launch = [sys.executable, "-m", "forge_train_harness_b200.train"] if nproc == 1 else \
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
         "--master-port", str(29700 + os.getpid() % 200), "-m", "forge_train_harness_b200.train"]
    sets = [f"train.num_steps={steps}", "train.cuda_graph=false"] + list(extra_sets or [])
    argv = launch + ["--config", config] + [x for s in sets for x in ("--set", s)]
    logs = {}
    with gpu_lock(exclusive=True):
        for side, env in (("ref", base_env), ("ours", cand_env)):
            try:
                p = subprocess.run(argv, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout_s)
                text, rc = p.stdout, p.returncode
                err = p.stderr[-4000:]
            except subprocess.TimeoutExpired as e:
                text, rc, err = (e.stdout or b"").decode(errors="replace") if isinstance(e.stdout, bytes) else (e.stdout or ""), -9, "timeout"
            with open(os.path.join(out_dir, f"{side}.log"), "w") as f:
                f.write(text + "\n--- stderr ---\n" + err)
            logs[side] = (text, rc)
            if rc != 0:
                res = {"passed": False, "op": name, "version": version, "reason": f"{side} run exited with status {rc}",
                       "failure_class": V.classify_failure(text + err, rc == -9)}
                _record(name, res)
                return res
    r = V.long_train(wire.parse_loss_lines(logs["ref"][0], strict=False), wire.parse_loss_lines(logs["ours"][0], strict=False),
                     window, threshold)
    res = dict(r, op=name, version=version, steps=steps, window=list(window), run_dir=out_dir)
    _record(name, res)
    return res


def _record(name: str, res: dict) -> None:
    """Last result per op, plus a running count of consecutive failed ``op-long`` runs (reset by a pass)."""
    os.makedirs(_results_dir(), exist_ok=True)
    path = os.path.join(_results_dir(), f"{name}.json")
    fails = 0
    if os.path.isfile(path):
        try:
            with open(path) as f:
                fails = int(json.load(f).get("consecutive_failures", 0))
        except (json.JSONDecodeError, ValueError, OSError):
            fails = 0
    fails = 0 if res.get("passed") else fails + 1
    with open(path, "w") as f:
        json.dump(dict({k: v for k, v in res.items() if k != "step_diffs"}, consecutive_failures=fails), f, indent=1)


def op_long_failures(name: str) -> int:
    path = os.path.join(_results_dir(), f"{name}.json")
    try:
        with open(path) as f:
            return int(json.load(f).get("consecutive_failures", 0))
    except (FileNotFoundError, json.JSONDecodeError, ValueError):
        return 0


def fan_out(worker_argv: list[str], ops: list[str] | None = None, max_concurrent: int | None = None,
            max_failures: int | None = None, timeout_s: float = 4 * 3600.0, log_dir: str | None = None) -> dict:
    """One worker process per operator, at most ``[automation].max_concurrent`` at a time (the reference's stage-2 main agent
    fans its sub-agents out the same way, tools/stage2_config.py, config [automation.stage2]).  ``worker_argv`` is a command
    template; ``{op}`` is replaced by the operator's name and ``OP_NAME`` is exported.  Operators whose last
    ``[automation].max_op_long_failures`` op-long runs all failed are skipped as ``exhausted`` — the safety net that stops a
    worker from burning GPU time on the same broken kernel round after round.  Workers share the GPU through ``gpu_lock``."""
    reg = load_registry()
    auto = reg.get("automation", {})
    max_concurrent = int(max_concurrent if max_concurrent is not None else auto.get("max_concurrent", 6))
    max_failures = int(max_failures if max_failures is not None else auto.get("max_op_long_failures", 3))
    names = list(ops) if ops else sorted(reg.get("ops", {}))
    unknown = [n for n in names if n not in reg.get("ops", {})]
    if unknown:
        raise KeyError(f"unknown operators: {unknown}")
    log_dir = log_dir or os.path.join(ROOT, ".artifacts", "stage2", "workers")
    os.makedirs(log_dir, exist_ok=True)
    result = {n: {"state": "exhausted", "failures": op_long_failures(n)} for n in names if op_long_failures(n) >= max_failures}
    todo = [n for n in names if n not in result]
    running: dict[str, tuple] = {}
    import time
    peak = 0
    while todo or running:
        while todo and len(running) < max(1, max_concurrent):
            n = todo.pop(0)
            lg = open(os.path.join(log_dir, f"{n}.log"), "ab")
            p = subprocess.Popen([a.replace("{op}", n) for a in worker_argv], cwd=ROOT, env=dict(os.environ, OP_NAME=n),
                                 stdin=subprocess.DEVNULL, stdout=lg, stderr=subprocess.STDOUT, start_new_session=True)
            running[n] = (p, lg, time.monotonic())
            peak = max(peak, len(running))
        for n, (p, lg, t0) in list(running.items()):
            rc = p.poll()
            if rc is None and time.monotonic() - t0 > timeout_s:
                with contextlib.suppress(ProcessLookupError):
                    os.killpg(p.pid, 15)   # the exact group this worker was started in
                try:
                    rc = p.wait(timeout=10)
                except subprocess.TimeoutExpired:
                    with contextlib.suppress(ProcessLookupError):
                        os.killpg(p.pid, 9)
                    rc = p.wait()
                rc = 124
            if rc is not None:
                lg.close()
                result[n] = {"state": "done" if rc == 0 else "failed", "rc": rc, "failures": op_long_failures(n)}
                del running[n]
        if running:
            time.sleep(0.05)
    return {"passed": all(r["state"] == "done" for r in result.values()), "max_concurrent": max_concurrent, "peak_running": peak,
            "ops": result}


def as_result(suite: str, r: dict) -> dict:
    metrics = {k: v for k, v in r.items() if k not in ("ops", "problems", "step_diffs")}
    return RS.make_run_result(suite, bool(r.get("passed")), f"{suite}: {'PASS' if r.get('passed') else 'FAIL'}", metrics,
                              {k: r[k] for k in ("ops", "problems") if k in r})
