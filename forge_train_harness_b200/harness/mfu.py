"""MFU history and the elastic throughput bar.

``record`` appends one JSON line per finished gate run to ``mfu_history.jsonl`` (tools/mfu_record.py:33-95).  ``evaluate``
decides a bar ``T`` the way the reference's review-side checker does (tools/mfu_elastic_check.py:224-250): strict pass if the
newest qualifying average is >= T; elastic pass if the last N qualifying runs are all >= T - tolerance and their spread is <=
eps (a plateau, not a lucky sample); otherwise fail.  Only full ``long-train`` runs whose loss verdict did not fail qualify.
"""
from __future__ import annotations

import json
import os
import time


def record(path: str, suite: str, mfu: float, loss_passed: bool | None, extra: dict | None = None) -> dict:
    row = {"ts": time.time(), "suite": suite, "mfu_avg": float(mfu), "loss_passed": loss_passed}
    row.update(extra or {})
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "a") as f:
        f.write(json.dumps(row) + "\n")
    return row


def history_path(env: dict | None = None) -> str | None:
    """Where a gate run's MFU sample belongs: the loop's own directory (``FORGE_LOOP_DIR``, exported to every worker and job
    of a development loop), else an explicit ``FORGE_MFU_HISTORY`` file, else nowhere."""
    env = os.environ if env is None else env
    if env.get("FORGE_MFU_HISTORY"):
        return env["FORGE_MFU_HISTORY"]
    if env.get("FORGE_LOOP_DIR"):
        return os.path.join(env["FORGE_LOOP_DIR"], "mfu_history.jsonl")
    return None


def record_result(result: dict, env: dict | None = None, out=None) -> dict | None:
    """Append the MFU sample of a finished gate run, if it measured one (tools/mfu_record.py:33-95; called by the runner after
    every suite, evals/runner.py:115).  Never raises and never changes the gate's verdict; a run that measured MFU but has no
    history to go to says so on stderr, because the review-side bar silently starves otherwise."""
    import sys
    out = out or sys.stderr
    metrics = result.get("metrics") or {}
    avg = metrics.get("avg_mfu_e2e_standard")
    if avg is None:
        return None
    path = history_path(env)
    if path is None:
        print("mfu_record: SKIPPED, no loop directory (set FORGE_LOOP_DIR or FORGE_MFU_HISTORY); this run will be missing "
              "from the MFU history", file=out)
        return None
    loss_passed = None if "mean_rel_diff" not in metrics else bool(metrics["mean_rel_diff"] < metrics.get("threshold", 0.01))
    try:
        return record(path, str(result.get("suite") or ""), float(avg), loss_passed,
                      {"mfu_target": metrics.get("mfu_target"), "status": result.get("status")})
    except OSError as e:
        print(f"mfu_record: persist failed: {e}", file=out)
        return None


def load(path: str) -> list[dict]:
    if not os.path.isfile(path):
        return []
    rows = []
    for ln in open(path):
        ln = ln.strip()
        if ln:
            try:
                rows.append(json.loads(ln))
            except json.JSONDecodeError:
                continue
    return rows


def qualifying(rows: list[dict], suite: str = "long-train") -> list[float]:
    return [r["mfu_avg"] for r in rows if r.get("suite") == suite and r.get("loss_passed") is not False]


def evaluate(samples: list[float], target: float, tolerance: float = 2.0, rounds: int = 3, eps: float = 0.5) -> tuple[bool, str]:
    if not samples:
        return False, "NO_QUALIFYING_RUNS"
    if samples[-1] >= target:
        return True, "STRICT_PASS"
    if samples[-1] < target - tolerance:
        return False, "BELOW_BAND"
    if len(samples) < rounds:
        return False, "IN_BAND_INSUFFICIENT_HISTORY"
    win = samples[-rounds:]
    if all(s >= target - tolerance for s in win) and max(win) - min(win) <= eps:
        return True, "ELASTIC_PASS"
    return False, "IN_BAND_UNSTABLE"
