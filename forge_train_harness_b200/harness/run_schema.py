"""Run request / result documents exchanged between the harness CLI and the gate dispatcher.

Same envelope as the reference (harness/run_schema.py:18-41): a request JSON goes in, a result JSON comes back on stdout
between ``---HARNESS-RESULT-BEGIN---`` / ``---HARNESS-RESULT-END---`` markers, with ``status`` in {passed, failed}, a
one-line ``summary``, a ``metrics`` table whose minimal keys are fixed per verdict kind, and free-form ``details``.
"""
from __future__ import annotations

import json
import time
import uuid

RESULT_BEGIN = "---HARNESS-RESULT-BEGIN---"
RESULT_END = "---HARNESS-RESULT-END---"
RUN_SCHEMA_VERSION = 1
_REQUEST_KEYS = {"schema_version", "run_id", "suite", "args", "gpu_count", "artifact_relpath", "requested_at", "workload_config"}
_RESULT_KEYS = {"schema_version", "status", "suite", "summary", "metrics", "details"}

# minimal metric keys per verdict kind (lower bound; extra keys are allowed)
RUNNER_METRICS = {
    "align": ["checks_total", "bitwise_match", "hash_capture_level"],
    "trajectory": ["steps", "max_abs_loss_diff", "max_abs_grad_norm_diff"],
    "long_train": ["mean_rel_diff", "max_rel_diff", "threshold"],
    "resume": ["steps", "max_abs_loss_diff", "max_abs_grad_norm_diff"],
    "resume_startup": ["seconds", "budget_s"],
    "wsd_sft": ["phases"],
    "production": ["missing"],
    "align_tolerance": ["checks_total", "within_tolerance", "worst_rel_err", "rel_tol"],
    "op_long": ["mean_rel_diff", "max_rel_diff", "threshold"],
}


def make_run_request(suite: str, args: dict | None = None, gpu_count: int = 1, workload_config: dict | None = None) -> dict:
    rid = f"{suite}-{time.strftime('%Y%m%dT%H%M%S')}-{uuid.uuid4().hex[:6]}"
    return {"schema_version": RUN_SCHEMA_VERSION, "run_id": rid, "suite": suite, "args": args or {}, "gpu_count": gpu_count,
            "artifact_relpath": f".artifacts/runs/{rid}", "requested_at": time.time(), "workload_config": workload_config or {}}


def validate_run_request(req: dict) -> None:
    missing = _REQUEST_KEYS - set(req)
    if missing:
        raise ValueError(f"run request lacks {sorted(missing)}")
    rel = req["artifact_relpath"]
    if rel.startswith("/") or ".." in rel.split("/"):
        raise ValueError("artifact_relpath must be a safe relative path")


def make_run_result(suite: str, passed: bool, summary: str, metrics: dict, details: dict | None = None) -> dict:
    return {"schema_version": RUN_SCHEMA_VERSION, "status": "passed" if passed else "failed", "suite": suite,
            "summary": summary, "metrics": metrics, "details": details or {}}


def make_failed_result(suite: str, reason: str, failure_class: str = "unknown") -> dict:
    return make_run_result(suite, False, reason, {}, {"failure_class": failure_class})


def validate_run_result(res: dict, kind: str | None = None) -> None:
    missing = _RESULT_KEYS - set(res)
    if missing:
        raise ValueError(f"run result lacks {sorted(missing)}")
    if res["status"] not in ("passed", "failed"):
        raise ValueError("status must be passed or failed")
    if kind and res["status"] == "passed":
        lack = [k for k in RUNNER_METRICS.get(kind, []) if k not in res["metrics"]]
        if lack:
            raise ValueError(f"result of kind {kind!r} lacks metrics {lack}")


def emit_result(res: dict, out) -> None:
    out.write(f"{RESULT_BEGIN}\n{json.dumps(res)}\n{RESULT_END}\n")
    out.flush()


def extract_result(text: str) -> dict | None:
    if RESULT_BEGIN not in text or RESULT_END not in text:
        return None
    body = text.split(RESULT_BEGIN, 1)[1].split(RESULT_END, 1)[0]
    return json.loads(body)
