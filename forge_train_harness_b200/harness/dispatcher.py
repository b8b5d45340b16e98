"""Gate dispatcher: the generic three-step executor (reference side -> this engine's side -> verdict).

Mirrors evals/dispatcher.py:159-331: (1) when the gate needs a reference trajectory, look it up in a content-addressed cache
keyed by sha256 over the side command, the bytes of every script it names, the product bytes and an environment fingerprint;
on a miss run the reference side under a wall-clock budget with process-group kill, and store its run directory; (2) run this
engine's side the same way; (3) call the verdict, which only reads files from the run directory.  A side that times out or
exits non-zero yields a structured failed result with a failure class (timeout / data_missing / network / training_failure /
script_setup / unknown), never an exception.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import sys

from ..gates import verdicts as V
from ..runtime.launcher import BoundedTimeout, run_bounded
from ..utils import wire
from . import run_schema as RS

ROOT_DIR = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _subst(argv, ctx):
    return [a.format(**ctx) for a in argv]


def cache_key(argv: list[str], product_bytes: bytes, env_fingerprint: dict) -> str:
    h = hashlib.sha256()
    for a in argv:
        h.update(a.encode() + b"\0")
        if os.path.isfile(a):
            h.update(open(a, "rb").read())
    h.update(product_bytes)
    h.update(json.dumps(env_fingerprint, sort_keys=True).encode())
    return h.hexdigest()


def _run_side(argv, log_path, timeout_s, env=None, cwd=None):
    os.makedirs(os.path.dirname(log_path), exist_ok=True)
    try:
        rc, out = run_bounded(argv, timeout_s, env=env, cwd=cwd)
        timed_out = False
    except BoundedTimeout as e:
        rc, out, timed_out = -1, str(e), True
    with open(log_path, "w") as f:
        f.write(out)
    return rc, out, timed_out


def _verdict(kind: str, gate: dict, run_dir: str, ours_rc: int | None = None) -> tuple[bool, dict]:
    ref_log = os.path.join(run_dir, "ref", "ref.log")
    our_log = os.path.join(run_dir, "ours", "ours.log")
    rd = lambda p: open(p).read() if os.path.isfile(p) else ""  # noqa: E731  (missing artefacts read as empty = failed)
    if kind == "long_train":
        r = V.long_train(wire.parse_loss_lines(rd(ref_log), strict=False), wire.parse_loss_lines(rd(our_log), strict=False),
                         tuple(gate["gate_window"]), gate.get("loss_rel_threshold", 0.01), gate.get("mfu_e2e_target"))
    elif kind == "loss_gate":
        # the loss-gate-200 rule (evals/verdicts/loss_gate.py): window-average relative loss difference below a threshold that
        # MUST be given (a missing key raises instead of silently passing); the window's mean MFU is reported, never gated
        r = V.long_train(wire.parse_loss_lines(rd(ref_log), strict=False), wire.parse_loss_lines(rd(our_log), strict=False),
                         tuple(gate["gate_window"]), float(gate["max_avg_relative_loss_diff"]))
    elif kind == "trajectory":
        r = V.trajectory(wire.parse_loss_lines(rd(ref_log), strict=False), wire.parse_loss_lines(rd(our_log), strict=False),
                         tuple(gate["gate_window"]) if "gate_window" in gate else None, gate.get("atol", 0.0), gate.get("rtol", 0.0))
    elif kind == "align":
        r = V.align(os.path.join(run_dir, "ref", "ref_hash_dump.json"), os.path.join(run_dir, "ours", "ours_hash_dump.json"),
                    gate.get("family", ".fwd."), gate.get("backward", False))
        r = {"passed": r["passed"], "checks_total": r["overlap"], "bitwise_match": r["overlap"] - len(r["mismatched"]),
             "hash_capture_level": gate.get("hash_capture_level", 2), "mismatched": r["mismatched"][:20]}
    elif kind == "align_tolerance":
        sc = os.path.join(run_dir, "ours", "scales.json")   # known constant factors between the two sides' capture points
        r = V.align_tolerance(os.path.join(run_dir, "ours", "ref_capture.pt"), os.path.join(run_dir, "ours", "ours_capture.pt"),
                              gate.get("family", "fwd"), gate.get("rel_tol", 1e-2), gate.get("fit_scale", False),
                              json.load(open(sc)) if os.path.isfile(sc) else None)
    elif kind == "op_long":
        from . import stage2
        r = stage2.op_long(gate["op"], os.path.join(ROOT_DIR, gate["config"]), int(gate.get("steps", 200)),
                           tuple(gate.get("gate_window", (101, 201))), out_dir=os.path.join(run_dir, "op_long"))
    elif kind == "resume":
        r = V.resume(rd(our_log), tuple(gate["gate_window"]), returncode=ours_rc)
    elif kind == "resume_startup":
        r = V.resume_startup(rd(our_log), gate.get("resume_startup_budget_s", 18.0))
    elif kind == "wsd_sft":
        r = V.wsd_sft(rd(ref_log), rd(our_log))
    elif kind == "profile":
        r = V.profile(run_dir, bool(gate.get("require_kernels", True)))
    elif kind == "exit_code":
        # the runner judged itself (it exited 0, or run_suite would not have come here); its last JSON line, if any, is kept
        r = {"passed": ours_rc == 0}
        for ln in reversed(rd(our_log).strip().splitlines()[-20:]):
            if ln.startswith("{"):
                try:
                    r.update({k: v for k, v in json.loads(ln).items() if k != "passed"})
                    break
                except json.JSONDecodeError:
                    continue
    elif kind == "production":
        r = V.production(os.path.join(run_dir, gate.get("ckpt_subdir", os.path.join("ours", "ckpt"))), gate["expected_steps"])
    else:
        raise KeyError(f"unknown verdict {kind!r}")
    return bool(r.get("passed")), r


def run_suite(request: dict, registry: dict, repo_root: str, artifact_dir: str, cache_dir: str | None = None) -> dict:
    RS.validate_run_request(request)
    suite = request["suite"]
    gate = registry.get("evals", {}).get(suite)
    if gate is None:
        return RS.make_failed_result(suite, f"unknown suite {suite!r}", "script_setup")
    os.makedirs(artifact_dir, exist_ok=True)
    ctx = {"python": sys.executable, "run_dir": artifact_dir, "repo": repo_root, "suite": suite}
    ctx.update({k: str(v) for k, v in request.get("args", {}).items()})
    timeout_s = float(request.get("args", {}).get("timeout_s", gate.get("timeout_s", 600)))
    env_fp = {k: os.environ.get(k, "") for k in registry.get("env_fingerprint", [])}
    details = {"run_dir": artifact_dir}
    if gate.get("needs_ref", False):
        argv = _subst(gate["ref_cmd"], ctx)
        key = cache_key(argv, json.dumps(gate, sort_keys=True).encode(), env_fp)
        hit = os.path.join(cache_dir, key) if cache_dir else None
        ref_dir = os.path.join(artifact_dir, "ref")
        if hit and os.path.isfile(os.path.join(hit, "ref.log")):
            shutil.copytree(hit, ref_dir, dirs_exist_ok=True)
            details["ref_cache"] = "hit"
        else:
            rc, out, to = _run_side(argv, os.path.join(ref_dir, "ref.log"), timeout_s, cwd=repo_root)
            if rc != 0:
                return RS.make_run_result(suite, False, f"reference side failed (rc {rc})", {},
                                          dict(details, failure_class=V.classify_failure(out, to), side="ref"))
            if hit:
                shutil.copytree(ref_dir, hit, dirs_exist_ok=True)
            details["ref_cache"] = "miss"
    ours_rc = None
    if gate.get("ours_cmd"):
        rc, out, to = _run_side(_subst(gate["ours_cmd"], ctx), os.path.join(artifact_dir, "ours", "ours.log"), timeout_s, cwd=repo_root)
        if rc != 0:
            return RS.make_run_result(suite, False, f"engine side failed (rc {rc})", {},
                                      dict(details, failure_class=V.classify_failure(out, to), side="ours"))
        ours_rc = rc
    ok, metrics = _verdict(gate["verdict"], gate, artifact_dir, ours_rc)
    metrics = {k: v for k, v in metrics.items() if k != "step_diffs"}
    res = RS.make_run_result(suite, ok, f"{suite}: {'PASS' if ok else 'FAIL'}", metrics, details)
    with open(os.path.join(artifact_dir, "result.json"), "w") as f:
        json.dump(res, f, indent=1)
    return res
