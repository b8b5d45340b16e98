"""Gate verdicts: file- and record-based judgments over ``[LOSS]`` trajectories and hash dumps.

The ladder mirrors the reference's (evals/verdicts/*.py, config/eval/dense_training/gate_config/*.toml):

* ``align``        forward-/backward-align: every overlapping hash equal, at least one overlap, baseline-authoritative
                   for backward keys (verdicts/align.py:1-20, _capture_diff.py:212-248)
* ``bitwise``      multistep / perf-bitwise: per-step ``abs diff == 0`` on loss and grad-norm (+ hashes, + MFU floor)
                   (verdicts/bitwise.py:163-241)
* ``tolerance``    the same trajectory compare with an absolute / relative budget — the single-card gate a B200 engine
                   with its own GEMM and attention kernels can be held to
* ``long_train``   mean |ours - ref| / |ref| over a step window below a threshold, with the four-bucket drift warning
                   (verdicts/long_train.py:177-220, _common.py:1050-1154)
* ``resume``       an uninterrupted run vs save -> load -> continue: max abs diff == 0 (verdicts/resume.py:143-188)
* ``resume_startup`` ``[RESUME_STARTUP] seconds=`` within a budget (evals/resume_startup_gate.py:45-135)
* ``wsd_sft``      three-phase stable -> decay -> sft structure and per-phase trajectory equality (verdicts/wsd_sft.py)
* ``production``   every expected checkpoint directory exists and is complete (verdicts/production.py)
"""
from __future__ import annotations

import os
import re
from typing import Any

from ..utils import wire
from . import capture as cap


def by_step(records) -> dict[int, wire.LossRecord]:
    return {r.step: r for r in records}


def window_loss_diff_metrics(baseline: dict[int, float], ours: dict[int, float], steps) -> dict[str, Any]:
    rel, signed, rows = [], [], []
    for s in steps:
        b, o = baseline[s], ours[s]
        if abs(b) < 1e-12:
            raise ValueError(f"baseline loss is 0 at step {s}")
        d = o - b
        rel.append(abs(d) / abs(b))
        signed.append(d)
        rows.append({"step": s, "our_loss": o, "baseline_loss": b, "rel_diff": abs(d) / abs(b), "signed_diff": d})
    if not rel:
        raise ValueError("no comparable steps in gate window")
    buckets, warning = [], None
    n = len(rows)
    if n >= 20:
        chunk = n // 4
        for i in range(4):
            sl = rows[i * chunk:(i + 1) * chunk if i < 3 else n]
            sm = sum(r["signed_diff"] for r in sl) / len(sl)
            mag = sum(abs(r["baseline_loss"]) for r in sl) / len(sl)
            buckets.append({"step_range": [sl[0]["step"], sl[-1]["step"]], "signed_mean": sm,
                            "rel_to_baseline": abs(sm) / max(mag, 1e-12)})
        if buckets[-1]["rel_to_baseline"] > 0.01:
            warning = (f"signed_mean={buckets[-1]['signed_mean']:+.4f} is {buckets[-1]['rel_to_baseline'] * 100:.2f}% of the "
                       "late-window |baseline|: systematic bias")
        else:
            sg = [b["signed_mean"] for b in buckets]
            if all(x > 0 for x in sg) and sg[3] > 1.5 * sg[0]:
                warning = "signed_mean grows monotonically positive across the window (compounding bias)"
            elif all(x < 0 for x in sg) and sg[3] < 1.5 * sg[0]:
                warning = "signed_mean grows monotonically negative across the window (compounding bias)"
    mean_base = sum(abs(r["baseline_loss"]) for r in rows) / n
    return {"compared_steps": n, "mean_rel_diff": sum(rel) / n, "max_rel_diff": max(rel),
            "signed_mean": sum(signed) / n, "signed_mean_rel": (sum(signed) / n) / mean_base,
            "step_diffs": rows, "buckets": buckets, "drift_warning": warning}


def long_train(ref_records, our_records, window: tuple[int, int], loss_rel_threshold: float = 0.01,
               mfu_floor: float | None = None) -> dict:
    ref, ours = by_step(ref_records), by_step(our_records)
    steps = [s for s in range(window[0], window[1]) if s in ref and s in ours]
    if len(steps) < (window[1] - window[0]):
        return {"passed": False, "reason": f"only {len(steps)} of {window[1] - window[0]} window steps present"}
    m = window_loss_diff_metrics({s: ref[s].loss for s in steps}, {s: ours[s].loss for s in steps}, steps)
    ok = m["mean_rel_diff"] < loss_rel_threshold
    out = {"passed": ok, "mean_rel_diff": m["mean_rel_diff"], "max_rel_diff": m["max_rel_diff"],
           "signed_mean_rel": m["signed_mean_rel"], "drift_warning": m["drift_warning"], "threshold": loss_rel_threshold}
    mfus = [ours[s].mfu for s in steps if ours[s].mfu is not None]
    if mfus:
        # always reported (the MFU history and the review-side elastic bar read it); it only GATES when a floor is given
        out["avg_mfu_e2e_standard"] = sum(mfus) / len(mfus)
    if mfu_floor is not None:
        out["mfu_avg"] = sum(mfus) / max(len(mfus), 1)
        out["mfu_target"] = mfu_floor
        out["passed"] = ok and out["mfu_avg"] >= mfu_floor
    return out


def trajectory(ref_records, our_records, window: tuple[int, int] | None = None, atol: float = 0.0, rtol: float = 0.0,
               check_grad_norm: bool = True) -> dict:
    """``atol = rtol = 0`` is the bitwise rule (max abs diff == 0); anything else is the tolerance gate.  With a window,
    EVERY step of ``[window[0], window[1])`` must be present on both sides (a run that printed one step and died must not
    pass; the reference compares over the whole gate window, verdicts/resume.py:143-188); without one, the steps both
    sides have are compared."""
    ref, ours = by_step(ref_records), by_step(our_records)
    steps = sorted(set(ref) & set(ours))
    if window:
        want = list(range(window[0], window[1]))
        missing_ref = [s for s in want if s not in ref]
        missing_ours = [s for s in want if s not in ours]
        if missing_ref or missing_ours:
            return {"passed": False, "reason": f"window [{window[0]}, {window[1]}) incomplete: baseline lacks "
                                               f"{len(missing_ref)} step(s), candidate lacks {len(missing_ours)}",
                    "missing_baseline_steps": missing_ref[:20], "missing_candidate_steps": missing_ours[:20]}
        steps = want
    if not steps:
        return {"passed": False, "reason": "no overlapping steps"}
    worst_l = worst_g = 0.0
    ok = True
    for s in steps:
        dl = abs(ref[s].loss - ours[s].loss)
        worst_l = max(worst_l, dl)
        ok &= dl <= atol + rtol * abs(ref[s].loss)
        if check_grad_norm:
            dg = abs(ref[s].grad_norm - ours[s].grad_norm)
            worst_g = max(worst_g, dg)
            ok &= dg <= atol + rtol * abs(ref[s].grad_norm)
    return {"passed": bool(ok), "steps": len(steps), "max_abs_loss_diff": worst_l, "max_abs_grad_norm_diff": worst_g}


def align(ref_dump: str, our_dump: str, family: str, backward: bool = False) -> dict:
    """``family`` is a key fragment such as ``.fwd.`` or ``.grad.``."""
    r = cap.diff_captures(cap.load_merged(ref_dump), cap.load_merged(our_dump), prefix=family,
                          require_baseline_complete=backward)
    return r


def align_tolerance(ref_file: str, our_file: str, family: str, rel_tol: float, fit_scale: bool = False,
                    scales: dict | None = None) -> dict:
    """forward-/backward-align against a stack whose kernels differ: both files are ``torch.save`` dicts of captured tensors
    (``baseline/ref_capture_bridge.py`` on the reference side, ``CaptureSession(mode="tensor")`` on this side); every key of
    ``family`` (``fwd`` | ``bwd`` | ``grad`` | ``loss``) both sides have must agree to a relative L2 error of ``rel_tol`` (and 25 x that for the largest element, relative to the reference's RMS)."""
    import torch
    ours: dict = {}
    import glob
    files = sorted(glob.glob(our_file + ".rank*")) or [our_file]
    for fn in files:
        ours.update(torch.load(fn, map_location="cpu", weights_only=True))
    ref = torch.load(ref_file, map_location="cpu", weights_only=True)
    r = cap.diff_tensors(ref, ours, family=family, rel_tol=rel_tol, fit_scale=fit_scale, scales=scales)
    worst = sorted(((v.get("rel_l2", float("inf")), k) for k, v in r["per_key"].items()), reverse=True)[:5]
    return {"passed": r["passed"], "checks_total": r["overlap"], "within_tolerance": r["overlap"] - len(r["mismatched"]),
            "worst_rel_err": r["worst_rel_err"], "rel_tol": rel_tol, "mismatched": r["mismatched"][:20],
            "worst_keys": [{"key": k, "rel_l2": e, "max_rel_err": r["per_key"][k].get("max_rel_err")} for e, k in worst],
            "family": family}


def resume(text: str, window: tuple[int, int], returncode: int | None = None) -> dict:
    """One log holding ``[LOSS_REF]`` (uninterrupted) and ``[LOSS_RES]`` (resumed) lines.  ``returncode`` is the exit
    status of the run that produced the log: a run that failed cannot pass, whatever it printed before it died."""
    ref = wire.parse_loss_lines(text, "LOSS_REF")
    res = wire.parse_loss_lines(text, "LOSS_RES")
    out = trajectory(ref, res, window)
    if returncode is not None:
        out["script_succeeded"] = returncode == 0
        if returncode != 0:
            out["passed"] = False
            out.setdefault("reason", f"the resume run exited with status {returncode}")
    return out


def resume_startup(text: str, budget_s: float) -> dict:
    m = re.search(r"\[RESUME_STARTUP\]\s+seconds=([0-9.eE+-]+)", text)
    if not m:
        return {"passed": False, "reason": "no [RESUME_STARTUP] line"}
    return {"passed": float(m[1]) <= budget_s, "seconds": float(m[1]), "budget_s": budget_s}


def wsd_sft(clean_text: str, main_text: str, phases=("stable", "decay", "sft"), atol: float = 0.0) -> dict:
    """Both logs must show the phases in order with the same start steps; per phase the trajectories must agree."""
    def split(text):
        out, cur = [], None
        for ln in text.splitlines():
            ph = wire.parse_phase_line(ln)
            if ph:
                cur = {"phase": ph, "records": []}
                out.append(cur)
                continue
            r = wire.parse_loss_line(ln, strict=False) if ln.startswith("[LOSS]") else None
            if r and cur is not None:
                cur["records"].append(r)
        return out
    a, b = split(clean_text), split(main_text)

    def merged(parts):
        m = {}
        for p in parts:  # a restarted phase prints its banner again; later records win
            d = m.setdefault(p["phase"]["name"], {"start": int(p["phase"]["start_step"]), "iwo": p["phase"]["init_weights_only"],
                                                   "records": {}})
            d["start"] = min(d["start"], int(p["phase"]["start_step"]))
            for r in p["records"]:
                d["records"][r.step] = r
        return m
    ma, mb = merged(a), merged(b)
    order_a = [n for n in dict.fromkeys(p["phase"]["name"] for p in a)]
    order_b = [n for n in dict.fromkeys(p["phase"]["name"] for p in b)]
    if order_a != list(phases) or order_b != list(phases):
        return {"passed": False, "reason": f"phase order {order_a} / {order_b}, expected {list(phases)}"}
    detail = {}
    ok = True
    for name in phases:
        if ma[name]["start"] != mb[name]["start"] or ma[name]["iwo"] != mb[name]["iwo"]:
            return {"passed": False, "reason": f"phase {name}: banner mismatch"}
        t = trajectory(list(ma[name]["records"].values()), list(mb[name]["records"].values()), atol=atol)
        t["complete"] = set(ma[name]["records"]) == set(mb[name]["records"])
        ok &= t["passed"] and t["complete"]
        detail[name] = t
    return {"passed": bool(ok), "phases": detail}


def production(save_root: str, expected_steps: list[int]) -> dict:
    from ..ckpt.manager import latest_iteration
    missing = []
    for s in expected_steps:
        d = os.path.join(save_root, f"iter_{s:07d}")
        legacy = os.path.join(save_root, f"step_{s}", "training_state.pt")
        if not (os.path.isfile(os.path.join(d, "metadata.json")) or (os.path.isfile(legacy) and os.path.getsize(legacy) > 0)):
            missing.append(s)
    return {"passed": not missing, "missing": missing, "latest": latest_iteration(save_root)}


def classify_failure(text: str, timed_out: bool = False) -> str:
    """Coarse failure classes of a side run (evals/_common.py:1162-1226)."""
    if timed_out:
        return "timeout"
    t = text.lower()
    if "no such file" in t and ("data" in t or ".bin" in t or ".idx" in t):
        return "data_missing"
    if "nccl" in t or "address already in use" in t or "connection refused" in t:
        return "network"
    if "out of memory" in t or "nan" in t or "traceback" in t:
        return "training_failure"
    if "command not found" in t or "permission denied" in t:
        return "script_setup"
    return "unknown"


def profile(run_dir: str, require_kernels: bool = True, rank: int = 0) -> dict:
    """Verdict of the ``profile-snapshot`` suite (evals/verdicts/profile.py; tools/profile_render.py:381-404): the one-step
    profile of ``rank`` exists and parses, names at least one device kernel (unless the run had no GPU), and is compared with
    the newest earlier snapshot of the same suite: step span, busy share and the kernels that moved most."""
    import glob
    import json
    import os
    found = sorted(glob.glob(os.path.join(run_dir, "ours", "profile", f"step_*_rank{rank}.json")))
    if not found:
        return {"passed": False, "reason": f"no step_*_rank{rank}.json under {os.path.join(run_dir, 'ours', 'profile')}"}
    try:
        with open(found[-1]) as f:
            cur = json.load(f)
    except (OSError, json.JSONDecodeError) as e:
        return {"passed": False, "reason": f"unreadable snapshot: {e}"}
    kernels = cur.get("kernels", {})
    out = {"passed": bool(kernels) or not require_kernels, "snapshot": found[-1], "n_kernels": len(kernels),
           "n_launches": cur.get("n_launches", 0), "span_ms": cur.get("span_us", 0.0) / 1e3,
           "busy_pct": 100.0 * cur.get("busy_us", 0.0) / max(cur.get("span_us", 0.0), 1e-9),
           "top": [[k, round(v["us"] / 1e3, 3)] for k, v in list(kernels.items())[:5]]}
    if not out["passed"]:
        out["reason"] = "the snapshot names no device kernel"
    # newest earlier snapshot of the same suite (run directories are <suite>-<utc stamp>-<id>, so names sort by time)
    parent, me = os.path.dirname(os.path.abspath(run_dir)), os.path.basename(os.path.abspath(run_dir))
    suite = me.rsplit("-", 2)[0] if me.count("-") >= 2 else me
    older = [d for d in sorted(os.listdir(parent)) if d.startswith(suite + "-") and d < me] if os.path.isdir(parent) else []
    for d in reversed(older):
        prev_files = sorted(glob.glob(os.path.join(parent, d, "ours", "profile", f"step_*_rank{rank}.json")))
        if prev_files:
            try:
                with open(prev_files[-1]) as f:
                    prev = json.load(f)
            except (OSError, json.JSONDecodeError):
                continue
            moved = sorted(((k, (v["us"] - prev["kernels"].get(k, {"us": 0.0})["us"]) / 1e3) for k, v in kernels.items()),
                           key=lambda kv: -abs(kv[1]))[:5]
            out["previous"] = prev_files[-1]
            out["delta_span_ms"] = (cur.get("span_us", 0.0) - prev.get("span_us", 0.0)) / 1e3
            out["moved_most_ms"] = [[k, round(dv, 3)] for k, dv in moved]
            break
    return out
