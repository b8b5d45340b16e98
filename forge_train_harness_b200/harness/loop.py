"""Round-based development loop: lease GPUs, run a worker per round, review, advance milestones, record events, report.

The reference drives its coding agents with ``agent-loop.sh`` (agent-loop.sh:677-1054, 1517-1826, 1971-2100) plus the helpers
``tools/agent_loop_milestone.sh`` (milestone state I/O), ``tools/agent_loop_retry.sh`` (retry decision),
``tools/loop_wrapper_event.py`` (typed event stream) and ``tools/loop_report.py`` (offline report).  The contract kept here:

* **Stages and milestones.**  Stage 1 walks a linear, named milestone order read from the suite registry
  (``[stage1].milestone_order``); the active milestone is one line in ``<state>/stage1.milestone``; a restart resumes from
  the first stage that is not ``finished``.
* **A round** = one worker run (any command: a coding agent CLI, a script, a person's shell) with a wall-clock cap, then an
  optional review command.  A worker that fails is retried unless its exit code says stop (130 / 143 / 137 = a signal, 64 /
  78 = a usage or configuration error, 124 = the round overran its cap: the workspace goes back to the round's baseline
  commit and a fresh round starts).
* **Advancing.**  The worker declares progress with a commit-message line ``MILESTONE_STATUS: <name> PASS``; after each round
  the last commits are scanned and the active milestone becomes the successor of the furthest declared one (capped at the
  last).  Milestones listed as review-gated ignore declarations and advance only when the review passes and writes
  ``MILESTONE_OVERRIDE: <active milestone>`` — or, with no review command and ``review_mfu_target`` set, when the loop's own
  review finds the throughput bar met on the MFU history the gate runs wrote.  With ``advance = "gates"`` the loop does not trust declarations at all: it
  runs the active milestone's suites itself (as short-lived GPU jobs, ``harness/jobs.py``) and advances on their verdicts.
* **Events.**  Every transition is one JSON line in ``<loop_dir>/events.jsonl``; ``report`` rebuilds the per-round table,
  the milestone table, the MFU trajectory and an error digest from files only, on a live or a dead loop.
* **Lease.**  GPUs are claimed before the first round and released on every exit path (``harness/lease.py``).

CLI::

    python -m forge_train_harness_b200.harness.loop run --config configs/loop.toml [--loop-id ID] [--max-rounds N] [--reset-state]
    python -m forge_train_harness_b200.harness.loop report <loop_dir> [--json out.json] [--md out.md]
    python -m forge_train_harness_b200.harness.loop fork --config configs/loop.toml --src-loop-id ID --at-milestone NAME [--workspace DIR]
    python -m forge_train_harness_b200.harness.loop should-retry <rc>
"""
from __future__ import annotations

import argparse
import json
import os
import re
import shlex
import signal
import subprocess
import sys
import time
import tomllib
import uuid
from dataclasses import dataclass, field

from . import jobs, lease, mfu

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
NO_RETRY_RCS = {0: "success", 130: "interrupted (SIGINT)", 143: "terminated (SIGTERM)", 137: "killed (SIGKILL)",
                64: "usage error", 78: "configuration error", 124: "round wall-clock cap exceeded"}
_DECL = re.compile(r"^MILESTONE_STATUS:[ \t]+(\S+)[ \t]+PASS[ \t]*$", re.M)
_CONTRACT = re.compile(r"^([A-Z_]+):[ \t]+(\S+)[ \t]*$", re.M)


# ---- pure helpers (the parts the reference keeps in separately tested shell files) ---------------------------------------------
def should_retry(rc: int) -> bool:
    """Retry by default on any failure; never on success, a stop signal, a usage / configuration error or a round that
    overran its cap (tools/agent_loop_retry.sh:29-80)."""
    return rc not in NO_RETRY_RCS


def classify_failure(rc: int, log_path: str | None = None) -> str:
    if rc in NO_RETRY_RCS and rc != 0:
        return f"{NO_RETRY_RCS[rc]} (rc={rc})"
    if rc == 75:
        return "temporary failure before the worker started (rc=75; transient)"
    last = ""
    if log_path and os.path.isfile(log_path):
        with open(log_path, "rb") as f:
            f.seek(0, os.SEEK_END)
            f.seek(max(0, f.tell() - 4096))
            lines = [ln for ln in f.read().decode("utf-8", "replace").splitlines() if ln.strip()]
            last = lines[-1][:200] if lines else ""
    return f"rc={rc}; last log line: {last}" if last else f"rc={rc}; no diagnostic available"


def parse_declared_milestone(commit_bodies: str, order: list[str]) -> str:
    """Furthest-along milestone named by a ``MILESTONE_STATUS: <name> PASS`` line; names outside ``order`` are ignored."""
    best = -1
    for m in _DECL.finditer(commit_bodies):
        if m.group(1) in order:
            best = max(best, order.index(m.group(1)))
    return order[best] if best >= 0 else ""


def next_milestone_after(highest: str, current: str, order: list[str]) -> str:
    """Milestone that becomes active once ``highest`` has passed: its successor, capped at the last; empty if that would
    not move ``current`` forward (tools/agent_loop_milestone.sh, same rule)."""
    if highest not in order or current not in order:
        return ""
    nxt = order[min(order.index(highest) + 1, len(order) - 1)]
    return nxt if order.index(nxt) > order.index(current) else ""


def read_contract(path: str) -> dict:
    """``KEY: value`` lines of a review status file (``REVIEW_STATUS``, ``STAGE_STATUS``, ``MILESTONE_OVERRIDE``)."""
    try:
        with open(path, encoding="utf-8") as f:
            return {k: v for k, v in _CONTRACT.findall(f.read())}
    except FileNotFoundError:
        return {}


# ---- configuration ------------------------------------------------------------------------------------------------------------
@dataclass
class LoopConfig:
    worker_cmd: list
    review_cmd: list = field(default_factory=list)
    registry: str = os.path.join(ROOT, "configs", "eval", "dense_training.toml")
    workspace: str = ROOT
    loops_dir: str = os.path.join(ROOT, ".artifacts", "loops")
    round_tries: int = 8
    round_timeout_s: float = 4 * 3600.0
    retry_backoff_s: float = 15.0
    max_rounds: int = 200
    review_gated: list = field(default_factory=lambda: ["long-horizon"])
    advance: str = "declared"  # "declared" | "gates"
    gpus: int = 0
    lease_timeout_s: float = 600.0
    rollback_on_timeout: bool = False
    remote: dict = field(default_factory=dict)
    prompt_dir: str = ""
    gate_poll_s: float = 30.0
    # built-in review of a review-gated milestone when no review command is configured: the throughput bar on the MFU history
    # the gate runs wrote (strict pass, or a plateau inside the tolerance band: harness/mfu.py).  0 = off.
    # stage 2 (per-operator work) after stage 1 has finished: one worker per operator, fanned out under the registry's
    # [automation] limits (harness/stage2.py::fan_out); {op} in the command is the operator's name.  Empty = no stage 2.
    stage2_worker_cmd: list = field(default_factory=list)
    stage2_max_rounds: int = 20
    review_mfu_target: float = 0.0
    review_suite: str = "long-train"
    mfu_elastic_tolerance: float = 2.0
    mfu_elastic_rounds: int = 3
    mfu_elastic_eps: float = 0.5

    @staticmethod
    def load(path: str) -> "LoopConfig":
        with open(path, "rb") as f:
            doc = tomllib.load(f)
        t = dict(doc.get("loop", {}))
        if not isinstance(t.get("worker_cmd"), list) or not t["worker_cmd"]:
            raise ValueError("[loop].worker_cmd must be a non-empty argv list")
        known = {f_.name for f_ in LoopConfig.__dataclass_fields__.values()}
        bad = sorted(set(t) - known)
        if bad:
            raise ValueError(f"unknown [loop] keys: {bad}")
        if t.get("advance", "declared") not in ("declared", "gates"):
            raise ValueError("[loop].advance must be 'declared' or 'gates'")
        base = os.path.dirname(os.path.abspath(path))
        for k in ("registry", "workspace", "loops_dir", "prompt_dir"):
            if t.get(k) and not os.path.isabs(t[k]):
                t[k] = os.path.normpath(os.path.join(base, t[k]))
        t["remote"] = doc.get("remote", {})
        return LoopConfig(**t)


def milestone_order(registry_path: str, stage: str = "stage1") -> list[str]:
    with open(registry_path, "rb") as f:
        doc = tomllib.load(f)
    order = (doc.get(stage) or {}).get("milestone_order") or []
    if not order or len(set(order)) != len(order):
        raise ValueError(f"[{stage}].milestone_order in {registry_path} must be a non-empty list without repeats")
    return list(order)


def suites_of_milestone(registry_path: str, milestone: str) -> list[tuple[str, dict]]:
    """Suites whose ``milestone`` is ``<milestone>`` or ``<milestone>.<part>`` (``alignment.forward`` belongs to ``alignment``)."""
    with open(registry_path, "rb") as f:
        doc = tomllib.load(f)
    out = []
    for name, gate in (doc.get("evals") or {}).items():
        ms = str(gate.get("milestone", ""))
        if ms == milestone or ms.startswith(milestone + "."):
            out.append((name, gate))
    return out


# ---- the loop -----------------------------------------------------------------------------------------------------------------
class Loop:
    def __init__(self, cfg: LoopConfig, loop_id: str | None = None, scheduler=None, out=sys.stderr):
        self.cfg = cfg
        self.loop_id = loop_id or uuid.uuid4().hex[:12]
        self.dir = os.path.join(cfg.loops_dir, self.loop_id)
        self.state_dir = os.path.join(self.dir, "state")
        os.makedirs(self.state_dir, exist_ok=True)
        self.order = milestone_order(cfg.registry)
        self.out = out
        self.scheduler = scheduler
        self._child = None
        self.exit_cause = "unknown"

    # -- state files
    def _sf(self, name: str) -> str:
        return os.path.join(self.state_dir, name)

    def _read(self, name: str, default: str = "") -> str:
        try:
            with open(self._sf(name), encoding="utf-8") as f:
                return f.read().strip() or default
        except FileNotFoundError:
            return default

    def _write(self, name: str, value: str) -> None:
        tmp = self._sf(f".{name}.tmp")
        with open(tmp, "w", encoding="utf-8") as f:
            f.write(value + "\n")
        os.replace(tmp, self._sf(name))

    def reset_state(self) -> None:
        for fn in os.listdir(self.state_dir):
            if fn.endswith((".status", ".milestone", ".round")):
                os.unlink(self._sf(fn))

    @property
    def milestone(self) -> str:
        v = self._read("stage1.milestone", self.order[0])
        if v not in self.order:
            self.event("milestone_state_invalid", value=v, text=f"stored milestone {v!r} is not in the order; using the first")
            return self.order[0]
        return v

    def event(self, subtype: str, **kw) -> dict:
        row = {"ts": time.time(), "loop_id": self.loop_id, "subtype": subtype}
        row.update(kw)
        with open(os.path.join(self.dir, "events.jsonl"), "a", encoding="utf-8") as f:
            f.write(json.dumps(row) + "\n")
        return row

    def backfill_mfu_events(self) -> int:
        """One ``mfu_record`` event per row of ``mfu_history.jsonl`` not yet seen (rows land there from gate runs, possibly
        on another host and synced back; a cursor file makes this idempotent — tools/mfu_backfill_events.py)."""
        rows = mfu.load(os.path.join(self.dir, "mfu_history.jsonl"))
        seen = int(self._read("mfu.cursor", "0"))
        for r in rows[seen:]:
            self.event("mfu_record", suite=r.get("suite"), mfu_avg=r.get("mfu_avg"), loss_passed=r.get("loss_passed"), sample_ts=r.get("ts"))
        if len(rows) != seen:
            self._write("mfu.cursor", str(len(rows)))
        return len(rows) - seen

    # -- git helpers (the workspace's history is the trajectory)
    def _git(self, *args: str) -> str:
        try:
            r = subprocess.run(["git", "-C", self.cfg.workspace, *args], capture_output=True, text=True, timeout=60)
            return r.stdout if r.returncode == 0 else ""
        except (OSError, subprocess.TimeoutExpired):
            return ""

    def head(self) -> str:
        return self._git("rev-parse", "HEAD").strip()

    # -- one worker / review process, in its own process group, with a wall-clock cap
    def _spawn(self, argv: list, ctx: dict, log_path: str, timeout_s: float) -> int:
        cmd = [str(a).format(**ctx) for a in argv]
        env = dict(os.environ, FORGE_LOOP_ID=self.loop_id, FORGE_LOOP_DIR=self.dir, FORGE_MILESTONE=ctx["milestone"],
                   FORGE_ROUND=str(ctx["round"]), FORGE_MILESTONE_ORDER=" ".join(self.order))
        env.update(ctx.get("lease_env", {}))
        with open(log_path, "ab") as lg:
            try:
                p = subprocess.Popen(cmd, cwd=self.cfg.workspace, stdin=subprocess.DEVNULL, stdout=lg, stderr=subprocess.STDOUT,
                                     start_new_session=True, env=env)
            except FileNotFoundError:
                lg.write(f"[loop] executable not found: {cmd[0]}\n".encode())
                return 78
            self._child = p
            try:
                return p.wait(timeout=timeout_s)
            except subprocess.TimeoutExpired:
                for sig, grace in ((signal.SIGTERM, 10.0), (signal.SIGKILL, 5.0)):
                    try:
                        os.killpg(p.pid, sig)  # the exact group this round started
                    except ProcessLookupError:
                        break
                    try:
                        p.wait(timeout=grace)
                        break
                    except subprocess.TimeoutExpired:
                        continue
                return 124
            finally:
                self._child = None

    def _prompt(self, rnd: int, ms: str) -> str:
        """Round prompt file: the stage's always-on notes plus the active milestone's, when a prompt directory is given."""
        path = os.path.join(self.dir, f"round_{rnd:03d}.prompt.md")
        parts = [f"# round {rnd}\n\nactive milestone: {ms}\nmilestone order: {' -> '.join(self.order)}\n"
                 f"declare a passed gate with a commit-message line `MILESTONE_STATUS: <name> PASS`\n"]
        suites = suites_of_milestone(self.cfg.registry, ms)
        if suites:
            parts.append("suites of this milestone: " + ", ".join(n for n, _ in suites) + "\n")
        pd = self.cfg.prompt_dir
        if pd and os.path.isdir(pd):
            for fn in ("overview.md", "constraint.md", f"{ms}.md"):
                fp = os.path.join(pd, fn)
                if os.path.isfile(fp):
                    with open(fp, encoding="utf-8") as f:
                        parts.append(f.read())
        with open(path, "w", encoding="utf-8") as f:
            f.write("\n".join(parts))
        return path

    # -- advancing
    def _advance_declared(self, rnd: int, review_passed: bool, review_file: str) -> None:
        cur = self.milestone
        gated = set(self.cfg.review_gated)
        if review_passed and cur in gated and read_contract(review_file).get("MILESTONE_OVERRIDE") == cur:
            nxt = next_milestone_after(cur, cur, self.order)
            if nxt:
                self._write("stage1.milestone", nxt)
                self.event("milestone_auto_advanced", round=rnd, **{"from": cur, "to": nxt, "max": self.order[-1]})
            elif cur == self.order[-1]:
                self._write("stage1.status", "finished")
                self.event("stage_finished", round=rnd, stage="stage1")
            return
        bodies = self._git("log", "-n", "50", "--format=%B")
        highest = parse_declared_milestone(bodies, self.order)
        if not highest:
            return
        if highest in gated:
            self.event("milestone_advance_withheld", round=rnd, milestone=highest, review_passed=review_passed,
                       text="review-gated milestone: declarations carry no weight; it advances only by the review's override")
            return
        if highest == self.order[-1] and self.order.index(cur) == len(self.order) - 1:
            self._write("stage1.status", "finished")
            self.event("stage_finished", round=rnd, stage="stage1")
            return
        nxt = next_milestone_after(highest, cur, self.order)
        if not nxt:
            return
        sha = ""
        for line in self._git("log", "-n", "50", "--format=%H%x00%B%x01").split("\x01"):
            h, _, body = line.strip().partition("\x00")
            if re.search(rf"^MILESTONE_STATUS:[ \t]+{re.escape(highest)}[ \t]+PASS[ \t]*$", body, re.M):
                sha = h
                break
        self._write("stage1.milestone", nxt)
        self.event("milestone_advanced", round=rnd, **{"from": cur, "to": nxt, "max": self.order[-1], "commit": sha})

    def run_stage2(self, max_rounds: int | None = None, lease_env: dict | None = None) -> int:
        """Stage 2: per round one worker per operator that is not yet ``merged`` (bounded concurrency, per-op failure budget),
        until ``op-status`` has every registered operator merged or the round limit is reached.  The reference fans its
        stage-2 sub-agents out the same way and re-fans each round (tools/stage2_config.py, agent-loop.sh)."""
        from . import stage2
        cfg = self.cfg
        if not cfg.stage2_worker_cmd:
            return 0
        if self._read("stage2.status") == "finished":
            return 0
        self._write("stage2.status", "in-progress")
        rnd = int(self._read("stage2.round", "0"))
        for _ in range(max_rounds if max_rounds is not None else cfg.stage2_max_rounds):
            rnd += 1
            self._write("stage2.round", str(rnd))
            st = stage2.op_status()
            todo = sorted(n for n, o in st["ops"].items() if o["state"] != "merged")
            self.event("stage2_round_started", round=rnd, pending=todo, counts=st["counts"])
            if not todo:
                self._write("stage2.status", "finished")
                self.event("stage_finished", round=rnd, stage="stage2")
                return 0
            argv = [str(a).format(workspace=cfg.workspace, loop_dir=self.dir, loop_id=self.loop_id, python=sys.executable, op="{op}")
                    for a in cfg.stage2_worker_cmd]
            env_before = dict(os.environ)
            os.environ.update(dict(lease_env or {}, FORGE_LOOP_ID=self.loop_id, FORGE_LOOP_DIR=self.dir, FORGE_ROUND=str(rnd)))
            try:
                res = stage2.fan_out(argv, ops=todo, timeout_s=cfg.round_timeout_s, log_dir=os.path.join(self.dir, f"stage2_round_{rnd:03d}"))
            finally:
                os.environ.clear()
                os.environ.update(env_before)
            self.event("stage2_round_finished", round=rnd, peak_running=res["peak_running"],
                       ops={n: r["state"] for n, r in res["ops"].items()})
        self.exit_cause = "stage 2 round limit reached"
        return 0

    def _builtin_review(self, rnd: int) -> bool:
        """The review the reference leaves to its review agent for the long-horizon milestone (review_stage1.md; tools/
        mfu_elastic_check.py): read the MFU history written by the gate runs, apply the elastic bar, and advance the ACTIVE
        review-gated milestone on a pass.  Returns True when it advanced."""
        cfg, cur = self.cfg, self.milestone
        if cfg.review_cmd or cfg.review_mfu_target <= 0 or cur not in cfg.review_gated:
            return False
        samples = mfu.qualifying(mfu.load(os.path.join(self.dir, "mfu_history.jsonl")), cfg.review_suite)
        ok, code = mfu.evaluate(samples, cfg.review_mfu_target, cfg.mfu_elastic_tolerance, cfg.mfu_elastic_rounds, cfg.mfu_elastic_eps)
        self.event("review_finished", round=rnd, rc=0, verdict="PASS" if ok else "FAIL",
                   contract={"by": "mfu-bar", "code": code, "samples": len(samples), "target": cfg.review_mfu_target})
        if not ok:
            return False
        if cur == self.order[-1]:
            self._write("stage1.status", "finished")
            self.event("stage_finished", round=rnd, stage="stage1")
        else:
            nxt = self.order[self.order.index(cur) + 1]
            self._write("stage1.milestone", nxt)
            self.event("milestone_auto_advanced", round=rnd, **{"from": cur, "to": nxt, "max": self.order[-1], "text": code})
        return True

    def _advance_by_gates(self, rnd: int, lease_env: dict) -> None:
        cur = self.milestone
        suites = suites_of_milestone(self.cfg.registry, cur)
        if not suites:
            self.event("milestone_has_no_suites", round=rnd, milestone=cur)
            return
        sched = self.scheduler or jobs.scheduler_from_config(self.cfg.remote)
        results = {}
        for name, gate in suites:
            outer = float(gate.get("timeout_s", 1800))
            entry = jobs.build_entry(suite=name, extra=["--registry", self.cfg.registry], loop_id=self.loop_id,
                                     workdir=self.cfg.workspace, loop_dir=self.dir)
            rc = jobs.run_suite(sched, suite=f"{self.loop_id}.{name}", entry=entry, gpus=int(gate.get("gpu_count", 0)),
                                outer=outer, poll_interval_s=self.cfg.gate_poll_s, out=self.out)
            results[name] = rc
            self.event("gate_run", round=rnd, milestone=cur, suite=name, rc=rc)
            if rc != 0:
                break
        if results and all(rc == 0 for rc in results.values()) and len(results) == len(suites):
            if cur == self.order[-1]:
                self._write("stage1.status", "finished")
                self.event("stage_finished", round=rnd, stage="stage1")
            else:
                nxt = self.order[self.order.index(cur) + 1]
                self._write("stage1.milestone", nxt)
                self.event("milestone_advanced", round=rnd, **{"from": cur, "to": nxt, "max": self.order[-1], "by": "gates"})

    # -- main
    def run(self, max_rounds: int | None = None) -> int:
        cfg = self.cfg
        provider = lease.provider_from_config(cfg.remote) if cfg.gpus or cfg.remote else None
        lease_env, handle = {}, ""
        prev_handlers = {}

        def _on_signal(signum, frame):
            self.exit_cause = f"signal {signum}"
            p = self._child
            if p is not None and p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)
                except ProcessLookupError:
                    pass
            raise KeyboardInterrupt

        for s in (signal.SIGTERM, signal.SIGINT):
            try:
                prev_handlers[s] = signal.signal(s, _on_signal)
            except ValueError:  # not the main thread (tests)
                pass
        self.event("loop_started", milestone=self.milestone, order=self.order, workspace=cfg.workspace, head=self.head())
        rc_final = 1
        try:
            if provider is not None:
                handle = lease.claim("gpu", spec=lease.LeaseSpec(cfg.gpus, dict(cfg.remote.get("labels", {}))), loop_id=self.loop_id,
                                     provider=provider, timeout=cfg.lease_timeout_s)
                lease_env = provider.env(handle)
                self.event("lease_claimed", handle=handle, gpus=cfg.gpus)
            if self._read("stage1.status") == "finished":
                self.exit_cause = "already finished"
                rc_final = self.run_stage2(max_rounds, lease_env)
                return rc_final
            self._write("stage1.status", "in-progress")
            rnd = int(self._read("stage1.round", "0"))
            limit = max_rounds if max_rounds is not None else cfg.max_rounds
            for _ in range(limit):
                rnd += 1
                self._write("stage1.round", str(rnd))
                ms = self.milestone
                base = self.head()
                t0 = time.time()
                self.event("round_started", round=rnd, milestone=ms, base=base)
                ctx = {"round": rnd, "milestone": ms, "workspace": cfg.workspace, "loop_dir": self.dir, "loop_id": self.loop_id,
                       "prompt_file": self._prompt(rnd, ms), "python": sys.executable, "lease_env": lease_env,
                       "review_file": os.path.join(self.dir, f"round_{rnd:03d}.review.status")}
                log = os.path.join(self.dir, f"round_{rnd:03d}.worker.log")
                rc, attempts = 1, 0
                for attempt in range(1, cfg.round_tries + 1):
                    attempts = attempt
                    rc = self._spawn(cfg.worker_cmd, ctx, log, cfg.round_timeout_s)
                    if rc == 0:
                        break
                    why = classify_failure(rc, log)
                    self.event("agent_failed", round=rnd, attempt=attempt, rc=rc, text=why)
                    if not should_retry(rc):
                        break
                    time.sleep(min(cfg.retry_backoff_s * attempt, 300.0))
                if rc == 124:
                    if cfg.rollback_on_timeout and base:
                        self._git("reset", "--hard", base)
                        self.event("round_rolled_back", round=rnd, to=base)
                    self.event("round_finished", round=rnd, status="timeout", attempts=attempts, duration_s=time.time() - t0)
                    continue  # a fresh round, not a retry of the wedged one
                if rc != 0:
                    self.event("round_finished", round=rnd, status="failed", attempts=attempts, rc=rc, duration_s=time.time() - t0)
                    self.exit_cause = f"worker failed: {classify_failure(rc, log)}"
                    rc_final = rc
                    return rc_final
                review_passed = True
                if cfg.review_cmd:
                    rrc = self._spawn(cfg.review_cmd, ctx, os.path.join(self.dir, f"round_{rnd:03d}.review.log"), cfg.round_timeout_s)
                    contract = read_contract(ctx["review_file"])
                    review_passed = rrc == 0 and contract.get("REVIEW_STATUS", "PASS") == "PASS"
                    self.event("review_finished", round=rnd, rc=rrc, verdict="PASS" if review_passed else "FAIL", contract=contract)
                    if contract.get("STAGE_STATUS") == "finished" and review_passed:
                        self._write("stage1.status", "finished")
                commits = [ln for ln in self._git("log", "--format=%h %s", f"{base}..HEAD").splitlines() if ln] if base else []
                if cfg.advance == "gates":
                    self._advance_by_gates(rnd, lease_env)
                else:
                    self._advance_declared(rnd, review_passed, ctx["review_file"])
                self.backfill_mfu_events()
                self._builtin_review(rnd)
                self.event("round_finished", round=rnd, status="ok", attempts=attempts, duration_s=time.time() - t0,
                           review="PASS" if review_passed else "FAIL", commits=commits, milestone_after=self.milestone)
                if self._read("stage1.status") == "finished":
                    self.exit_cause = "stage finished"
                    rc_final = self.run_stage2(None, lease_env)
                    return rc_final
            self.exit_cause = "round limit reached"
            rc_final = 0
            return 0
        except KeyboardInterrupt:
            rc_final = 130
            return 130
        except lease.LeaseError as e:
            self.exit_cause = f"lease: {e}"
            rc_final = 75
            return 75
        finally:
            if provider is not None and handle:
                lease.release("gpu", loop_id=self.loop_id, provider=provider)
                self.event("lease_released", handle=handle)
            self.event("loop_exit", rc=rc_final, cause=self.exit_cause, milestone=self.milestone)
            for s, h in prev_handlers.items():
                signal.signal(s, h)


# ---- fork a loop at a passed milestone -----------------------------------------------------------------------------------------
def fork(cfg: LoopConfig, src_loop_id: str, at_milestone: str, new_loop_id: str | None = None, at_sha: str = "",
         workspace_dst: str | None = None) -> dict:
    """New loop whose state equals the source loop's at the moment ``at_milestone`` was accepted, so a normal ``run
    --loop-id`` continues from the NEXT milestone (tools/fork_loop.py).  The anchor commit comes from the source's
    ``milestone_advanced`` event, else from the one commit that declares the milestone; several declarations without an event
    are ambiguous and need ``at_sha``.  The source loop is not touched; with ``workspace_dst`` the workspace history up to
    the anchor is cloned there (``git clone`` + ``reset --hard``) for the new loop to work in."""
    if not os.path.isdir(os.path.join(cfg.loops_dir, src_loop_id)):
        raise ValueError(f"no loop {src_loop_id!r} under {cfg.loops_dir}")
    src = Loop(cfg, loop_id=src_loop_id)
    order = src.order
    if at_milestone not in order:
        raise ValueError(f"{at_milestone!r} is not in the milestone order {order}")
    decl = re.compile(rf"^MILESTONE_STATUS:[ \t]+{re.escape(at_milestone)}[ \t]+PASS[ \t]*$", re.M)

    def declares(sha: str) -> bool:
        return bool(sha) and bool(decl.search(src._git("show", "-s", "--format=%B", sha)))

    events = []
    ep = os.path.join(src.dir, "events.jsonl")
    if os.path.isfile(ep):
        for ln in open(ep, encoding="utf-8"):
            try:
                events.append(json.loads(ln))
            except json.JSONDecodeError:
                continue
    anchor, rnd, source = "", 0, ""
    if at_sha:
        full = src._git("rev-parse", at_sha).strip()
        if not declares(full):
            raise ValueError(f"{at_sha} does not exist in the workspace or does not declare 'MILESTONE_STATUS: {at_milestone} PASS'")
        anchor, source = full, "explicit-sha"
    else:
        hits = [e for e in events if e.get("subtype") == "milestone_advanced" and e.get("from") == at_milestone and declares(e.get("commit", ""))]
        if hits:
            anchor, rnd, source = hits[-1]["commit"], int(hits[-1].get("round", 0)), "event"
        else:
            shas = [h for h in src._git("log", "--format=%H").split() if declares(h)]
            if len(shas) != 1:
                raise ValueError(f"{len(shas)} commits declare {at_milestone!r} and no event names one: pass at_sha")
            anchor, source = shas[0], "git-fallback"
    nxt = order[min(order.index(at_milestone) + 1, len(order) - 1)]
    ws = cfg.workspace
    if workspace_dst:
        if os.path.exists(workspace_dst) and os.listdir(workspace_dst):
            raise ValueError(f"{workspace_dst} exists and is not empty")
        subprocess.run(["git", "clone", "-q", cfg.workspace, workspace_dst], check=True, timeout=600)
        subprocess.run(["git", "-C", workspace_dst, "reset", "-q", "--hard", anchor], check=True, timeout=120)
        ws = workspace_dst
    import dataclasses as _dc
    new = Loop(_dc.replace(cfg, workspace=ws), loop_id=new_loop_id)
    if os.path.exists(os.path.join(new.dir, "events.jsonl")):
        raise ValueError(f"loop {new.loop_id} already exists")
    new._write("stage1.milestone", nxt)
    new._write("stage1.status", "in-progress")
    new._write("stage1.round", str(rnd))
    src_hist = os.path.join(src.dir, "mfu_history.jsonl")
    if os.path.isfile(src_hist):
        import shutil
        shutil.copyfile(src_hist, os.path.join(new.dir, "mfu_history.jsonl"))
    info = {"src_loop_id": src_loop_id, "loop_id": new.loop_id, "anchor": anchor, "anchor_source": source, "passed": at_milestone,
            "next_milestone": nxt, "round": rnd, "workspace": ws}
    new.event("loop_forked", **info)
    return info


# ---- offline report -----------------------------------------------------------------------------------------------------------
def _fdur(s: float | None) -> str:
    if s is None:
        return "?"
    s = int(s)
    h, m = divmod(s // 60, 60)
    return f"{h}h{m:02d}m" if h else f"{m}m{s % 60:02d}s"


def report(loop_dir: str) -> dict:
    """Everything from files: events.jsonl, state/, mfu_history.jsonl.  Works on a live or a dead loop."""
    ev = []
    p = os.path.join(loop_dir, "events.jsonl")
    if os.path.isfile(p):
        for ln in open(p, encoding="utf-8"):
            try:
                ev.append(json.loads(ln))
            except json.JSONDecodeError:
                continue
    started = next((e for e in ev if e["subtype"] == "loop_started"), None)
    exits = [e for e in ev if e["subtype"] == "loop_exit"]
    rounds: dict[int, dict] = {}
    for e in ev:
        r = e.get("round")
        if r is None:
            continue
        row = rounds.setdefault(int(r), {"round": int(r), "errors": [], "status": "running", "review": "", "commits": [],
                                         "milestone": "", "attempts": 0, "duration_s": None})
        st = e["subtype"]
        if st == "round_started":
            row["milestone"], row["started"] = e.get("milestone", ""), e["ts"]
        elif st == "agent_failed":
            row["errors"].append(e.get("text", ""))
        elif st == "review_finished":
            row["review"] = e.get("verdict", "")
        elif st == "round_finished":
            row.update(status=e.get("status", ""), attempts=e.get("attempts", 0), duration_s=e.get("duration_s"),
                       commits=e.get("commits", []))
        elif st == "gate_run" and e.get("rc"):
            row["errors"].append(f"suite {e.get('suite')} rc={e.get('rc')}")
    adv = [e for e in ev if e["subtype"] in ("milestone_advanced", "milestone_auto_advanced", "milestone_advance_withheld")]
    order = (started or {}).get("order", [])
    passed_at = {e["from"]: e for e in adv if "from" in e}
    milestones = [{"milestone": m, "passed_round": passed_at[m]["round"] if m in passed_at else None,
                   "commit": passed_at[m].get("commit", "") if m in passed_at else ""} for m in order]
    rows = mfu.load(os.path.join(loop_dir, "mfu_history.jsonl"))
    traj, last = [], {}
    for r in rows:
        s = r.get("suite", "")
        d = r["mfu_avg"] - last[s] if s in last else None
        last[s] = r["mfu_avg"]
        traj.append({"ts": r.get("ts"), "suite": s, "mfu_avg": r["mfu_avg"], "delta": d, "loss_passed": r.get("loss_passed")})
    storms = [r["round"] for r in rounds.values() if len(r["errors"]) >= 3]
    live = not exits or (ev and ev[-1]["subtype"] != "loop_exit")
    return {"loop_id": (started or {}).get("loop_id", os.path.basename(loop_dir)), "live": bool(live),
            "started": (started or {}).get("ts"), "exit": exits[-1] if exits else None, "order": order,
            "milestones": milestones, "rounds": [rounds[k] for k in sorted(rounds)], "mfu": traj,
            "errors": {"exit_cause": exits[-1].get("cause") if exits else None,
                       "review_fails": [r["round"] for r in rounds.values() if r["review"] == "FAIL"],
                       "retry_storms": storms,
                       "withheld": [e.get("milestone") for e in adv if e["subtype"] == "milestone_advance_withheld"]}}


def report_markdown(rep: dict) -> str:
    ln = [f"# loop {rep['loop_id']}", "", f"state: {'live' if rep['live'] else 'exited'}"
          + (f" (rc={rep['exit']['rc']}, {rep['exit']['cause']})" if rep["exit"] else ""), "", "## milestones", "",
          "| milestone | passed in round | commit |", "|---|---|---|"]
    for m in rep["milestones"]:
        ln.append(f"| {m['milestone']} | {m['passed_round'] if m['passed_round'] is not None else '-'} | {m['commit'][:10]} |")
    ln += ["", "## rounds", "", "| round | milestone | status | duration | attempts | review | commits | errors |", "|---|---|---|---|---|---|---|---|"]
    for r in rep["rounds"]:
        ln.append(f"| {r['round']} | {r['milestone']} | {r['status']} | {_fdur(r['duration_s'])} | {r['attempts']} | {r['review'] or '-'} "
                  f"| {len(r['commits'])} | {'; '.join(x[:80] for x in r['errors']) or '-'} |")
    if rep["mfu"]:
        ln += ["", "## MFU trajectory", "", "| suite | MFU % | delta | loss |", "|---|---|---|---|"]
        for t in rep["mfu"]:
            d = f"{t['delta']:+.2f}" if t["delta"] is not None else "-"
            ln.append(f"| {t['suite']} | {t['mfu_avg']:.2f} | {d} | {t['loss_passed']} |")
    e = rep["errors"]
    ln += ["", "## error digest", "", f"* exit cause: {e['exit_cause']}", f"* review FAIL rounds: {e['review_fails'] or '-'}",
           f"* retry storms (>= 3 failed attempts) in rounds: {e['retry_storms'] or '-'}",
           f"* withheld declarations: {e['withheld'] or '-'}"]
    return "\n".join(ln) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="loop")
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run")
    r.add_argument("--config", required=True)
    r.add_argument("--loop-id", default=os.environ.get("FORGE_LOOP_ID", ""))
    r.add_argument("--max-rounds", type=int, default=None)
    r.add_argument("--reset-state", action="store_true")
    rp = sub.add_parser("report")
    rp.add_argument("loop_dir")
    rp.add_argument("--json", default="")
    rp.add_argument("--md", default="")
    fk = sub.add_parser("fork")
    fk.add_argument("--config", required=True)
    fk.add_argument("--src-loop-id", required=True)
    fk.add_argument("--at-milestone", required=True)
    fk.add_argument("--at-sha", default="")
    fk.add_argument("--new-loop-id", default="")
    fk.add_argument("--workspace", default="", help="clone the workspace at the anchor commit into this empty directory")
    sr = sub.add_parser("should-retry")
    sr.add_argument("rc", type=int)
    ms = sub.add_parser("stage-milestones")
    ms.add_argument("--registry", default=os.path.join(ROOT, "configs", "eval", "dense_training.toml"))
    a = ap.parse_args(argv)
    if a.cmd == "should-retry":
        return 0 if should_retry(a.rc) else 1
    if a.cmd == "stage-milestones":
        print("\n".join(milestone_order(a.registry)))
        return 0
    if a.cmd == "fork":
        try:
            info = fork(LoopConfig.load(a.config), a.src_loop_id, a.at_milestone, a.new_loop_id or None, a.at_sha, a.workspace or None)
        except ValueError as e:
            print(f"fork: {e}", file=sys.stderr)
            return 1
        print(json.dumps(info, indent=1))
        print(f"continue with: python -m forge_train_harness_b200.harness.loop run --config {a.config} --loop-id {info['loop_id']}", file=sys.stderr)
        return 0
    if a.cmd == "report":
        rep = report(a.loop_dir)
        md = report_markdown(rep)
        if a.json:
            with open(a.json, "w", encoding="utf-8") as f:
                json.dump(rep, f, indent=1)
        if a.md:
            with open(a.md, "w", encoding="utf-8") as f:
                f.write(md)
        print(md)
        return 0
    loop = Loop(LoopConfig.load(a.config), loop_id=a.loop_id or None)
    if a.reset_state:
        loop.reset_state()
    print(f"loop {loop.loop_id}: {loop.dir}  ({shlex.join(str(x) for x in loop.cfg.worker_cmd)})", file=sys.stderr)
    return loop.run(a.max_rounds)


if __name__ == "__main__":
    sys.exit(main())
