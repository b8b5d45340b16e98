"""Short-lived GPU jobs: run one gate suite on leased GPUs, release them the moment it ends.

The reference's ``tools/gpu_job.py`` (gpu_job.py:361-505) keeps a loop's gateway machine GPU-less and submits every GPU
suite as its own job: one submission per ``(suite, commit)``, a persisted handle so a poll that was cut short can be
resumed by a separate invocation, an exec deadline that the CALLER supplies and that is anchored at the first ``running``
poll (time spent queued never counts), logs dumped and the handle marked consumed once a verdict exists, terminal phase
mapped to an exit code.  This module owns the same lifecycle against a small scheduler interface:

* ``LocalScheduler`` — jobs are process groups on this node.  A detached supervisor (this module run with ``_supervise``)
  waits for a GPU lease (phase ``queued``), runs the entry with ``CUDA_VISIBLE_DEVICES`` set to the leased ordinals (phase
  ``running``), records the exit code and releases the lease.  Everything the poller needs is in files under the job
  directory, so submit and poll can be different processes.
* any object with ``submit / phase / stop / logs`` (an external scheduler; the tests use a scripted fake).

Exit codes of ``run_suite`` / ``poll_suite``: 0 the job succeeded, 1 it failed, 124 it overran the exec window and was
stopped, 75 an in-flight job for this suite and commit already exists (nothing submitted), 76 there is nothing to poll.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time
import uuid

from . import lease

__all__ = ["LocalScheduler", "CommandScheduler", "scheduler_from_config", "run_suite", "poll_suite", "build_entry", "main", "TIMEOUT_RC", "INFLIGHT_RC", "NO_JOB_RC"]

TIMEOUT_RC, INFLIGHT_RC, NO_JOB_RC = 124, 75, 76
SUCCESS_PHASES = frozenset({"succeeded"})
FAIL_PHASES = frozenset({"failed", "stopped", "unknown"})
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _state_dir() -> str:
    d = os.environ.get("FORGE_JOBS_DIR") or os.path.join(ROOT, ".artifacts", "gpu_jobs")
    os.makedirs(d, exist_ok=True)
    return d


# ---- handle store ------------------------------------------------------------------------------------------------------------
def _handle_path(suite: str) -> str:
    safe = "".join(c if c.isalnum() or c in "._-" else "_" for c in suite)
    return os.path.join(_state_dir(), f"{safe}.handle.json")


def _read_handle(path: str) -> dict | None:
    try:
        with open(path, encoding="utf-8") as f:
            rec = json.load(f)
        return rec if isinstance(rec, dict) else None
    except (FileNotFoundError, json.JSONDecodeError):
        return None


def _write_handle(path: str, rec: dict) -> None:
    tmp = path + f".tmp{os.getpid()}"
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(rec, f, indent=1)
    os.replace(tmp, path)


def workspace_commit(cwd: str | None = None) -> str:
    """Identity of the code a job runs: the git commit, plus a marker when the tree has uncommitted changes."""
    cwd = cwd or ROOT
    try:
        sha = subprocess.run(["git", "rev-parse", "HEAD"], cwd=cwd, capture_output=True, text=True, timeout=20).stdout.strip()
        dirty = subprocess.run(["git", "status", "--porcelain"], cwd=cwd, capture_output=True, text=True, timeout=20).stdout.strip()
        return sha + ("+dirty" if dirty else "") if sha else ""
    except (OSError, subprocess.TimeoutExpired):
        return ""


# ---- local scheduler ---------------------------------------------------------------------------------------------------------
class LocalScheduler:
    """Jobs as supervised process groups on this node; GPUs come from the ``lease`` registry."""

    def __init__(self, jobs_dir: str | None = None, total_gpus: int | None = None):
        self.dir = jobs_dir or os.path.join(_state_dir(), "local")
        os.makedirs(self.dir, exist_ok=True)
        self.total_gpus = total_gpus

    def _job(self, job_id: str) -> str:
        return os.path.join(self.dir, job_id)

    def submit(self, entry: str, *, gpus: int, nodes: int = 1, env: dict | None = None, cwd: str | None = None,
               queue_timeout_s: float = 86400.0) -> str:
        if nodes != 1:
            raise ValueError("the local scheduler runs single-node jobs; use an external scheduler for nodes > 1")
        job_id = uuid.uuid4().hex[:12]
        jd = self._job(job_id)
        os.makedirs(jd)
        with open(os.path.join(jd, "spec.json"), "w", encoding="utf-8") as f:
            json.dump({"entry": entry, "gpus": gpus, "env": env or {}, "cwd": cwd or ROOT, "total_gpus": self.total_gpus,
                       "queue_timeout_s": queue_timeout_s}, f)
        self._set(jd, "phase", "queued")
        envp = dict(os.environ)
        envp["PYTHONPATH"] = os.pathsep.join([ROOT, envp.get("PYTHONPATH", "")])
        with open(os.path.join(jd, "supervisor.log"), "wb") as lg:
            p = subprocess.Popen([sys.executable, "-m", "forge_train_harness_b200.harness.jobs", "_supervise", jd],
                                 stdin=subprocess.DEVNULL, stdout=lg, stderr=lg, start_new_session=True, env=envp, cwd=ROOT)
        self._set(jd, "supervisor_pid", str(p.pid))
        return job_id

    @staticmethod
    def _set(jd: str, name: str, value: str) -> None:
        tmp = os.path.join(jd, f".{name}.tmp{os.getpid()}")
        with open(tmp, "w", encoding="utf-8") as f:
            f.write(value)
        os.replace(tmp, os.path.join(jd, name))

    @staticmethod
    def _get(jd: str, name: str) -> str:
        try:
            with open(os.path.join(jd, name), encoding="utf-8") as f:
                return f.read().strip()
        except FileNotFoundError:
            return ""

    def phase(self, job_id: str) -> str:
        jd = self._job(job_id)
        if not os.path.isdir(jd):
            return "unknown"
        ph = self._get(jd, "phase") or "unknown"
        if ph in ("queued", "running"):
            sup = int(self._get(jd, "supervisor_pid") or 0)
            if sup and not lease._pid_alive(sup) and not self._get(jd, "rc"):
                return "failed"  # the supervisor died without a verdict
        return ph

    def stop(self, job_id: str, reason: str = "") -> None:
        jd = self._job(job_id)
        self._set(jd, "stop_reason", reason or "stopped")
        # the exact process groups this job started: the entry's, then the supervisor's
        for name in ("pgid", "supervisor_pid"):
            pid = int(self._get(jd, name) or 0)
            if pid > 1:
                try:
                    os.killpg(pid, signal.SIGTERM)
                except (ProcessLookupError, PermissionError):
                    pass
        end = time.monotonic() + 10.0
        while time.monotonic() < end and lease._pid_alive(int(self._get(jd, "supervisor_pid") or 0)):
            time.sleep(0.05)
        for name in ("pgid", "supervisor_pid"):
            pid = int(self._get(jd, name) or 0)
            if pid > 1 and lease._pid_alive(pid):
                try:
                    os.killpg(pid, signal.SIGKILL)
                except (ProcessLookupError, PermissionError):
                    pass
        if self._get(jd, "phase") in ("queued", "running"):
            self._set(jd, "phase", "stopped")
        lease.release("gpu", loop_id=f"job-{job_id}", provider=lease.LocalGpuProvider(total_gpus=self.total_gpus or 0))

    def logs(self, job_id: str, tail_bytes: int = 65536) -> str:
        p = os.path.join(self._job(job_id), "log")
        try:
            with open(p, "rb") as f:
                f.seek(0, os.SEEK_END)
                n = f.tell()
                f.seek(max(0, n - tail_bytes))
                return f.read().decode("utf-8", "replace")
        except FileNotFoundError:
            return ""


class CommandScheduler:
    """An external job scheduler behind argv templates (the form the reference hard-codes for its cluster CLI,
    tools/gpu_job.py:273-360)::

        [remote.jobs]
        submit = ["sched", "job", "create", "--gpus", "{gpus}", "--nodes", "{nodes}", "--entry", "{entry}"]
        id_regex = "tasks/([0-9a-f]+)"
        phase  = ["sched", "job", "get", "tasks/{job_id}", "--field", "phase"]
        stop   = ["sched", "job", "stop", "--yes", "tasks/{job_id}"]
        logs   = ["sched", "job", "logs", "tasks/{job_id}", "--tail", "200"]
        phase_map = {Queued = "queued", Running = "running", Succeeded = "succeeded", Failed = "failed", Stopped = "stopped"}

    Multi-node jobs are the scheduler's business: ``nodes`` pods of ``gpus`` GPUs each, rendezvous variables injected by it."""

    def __init__(self, table: dict):
        import re
        for k in ("submit", "phase", "stop"):
            if not isinstance(table.get(k), list) or not table[k]:
                raise ValueError(f"[remote.jobs].{k} must be a non-empty argv list")
        self.t = table
        self.id_re = re.compile(table.get("id_regex", r"([A-Za-z0-9_.-]+)\s*$"))
        self.phase_map = {str(k).lower(): str(v) for k, v in (table.get("phase_map") or {}).items()}

    def _run(self, argv, **kw):
        cmd = [a.format(**kw) for a in argv]
        return subprocess.run(cmd, capture_output=True, text=True, timeout=float(self.t.get("call_timeout_s", 120)))

    def submit(self, entry: str, *, gpus: int, nodes: int = 1, env: dict | None = None) -> str:
        import shlex
        if env:
            entry = " ".join(f"{k}={shlex.quote(str(v))}" for k, v in env.items()) + " " + entry
        r = self._run(self.t["submit"], entry=entry, gpus=gpus, nodes=nodes)
        m = self.id_re.search(r.stdout) if r.returncode == 0 else None
        if not m:
            raise RuntimeError(f"job submission failed (rc {r.returncode}): {(r.stderr or r.stdout)[-400:]}")
        return m.group(1)

    def phase(self, job_id: str) -> str:
        r = self._run(self.t["phase"], job_id=job_id)
        if r.returncode != 0 or not r.stdout.strip():
            return "unknown"
        raw = r.stdout.strip().splitlines()[-1].strip().lower()
        return self.phase_map.get(raw, raw)

    def stop(self, job_id: str, reason: str = "") -> None:
        self._run(self.t["stop"], job_id=job_id, reason=reason)

    def logs(self, job_id: str) -> str:
        if not self.t.get("logs"):
            return ""
        r = self._run(self.t["logs"], job_id=job_id)
        return r.stdout[-65536:]


def scheduler_from_config(remote: dict | None):
    """``[remote]`` -> scheduler: ``kind = "local"`` (or no table) runs jobs on this node's GPUs, ``"job"`` / ``"scheduler"`` with a
    ``[remote.jobs]`` table drives an external scheduler."""
    remote = remote or {}
    if remote.get("kind", "local") == "local" or not remote.get("jobs"):
        return LocalScheduler(total_gpus=remote.get("total_gpus"))
    return CommandScheduler(remote["jobs"])


def _supervise(jd: str) -> int:
    """Body of the detached supervisor: lease -> run -> record -> release."""
    with open(os.path.join(jd, "spec.json"), encoding="utf-8") as f:
        spec = json.load(f)
    job_id = os.path.basename(jd)
    prov = lease.LocalGpuProvider(total_gpus=spec.get("total_gpus"), holder_pid=os.getpid())
    loop_id = f"job-{job_id}"
    child = {"p": None}

    def _term(signum, frame):
        p = child["p"]
        if p is not None and p.poll() is None:
            try:
                os.killpg(p.pid, signal.SIGTERM)
            except ProcessLookupError:
                pass
        else:
            lease.release("gpu", loop_id=loop_id, provider=prov)
            LocalScheduler._set(jd, "phase", "stopped")
            os._exit(143)

    signal.signal(signal.SIGTERM, _term)
    try:
        handle = lease.claim("gpu", spec=lease.LeaseSpec(int(spec["gpus"])), loop_id=loop_id, provider=prov,
                             timeout=float(spec.get("queue_timeout_s", 86400.0)), poll_s=float(os.environ.get("FORGE_JOBS_POLL_S", "2")))
    except lease.LeaseError as e:
        with open(os.path.join(jd, "log"), "a", encoding="utf-8") as lg:
            lg.write(f"[supervisor] no lease: {e}\n")
        LocalScheduler._set(jd, "rc", "1")
        LocalScheduler._set(jd, "phase", "failed")
        return 1
    rc = 1
    try:
        env = dict(os.environ)
        env.update({k: str(v) for k, v in spec.get("env", {}).items()})
        if int(spec["gpus"]) > 0:
            env.update(prov.env(handle))
        env["FORGE_JOB_ID"] = job_id
        with open(os.path.join(jd, "log"), "ab") as lg:
            p = subprocess.Popen(["bash", "-c", spec["entry"]], stdin=subprocess.DEVNULL, stdout=lg, stderr=subprocess.STDOUT,
                                 start_new_session=True, env=env, cwd=spec.get("cwd") or ROOT)
            child["p"] = p
            LocalScheduler._set(jd, "pgid", str(p.pid))
            LocalScheduler._set(jd, "started_at", repr(time.time()))
            LocalScheduler._set(jd, "phase", "running")
            rc = p.wait()
    finally:
        lease.release("gpu", loop_id=loop_id, provider=prov)
        LocalScheduler._set(jd, "rc", str(rc))
        stopped = bool(LocalScheduler._get(jd, "stop_reason"))
        LocalScheduler._set(jd, "phase", "stopped" if stopped else ("succeeded" if rc == 0 else "failed"))
    return rc


# ---- lifecycle ---------------------------------------------------------------------------------------------------------------
def build_entry(*, suite: str, extra: list[str], loop_id: str = "", workdir: str | None = None, loop_dir: str = "") -> str:
    """Shell line a job runs for a suite: the harness CLI from the synced workspace, with the loop id exported so the run's
    records land under the loop's directory."""
    import shlex
    loop_dir = loop_dir or os.environ.get("FORGE_LOOP_DIR", "")
    parts = [f"cd {shlex.quote(workdir or ROOT)}", f"export FORGE_LOOP_ID={shlex.quote(loop_id)}" if loop_id else "true",
             f"export FORGE_LOOP_DIR={shlex.quote(loop_dir)}" if loop_dir else "true",
             " ".join([shlex.quote(sys.executable), "-m", "forge_train_harness_b200.harness", "run", shlex.quote(suite)]
                      + [shlex.quote(x) for x in extra])]
    return " && ".join(parts)


def _poll_to_terminal(sched, hpath: str, rec: dict, *, outer: float, poll_interval_s: float, out=sys.stderr) -> int:
    job_id = str(rec["job_id"])
    while True:
        phase = sched.phase(job_id)
        if phase in SUCCESS_PHASES:
            rc = 0
            break
        if phase in FAIL_PHASES:
            print(f"gpu_job: job {job_id} ended in phase {phase!r}", file=out)
            rc = 1
            break
        if phase == "running" and not rec.get("running_since"):
            rec["running_since"] = time.time()
            rec["status"] = "running"
            _write_handle(hpath, rec)
            queued = rec["running_since"] - float(rec.get("submitted_at") or rec["running_since"])
            print(f"gpu_job: job {job_id} started running after {queued:.0f}s queued; exec window {outer:.0f}s", file=out)
        since = rec.get("running_since")
        if since and time.time() - float(since) >= outer:
            print(f"gpu_job: job {job_id} exceeded the {outer:.0f}s exec window (counted from running); stopping it", file=out)
            sched.stop(job_id, reason="exec wall-clock window exceeded")
            rc = TIMEOUT_RC
            break
        time.sleep(poll_interval_s)
    rec["status"] = "consumed"
    rec["rc"] = rc
    _write_handle(hpath, rec)
    tail = sched.logs(job_id)
    if tail:
        print(f"---- job {job_id} log tail ----\n{tail}", file=out)
    return rc


def run_suite(sched, *, suite: str, entry: str, gpus: int, outer: float, nodes: int = 1, env: dict | None = None,
              commit: str | None = None, poll_interval_s: float = 30.0, out=sys.stderr) -> int:
    """Submit ``entry`` for ``suite`` and poll it.  Submission is one-shot per (suite, commit): a live handle at the same
    commit is never resubmitted (returns 75; use ``poll_suite``); one at another commit is stale — stopped and replaced."""
    hpath = _handle_path(suite)
    commit = workspace_commit() if commit is None else commit
    rec = _read_handle(hpath)
    if rec and rec.get("status") != "consumed" and rec.get("job_id"):
        if rec.get("commit_sha") == commit:
            print(f"gpu_job: job {rec['job_id']} is in flight for suite={suite} at {commit[:8] or '?'}; not resubmitting "
                  f"(poll it instead)", file=out)
            return INFLIGHT_RC
        sched.stop(str(rec["job_id"]), reason="superseded by a new commit")
    job_id = sched.submit(entry, gpus=gpus, nodes=nodes, env=env)
    print(f"gpu_job: submitted suite={suite} as job {job_id} (nodes={nodes}, gpus per node={gpus})", file=out)
    rec = {"suite": suite, "job_id": job_id, "commit_sha": commit, "submitted_at": time.time(), "running_since": None,
           "status": "submitted"}
    _write_handle(hpath, rec)  # before the first poll: a killed poller must leave something to resume from
    return _poll_to_terminal(sched, hpath, rec, outer=outer, poll_interval_s=poll_interval_s, out=out)


def poll_suite(sched, *, suite: str, outer: float, poll_interval_s: float = 30.0, out=sys.stderr) -> int:
    """Continue polling the job recorded for ``suite``.  Never submits."""
    hpath = _handle_path(suite)
    rec = _read_handle(hpath)
    if not rec or rec.get("status") == "consumed" or not rec.get("job_id"):
        print(f"gpu_job: no in-flight job for suite={suite}", file=out)
        return NO_JOB_RC
    return _poll_to_terminal(sched, hpath, rec, outer=outer, poll_interval_s=poll_interval_s, out=out)


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv[:1] == ["_supervise"]:
        return _supervise(argv[1])
    ap = argparse.ArgumentParser(prog="gpu_job")
    ap.add_argument("suite")
    ap.add_argument("--outer", type=float, default=0.0,
                    help="exec window in seconds, owned by the caller; default: the suite's `harness budget` plus a 120 s margin "
                         "for start-up and result write-back (the sum the reference's tools/remote_run.sh passes)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--poll", action="store_true", help="poll the in-flight job of this suite; never submit")
    ap.add_argument("--poll-interval", type=float, default=30.0)
    ap.add_argument("--loop-id", default=os.environ.get("FORGE_LOOP_ID", ""))
    ap.add_argument("--entry", default="", help="shell line to run instead of `harness run <suite>`")
    ap.add_argument("--remote-toml", default="", help="file with a [remote] table ([remote.jobs] = an external scheduler)")
    ap.add_argument("--nodes", type=int, default=1)
    ap.add_argument("extra", nargs="*")
    a = ap.parse_args(argv)
    if a.outer <= 0:
        r = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.harness", "budget", a.suite], capture_output=True, text=True, cwd=ROOT)
        if r.returncode != 0 or not r.stdout.strip().isdigit():
            print(f"gpu_job: no budget for suite {a.suite!r}: {r.stderr.strip()}", file=sys.stderr)
            return 64
        a.outer = float(r.stdout.strip()) + 120.0
    remote = {}
    if a.remote_toml:
        import tomllib
        with open(a.remote_toml, "rb") as f:
            remote = tomllib.load(f).get("remote", {})
    sched = scheduler_from_config(remote)
    if a.poll:
        return poll_suite(sched, suite=a.suite, outer=a.outer, poll_interval_s=a.poll_interval)
    entry = a.entry or build_entry(suite=a.suite, extra=a.extra, loop_id=a.loop_id)
    return run_suite(sched, suite=a.suite, entry=entry, gpus=a.gpus, nodes=a.nodes, outer=a.outer, poll_interval_s=a.poll_interval)


if __name__ == "__main__":
    sys.exit(main())
