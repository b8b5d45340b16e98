"""GPU lease registry and short-lived GPU jobs, on CPU with fake schedulers (reference contract: tools/lease.py,
tools/gpu_job.py; their tests inject a fake scheduler CLI the same way)."""
import io
import json
import os
import stat
import subprocess
import sys
import time

import pytest

from forge_train_harness_b200.harness import jobs, lease


@pytest.fixture()
def lease_root(tmp_path, monkeypatch):
    monkeypatch.setenv("FORGE_LEASE_DIR", str(tmp_path / "lease"))
    monkeypatch.setenv("FORGE_JOBS_DIR", str(tmp_path / "jobs"))
    monkeypatch.setenv("FORGE_JOBS_POLL_S", "0.05")
    return tmp_path


def _sleeper():
    return subprocess.Popen([sys.executable, "-c", "import time; time.sleep(60)"])


def test_local_claims_are_exclusive_idempotent_and_aligned(lease_root):
    a, b = _sleeper(), _sleeper()
    try:
        pa = lease.LocalGpuProvider(total_gpus=8, holder_pid=a.pid)
        pb = lease.LocalGpuProvider(total_gpus=8, holder_pid=b.pid)
        ha = lease.claim("gpu", spec=lease.LeaseSpec(4), loop_id="loopA", provider=pa)
        hb = lease.claim("gpu", spec=lease.LeaseSpec(4), loop_id="loopB", provider=pb)
        assert ha == "gpu-0-1-2-3" and hb == "gpu-4-5-6-7"  # halves of the box, not interleaved
        assert lease.claim("gpu", spec=lease.LeaseSpec(4), loop_id="loopA", provider=pa) == ha  # idempotent
        with pytest.raises(lease.LeaseTimeoutError):
            lease.claim("gpu", spec=lease.LeaseSpec(1), loop_id="loopC", provider=lease.LocalGpuProvider(8), timeout=0.2, poll_s=0.05)
        assert pa.env(ha) == {"CUDA_VISIBLE_DEVICES": "0,1,2,3"}
        lease.release("gpu", loop_id="loopA", provider=pa)
        reg = lease.holders("gpu")
        assert list(reg) == [hb] and reg[hb]["loop_id"] == "loopB"
        assert not os.path.exists(os.path.join(str(lease_root), "lease", "gpu", "loopA.handle"))
        assert lease.claim("gpu", spec=lease.LeaseSpec(2), loop_id="loopC", provider=lease.LocalGpuProvider(8)) == "gpu-0-1"
        lease.release("gpu", loop_id="nobody")  # nothing held: silent
    finally:
        a.kill(), b.kill()
        a.wait(), b.wait()


def test_gpu_less_gateway_leases_coexist_with_gpu_leases(lease_root):
    a = _sleeper()
    try:
        p = lease.LocalGpuProvider(total_gpus=2, holder_pid=a.pid)
        g1 = lease.claim("gpu", spec=lease.LeaseSpec(0), loop_id="gw1", provider=p)
        g2 = lease.claim("gpu", spec=lease.LeaseSpec(0), loop_id="gw2", provider=p)
        assert g1 == "gpu-none@gw1" and g2 == "gpu-none@gw2" and p.env(g1) == {"CUDA_VISIBLE_DEVICES": ""}
        assert lease.claim("gpu", spec=lease.LeaseSpec(2), loop_id="worker", provider=p) == "gpu-0-1"   # gateways hold no ordinals
        lease.release("gpu", loop_id="gw1", provider=p)
        assert sorted(lease.holders("gpu")) == ["gpu-0-1", "gpu-none@gw2"]
    finally:
        a.kill()
        a.wait()


def test_dead_holder_is_reclaimed(lease_root):
    a = _sleeper()
    pa = lease.LocalGpuProvider(total_gpus=2, holder_pid=a.pid)
    assert lease.claim("gpu", spec=lease.LeaseSpec(2), loop_id="crashed", provider=pa) == "gpu-0-1"
    a.kill()
    a.wait()
    h = lease.claim("gpu", spec=lease.LeaseSpec(2), loop_id="next", provider=lease.LocalGpuProvider(2), timeout=1.0, poll_s=0.05)
    assert h == "gpu-0-1"
    reg = lease.holders("gpu")
    assert reg[h]["loop_id"] == "next" and len(reg) == 1
    # the crashed loop's late release must not drop the new holder's row
    lease.release("gpu", loop_id="crashed", provider=pa)
    assert lease.holders("gpu")[h]["loop_id"] == "next"
    # a recycled process id is not the holder: same pid, another start time -> reclaimable
    row = dict(lease.holders("gpu")[h])
    assert row["task_start"] and lease.LocalGpuProvider(2).live(row)
    assert not lease.LocalGpuProvider(2).live(dict(row, task_start="1"))


def _fake_scheduler(tmp_path, flake_first_create=False):
    """A scripted scheduler CLI: ``create`` prints ``tasks/<n>``, ``get`` walks Queued -> Running, ``stop`` records."""
    state = tmp_path / "sched_state.json"
    state.write_text(json.dumps({"n": 0, "polls": {}, "stopped": [], "creates": 0}))
    exe = tmp_path / "sched"
    exe.write_text(f"""#!{sys.executable}
import json, sys
p = {str(state)!r}
s = json.load(open(p))
cmd = sys.argv[1]
rc = 0
if cmd == "create":
    s["creates"] += 1
    if {flake_first_create!r} and s["creates"] == 1:
        sys.stderr.write("error: not_found (lookup)\\n"); rc = 2
    else:
        s["n"] += 1; s["polls"][str(s["n"])] = 0
        s["last_args"] = sys.argv[2:]
        print("created tasks/%d" % s["n"])
elif cmd == "get":
    t = sys.argv[2].split("/")[1]
    if t in [x.split("/")[1] for x in s["stopped"]]:
        print("Stopped")
    else:
        s["polls"][t] = s["polls"].get(t, 0) + 1
        print("Queued" if s["polls"][t] < 2 else "Running")
elif cmd == "stop":
    s["stopped"].append(sys.argv[-1])
json.dump(s, open(p, "w"))
sys.exit(rc)
""")
    exe.chmod(exe.stat().st_mode | stat.S_IEXEC)
    table = {"create": [str(exe), "create", "--gpus", "{gpu_count}", "--pool", "{pool}"], "id_regex": r"tasks/(\d+)",
             "phase": [str(exe), "get", "tasks/{task_id}"], "stop": [str(exe), "stop", "--yes", "tasks/{task_id}"],
             "handle": "box-{task_id}", "retry_regex": "not_found", "retry_sleep_scale": 0.0,
             "phase_map": {"Running": "running", "Queued": "queued", "Stopped": "stopped"}}
    return table, state


def test_scheduler_claim_polls_to_ready_retries_flake_and_release_stops(lease_root):
    table, state = _fake_scheduler(lease_root, flake_first_create=True)
    prov = lease.provider_from_config({"kind": "scheduler", "provider": table})
    h = lease.claim("box", spec=lease.LeaseSpec(8, {"pool": "b200"}), loop_id="L1", provider=prov, timeout=5, poll_s=0.01)
    s = json.loads(state.read_text())
    assert h == "box-1" and s["creates"] == 2 and s["last_args"] == ["--gpus", "8", "--pool", "b200"]
    assert lease.claim("box", spec=lease.LeaseSpec(8, {"pool": "b200"}), loop_id="L1", provider=prov) == h  # live: reused
    assert json.loads(state.read_text())["creates"] == 2
    # the box dropped; the operator re-created one by hand: rebind, then release stops the NEW one only
    lease.rebind("box", loop_id="L1", handle="box-77", provider=prov)
    assert list(lease.holders("box")) == ["box-77"]
    lease.release("box", loop_id="L1", provider=prov)
    assert json.loads(state.read_text())["stopped"] == ["tasks/77"] and lease.holders("box") == {}


def test_scheduler_template_needs_its_labels(lease_root):
    table, _ = _fake_scheduler(lease_root)
    prov = lease.CommandProvider(table)
    with pytest.raises(lease.LeaseError, match="pool"):
        lease.claim("box", spec=lease.LeaseSpec(1), loop_id="L2", provider=prov, timeout=1, poll_s=0.01)


def test_lease_cli_follows_the_parent_process(lease_root):
    env = dict(os.environ, FORGE_LEASE_TOTAL_GPUS="4")
    holder = _sleeper()
    try:
        r = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.harness.lease", "claim", "gpu", "--loop-id", "cli",
                            "--gpus", "2", "--holder-pid", str(holder.pid)], capture_output=True, text=True, env=env)
        assert r.returncode == 0 and r.stdout.strip() == "gpu-0-1", r.stderr
        r = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.harness.lease", "claim", "gpu", "--loop-id", "cli2",
                            "--gpus", "4", "--timeout", "0.2", "--holder-pid", str(holder.pid)], capture_output=True, text=True, env=env)
        assert r.returncode == 4 and "timeout" in r.stderr
        r = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.harness.lease", "list", "gpu"], capture_output=True, text=True, env=env)
        assert json.loads(r.stdout)["gpu-0-1"]["loop_id"] == "cli"
        subprocess.run([sys.executable, "-m", "forge_train_harness_b200.harness.lease", "release", "gpu", "--loop-id", "cli"], env=env, check=True)
        assert lease.holders("gpu") == {}
    finally:
        holder.kill()
        holder.wait()


# ---- jobs ------------------------------------------------------------------------------------------------------------------
class ScriptedScheduler:
    def __init__(self, phases):
        self.phases = list(phases)
        self.submitted, self.stopped = [], []

    def submit(self, entry, *, gpus, nodes=1, env=None):
        self.submitted.append(entry)
        return f"j{len(self.submitted)}"

    def phase(self, job_id):
        return self.phases.pop(0) if len(self.phases) > 1 else self.phases[0]

    def stop(self, job_id, reason=""):
        self.stopped.append((job_id, reason))

    def logs(self, job_id):
        return "the log"


def test_job_exec_window_is_anchored_at_running_and_handle_is_consumed(lease_root):
    out = io.StringIO()
    s = ScriptedScheduler(["queued"] * 5 + ["running", "running", "succeeded"])
    rc = jobs.run_suite(s, suite="long-train", entry="true", gpus=2, outer=0.5, commit="abc", poll_interval_s=0.05, out=out)
    assert rc == 0 and "started running after" in out.getvalue() and "the log" in out.getvalue()
    rec = json.load(open(jobs._handle_path("long-train")))
    assert rec["status"] == "consumed" and rec["rc"] == 0 and rec["running_since"]
    assert jobs.poll_suite(s, suite="long-train", outer=1, out=out) == jobs.NO_JOB_RC
    # queued for longer than the window never trips it; running for longer does, and the job is stopped
    s = ScriptedScheduler(["queued"] * 20 + ["running"])
    rc = jobs.run_suite(s, suite="slow", entry="true", gpus=1, outer=0.3, commit="abc", poll_interval_s=0.05, out=out)
    assert rc == jobs.TIMEOUT_RC and s.stopped and "exec" in s.stopped[0][1]
    s = ScriptedScheduler(["failed"])
    assert jobs.run_suite(s, suite="bad", entry="false", gpus=1, outer=5, commit="abc", poll_interval_s=0.01, out=out) == 1


def test_job_dedup_per_commit_and_resume_by_poll(lease_root):
    out = io.StringIO()
    hp = jobs._handle_path("gate")
    os.makedirs(os.path.dirname(hp), exist_ok=True)
    jobs._write_handle(hp, {"suite": "gate", "job_id": "j0", "commit_sha": "abc", "status": "submitted", "submitted_at": time.time()})
    s = ScriptedScheduler(["running", "succeeded"])
    assert jobs.run_suite(s, suite="gate", entry="true", gpus=1, outer=5, commit="abc", out=out) == jobs.INFLIGHT_RC
    assert s.submitted == []
    assert jobs.poll_suite(s, suite="gate", outer=5, poll_interval_s=0.01, out=out) == 0  # a separate poll finishes it
    # same suite at another commit: the stale job is stopped, a new one submitted
    jobs._write_handle(hp, {"suite": "gate", "job_id": "j0", "commit_sha": "abc", "status": "running", "submitted_at": time.time()})
    s = ScriptedScheduler(["succeeded"])
    assert jobs.run_suite(s, suite="gate", entry="true", gpus=1, outer=5, commit="def", poll_interval_s=0.01, out=out) == 0
    assert s.stopped == [("j0", "superseded by a new commit")] and len(s.submitted) == 1


def test_local_scheduler_runs_queues_and_stops(lease_root):
    sched = jobs.LocalScheduler(total_gpus=2)
    out = io.StringIO()
    rc = jobs.run_suite(sched, suite="echo", entry='echo "devices=$CUDA_VISIBLE_DEVICES job=$FORGE_JOB_ID"', gpus=2, outer=30,
                        commit="c1", poll_interval_s=0.05, out=out)
    assert rc == 0 and "devices=0,1" in out.getvalue(), out.getvalue()
    assert lease.holders("gpu") == {}  # released the moment it ended
    assert jobs.run_suite(sched, suite="fails", entry="exit 3", gpus=1, outer=30, commit="c1", poll_interval_s=0.05, out=out) == 1
    # a second job queues behind a first that holds both GPUs, then runs
    j1 = sched.submit("sleep 0.6", gpus=2)
    t0 = time.time()
    while sched.phase(j1) != "running" and time.time() - t0 < 10:
        time.sleep(0.02)
    j2 = sched.submit("echo second", gpus=1)
    time.sleep(0.2)
    assert sched.phase(j2) == "queued"
    t0 = time.time()
    while sched.phase(j2) not in ("succeeded", "failed") and time.time() - t0 < 15:
        time.sleep(0.05)
    assert sched.phase(j1) == "succeeded" and sched.phase(j2) == "succeeded" and "second" in sched.logs(j2)
    # an overrunning job is stopped by the exec window: its process group is gone and its GPUs are free again
    rc = jobs.run_suite(sched, suite="hang", entry="sleep 100", gpus=1, outer=0.3, commit="c1", poll_interval_s=0.05, out=out)
    assert rc == jobs.TIMEOUT_RC
    rec = json.load(open(jobs._handle_path("hang")))
    assert sched.phase(rec["job_id"]) == "stopped" and lease.holders("gpu") == {}
    pg = int(jobs.LocalScheduler._get(sched._job(rec["job_id"]), "pgid"))
    time.sleep(0.2)
    assert not lease._pid_alive(pg)


_CLAIMER = r'''
import os, sys, time, random
sys.path.insert(0, sys.argv[1])
from forge_train_harness_b200.harness import lease
me, marks, rounds = sys.argv[2], sys.argv[3], int(sys.argv[4])
random.seed(int(me[1:]))
prov = lease.LocalGpuProvider(total_gpus=8)
for i in range(rounds):
    n = random.choice([1, 2, 4])
    h = lease.claim("gpu", spec=lease.LeaseSpec(n), loop_id=me, provider=prov, timeout=60, poll_s=0.01)
    ords = prov.ordinals(h)
    assert len(ords) == n
    for o in ords:                      # exclusive create: a second holder of the same ordinal fails here
        fd = os.open(os.path.join(marks, "gpu%d" % o), os.O_CREAT | os.O_EXCL | os.O_WRONLY)
        os.write(fd, me.encode()); os.close(fd)
    time.sleep(random.random() * 0.02)
    for o in ords:
        os.unlink(os.path.join(marks, "gpu%d" % o))
    lease.release("gpu", loop_id=me, provider=prov)
print("ok")
'''


def test_concurrent_claimers_never_share_a_gpu(lease_root):
    """Six processes claim and release 1 / 2 / 4 of 8 ordinals in a tight loop; while a lease is held its holder owns an
    exclusively-created marker per ordinal, so any double booking makes a claimer crash."""
    marks = lease_root / "marks"
    marks.mkdir()
    script = lease_root / "claimer.py"
    script.write_text(_CLAIMER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, FORGE_LEASE_DIR=str(lease_root / "lease"))
    procs = [subprocess.Popen([sys.executable, str(script), root, f"c{i}", str(marks), "15"], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for i in range(6)]
    outs = [p.communicate(timeout=240) for p in procs]
    assert all(p.returncode == 0 and o[0].strip() == "ok" for p, o in zip(procs, outs)), [o[1][-400:] for o in outs]
    assert lease.holders("gpu") == {} and os.listdir(marks) == []


def test_external_job_scheduler_behind_argv_templates(lease_root):
    """Submit / poll / logs / stop against a scripted scheduler executable, through the same lifecycle as local jobs."""
    state = lease_root / "jobs_state.json"
    state.write_text(json.dumps({"n": 0, "polls": {}, "stopped": [], "entries": []}))
    exe = lease_root / "jsched"
    exe.write_text(f"""#!{sys.executable}
import json, sys
p = {str(state)!r}
s = json.load(open(p)); cmd = sys.argv[1]
if cmd == "create":
    s["n"] += 1; s["entries"].append(sys.argv[2:]); print("submitted tasks/%d" % s["n"])
elif cmd == "get":
    t = sys.argv[2].split("/")[1]; s["polls"][t] = s["polls"].get(t, 0) + 1
    print("Stopped" if sys.argv[2] in s["stopped"] else ["Queued", "Queued", "Running", "Succeeded"][min(s["polls"][t] - 1, 3)])
elif cmd == "logs":
    print("remote log line")
elif cmd == "stop":
    s["stopped"].append(sys.argv[-1])
json.dump(s, open(p, "w"))
""")
    exe.chmod(exe.stat().st_mode | stat.S_IEXEC)
    table = {"submit": [str(exe), "create", "--gpus", "{gpus}", "--nodes", "{nodes}", "--entry", "{entry}"], "id_regex": r"tasks/(\d+)",
             "phase": [str(exe), "get", "tasks/{job_id}"], "stop": [str(exe), "stop", "--yes", "tasks/{job_id}"],
             "logs": [str(exe), "logs", "tasks/{job_id}"],
             "phase_map": {"Queued": "queued", "Running": "running", "Succeeded": "succeeded", "Stopped": "stopped"}}
    sched = jobs.scheduler_from_config({"kind": "job", "jobs": table})
    assert isinstance(sched, jobs.CommandScheduler) and isinstance(jobs.scheduler_from_config({}), jobs.LocalScheduler)
    out = io.StringIO()
    rc = jobs.run_suite(sched, suite="long-train", entry="harness run long-train", gpus=8, nodes=2, outer=30, commit="c", poll_interval_s=0.01, out=out)
    s = json.loads(state.read_text())
    assert rc == 0 and s["entries"] == [["--gpus", "8", "--nodes", "2", "--entry", "harness run long-train"]] and "remote log line" in out.getvalue()
    # an overrunning remote job is stopped through the scheduler
    s["polls"] = {}
    state.write_text(json.dumps(s))
    table2 = dict(table, phase=[str(exe), "get", "tasks/{job_id}", "x"])
    class Slow(jobs.CommandScheduler):
        def phase(self, job_id):
            return "running"
    rc = jobs.run_suite(Slow(table2), suite="slow-remote", entry="e", gpus=1, outer=0.1, commit="c", poll_interval_s=0.02, out=out)
    assert rc == jobs.TIMEOUT_RC and json.loads(state.read_text())["stopped"] == ["tasks/2"]
    with pytest.raises(ValueError, match="submit"):
        jobs.CommandScheduler({"phase": ["x"], "stop": ["x"]})
