"""Failure handling on the host: fast-fail launcher, bounded transport, SIGKILL mid-phase + checkpoint-driven restart."""
import os
import subprocess
import sys
import time

import pytest

from forge_train_harness_b200.gates import verdicts as V
from forge_train_harness_b200.runtime import launcher as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class FakeProc:
    def __init__(self, exit_after=None, rc=0, ignores_term=False):
        self.t0, self.exit_after, self.rc, self.ignores_term = None, exit_after, rc, ignores_term
        self.terminated = self.killed = False

    def poll(self):
        if self.killed:
            return -9
        if self.terminated and not self.ignores_term:
            return -15
        if self.exit_after is not None and FakeClock.now >= self.exit_after:
            return self.rc
        return None

    def terminate(self):
        self.terminated = True

    def kill(self):
        self.killed = True

    def wait(self):
        return self.poll()


class FakeClock:
    now = 0.0

    @classmethod
    def sleep(cls, s):
        cls.now += s

    @classmethod
    def clock(cls):
        return cls.now


def test_fast_fail_terminates_peers_within_one_poll_and_kills_stragglers():
    FakeClock.now = 0.0
    crash, peer, stubborn = FakeProc(exit_after=1.0, rc=3), FakeProc(), FakeProc(ignores_term=True)
    rc = L.wait_with_fast_fail([crash, peer, stubborn], poll_s=0.5, grace_s=30.0, sleep=FakeClock.sleep, clock=FakeClock.clock)
    assert rc == 3 and peer.terminated and not peer.killed
    assert stubborn.terminated and stubborn.killed and FakeClock.now >= 30.0
    FakeClock.now = 0.0
    assert L.wait_with_fast_fail([FakeProc(exit_after=0.5), FakeProc(exit_after=1.0)], sleep=FakeClock.sleep, clock=FakeClock.clock) == 0


def test_launcher_real_processes_rank_env_and_fast_fail():
    code = "import os,sys,time; r=int(os.environ['RANK']); assert os.environ['WORLD_SIZE']=='3' and os.environ['MASTER_ADDR']=='127.0.0.1'; " \
           "sys.exit(7) if r==1 else time.sleep(60)"
    t0 = time.time()
    assert L.launch([sys.executable, "-c", code], 3) == 7
    assert time.time() - t0 < 20  # peers were terminated, not waited for


def test_run_bounded_kills_the_process_group_on_timeout():
    rc, out = L.run_bounded([sys.executable, "-c", "print('hi')"], 20)
    assert rc == 0 and "hi" in out
    with pytest.raises(L.BoundedTimeout):
        L.run_bounded(["bash", "-c", "sleep 100 & sleep 100"], 1.0, term_grace_s=2.0)
    assert L.gpu_is_dirty(lambda: "123\n%d\n" % os.getpid()) == ["123"]


def _run_phases(root, kill_at):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "_phase_worker.py"), root, str(kill_at)], cwd=ROOT,
                       capture_output=True, text=True, timeout=600)
    return p.returncode, p.stdout


def test_sigkill_mid_phase_then_restart_matches_clean_run(tmp_path):
    rc, clean = _run_phases(str(tmp_path / "clean"), 0)
    assert rc == 0
    main_root = str(tmp_path / "main")
    os.makedirs(main_root)
    log = ""
    for kill_at in (3, 7, 10, 0):  # three kills (one per phase), then a run to completion
        rc, out = _run_phases(main_root, kill_at)
        log += out
        assert (rc == -9) == (kill_at != 0), (kill_at, rc, out[-500:])
    v = V.wsd_sft(clean, log)
    assert v["passed"], v
    assert V.production(os.path.join(main_root, "sft"), [10, 12])["passed"]
    assert not V.production(os.path.join(main_root, "sft"), [11])["passed"]


def test_profile_snapshot_wraps_rank0_only_behind_one_variable(tmp_path):
    """NSYS_PROFILE=1: rank 0 runs under the profiler executable when there is one, else the engine's own one-step profiler is
    switched on for it; the other ranks are untouched (evals/scripts/launch_dp.py:35-56)."""
    import stat
    from forge_train_harness_b200.runtime import launcher
    argv = [sys.executable, "-c", "pass"]
    base = {"PATH": "/nonexistent", "NSYS_PROFILE": "1", "NSYS_OUTPUT": str(tmp_path / "prof" / "rank0")}
    cmd, env = launcher.profile_wrap(argv, 1, dict(base))
    assert cmd == argv and "FORGE_PROFILE_STEP" not in env                      # not rank 0: as it is
    cmd, env = launcher.profile_wrap(argv, 0, dict(base))
    assert cmd == argv and env["FORGE_PROFILE_STEP"] == "5" and env["FORGE_PROFILE_RANK"] == "0" and env["FORGE_PROFILE_DIR"] == str(tmp_path / "prof")
    assert launcher.profile_wrap(argv, 0, {"PATH": "/nonexistent"}) == (argv, {"PATH": "/nonexistent"})  # variable unset: nothing
    # with a profiler executable: rank 0's command line is wrapped, and the wrapped program still runs with its rank env
    fake = tmp_path / "nsys"
    fake.write_text("#!/bin/bash\nout=\"\"; while [ $# -gt 0 ]; do if [ \"$1\" = -o ]; then out=$2; shift 2; break; fi; shift; done\n"
                    "echo \"wrapped rank=$RANK\" > \"$out.txt\"\nexec \"$@\"\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    marks = tmp_path / "marks"
    marks.mkdir()
    prog = [sys.executable, "-c", f"import os; open(os.path.join({str(marks)!r}, os.environ['RANK']), 'w').write('ran')"]
    env = dict(os.environ, NSYS_PROFILE="1", NSYS_BIN=str(fake), NSYS_OUTPUT=str(tmp_path / "prof" / "rank0"))
    assert launcher.launch(prog, 2, env=env) == 0
    assert sorted(os.listdir(marks)) == ["0", "1"]
    assert open(str(tmp_path / "prof" / "rank0") + ".txt").read().strip() == "wrapped rank=0"
