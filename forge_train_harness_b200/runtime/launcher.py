"""Single-node launcher with fast-fail, plus a bounded subprocess transport.

``launch(argv, nproc)`` starts one process per rank with RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT set
(MASTER_PORT "auto" picks a free ephemeral port), polls every 0.5 s and, as soon as one rank exits non-zero, sends
SIGTERM to its peers, waits ``grace_s`` and SIGKILLs what is left — so a crashed rank costs seconds, not a 600 s
rendezvous timeout (evals/scripts/launch_dp.py:59-137).  ``run_bounded`` runs a command in its own session with a
wall-clock budget and kills exactly that process group on expiry (harness/transport.py:319-460, evals/_common.py:935-996).
``gpu_is_dirty`` refuses to start on a GPU that still shows compute apps (evals/scripts/_runner_utils.py:20-79).
"""
from __future__ import annotations

import os
import signal
import socket
import subprocess
import sys
import time


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def rank_env(rank: int, world: int, port: int, base=None) -> dict:
    env = dict(base if base is not None else os.environ)
    env.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    return env


def wait_with_fast_fail(procs, poll_s: float = 0.5, grace_s: float = 30.0, sleep=time.sleep, clock=time.monotonic) -> int:
    """``procs`` need ``poll()``, ``terminate()``, ``kill()``.  Returns the first non-zero exit code, else 0."""
    live = list(procs)
    failed = 0
    while live:
        for p in list(live):
            rc = p.poll()
            if rc is None:
                continue
            live.remove(p)
            if rc != 0 and not failed:
                failed = rc
        if failed and live:
            for p in live:
                p.terminate()
            deadline = clock() + grace_s
            while live and clock() < deadline:
                live = [p for p in live if p.poll() is None]
                if live:
                    sleep(poll_s)
            for p in live:
                p.kill()
            for p in live:
                try:
                    p.wait()
                except Exception:  # noqa: BLE001
                    pass
            return failed
        if live:
            sleep(poll_s)
    return failed


def profile_wrap(argv: list[str], rank: int, env: dict) -> tuple[list[str], dict]:
    """Profile snapshot behind ONE variable (evals/scripts/launch_dp.py:35-56): with ``NSYS_PROFILE=1`` rank 0 alone is
    profiled, the other ranks run as they are.  Where an ``nsys`` executable exists (``NSYS_BIN`` or PATH) rank 0 is wrapped
    in ``nsys profile`` writing ``$NSYS_OUTPUT`` (default ``profile_out/rank0``); where it does not, the same variable turns
    on the engine's own one-step profiler (``utils/step_profile.py``: ``FORGE_PROFILE_STEP``, default step 5) — the per-kernel
    summary is the same table either way."""
    if env.get("NSYS_PROFILE", "0") != "1" or rank != 0:
        return argv, env
    import shutil
    nsys = env.get("NSYS_BIN") or shutil.which("nsys")
    env = dict(env)
    if nsys:
        out = env.get("NSYS_OUTPUT", os.path.join("profile_out", "rank0"))
        os.makedirs(os.path.dirname(os.path.abspath(out)), exist_ok=True)
        return [nsys, "profile", "--trace=cuda,nvtx", "--sample=none", "--cpuctxsw=none", "--force-overwrite=true",
                "-o", out] + list(argv), env
    env.setdefault("FORGE_PROFILE_STEP", "5")
    env.setdefault("FORGE_PROFILE_RANK", "0")
    env.setdefault("FORGE_PROFILE_DIR", os.path.dirname(env.get("NSYS_OUTPUT", "")) or "profile_out")
    return argv, env


def launch(argv: list[str], nproc: int, master_port="auto", env=None, stdout=None, stderr=None) -> int:
    port = free_port() if master_port in ("auto", None, 0) else int(master_port)
    procs = []
    for r in range(nproc):
        cmd, renv = profile_wrap(list(argv), r, rank_env(r, nproc, port, env))
        procs.append(subprocess.Popen(cmd, env=renv, stdout=stdout if r == 0 else subprocess.DEVNULL, stderr=stderr))
    return wait_with_fast_fail(procs)


class BoundedTimeout(RuntimeError):
    pass


def run_bounded(argv, timeout_s: float, term_grace_s: float = 30.0, env=None, cwd=None) -> tuple[int, str]:
    """Run in a new session; on timeout SIGTERM the process GROUP, wait, SIGKILL it.  Returns (rc, combined output)."""
    p = subprocess.Popen(argv, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, cwd=cwd,
                         start_new_session=True)
    try:
        out, _ = p.communicate(timeout=timeout_s)
        return p.returncode, out
    except subprocess.TimeoutExpired:
        pgid = os.getpgid(p.pid)
        os.killpg(pgid, signal.SIGTERM)
        try:
            out, _ = p.communicate(timeout=term_grace_s)
        except subprocess.TimeoutExpired:
            os.killpg(pgid, signal.SIGKILL)
            out, _ = p.communicate()
        raise BoundedTimeout(f"command exceeded {timeout_s}s: {' '.join(map(str, argv))}\n{out[-2000:]}")


def gpu_is_dirty(query=None) -> list[str]:
    """PIDs of compute apps nvidia-smi reports (empty when clean or when nvidia-smi is absent)."""
    if query is None:
        def query():
            try:
                return subprocess.run(["nvidia-smi", "--query-compute-apps=pid", "--format=csv,noheader"],
                                      capture_output=True, text=True, timeout=20).stdout
            except (OSError, subprocess.TimeoutExpired):
                return ""
    me = str(os.getpid())
    return [ln.strip() for ln in query().splitlines() if ln.strip() and ln.strip() != me]


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(description="launch one process per rank with fast-fail")
    ap.add_argument("--nproc", type=int, default=int(os.environ.get("NUM_PROCS", "1")))
    ap.add_argument("--master-port", default="auto")
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = a.cmd[1:] if a.cmd and a.cmd[0] == "--" else a.cmd
    sys.exit(launch(cmd, a.nproc, a.master_port))


if __name__ == "__main__":
    main()
