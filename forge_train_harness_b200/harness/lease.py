"""Exclusive GPU leases for development loops that share one node (or one external scheduler).

What the reference's ``tools/lease.py`` does for its cluster (lease.py:519-661): every loop claims an exclusive machine during
bootstrap, the claim is idempotent per loop id, a flock-guarded ``registry.json`` plus a per-loop reverse-lookup file say
who holds what, ``release`` drops the row first and stops the machine afterwards, ``rebind`` re-points a lease at a
recovered machine without stopping the dead one.  The same contract here, with the machine behind a small provider
interface instead of one vendor CLI:

* ``LocalGpuProvider`` — the resource is a set of GPU ordinals of THIS node (the natural unit on an 8 x B200 NVSwitch box,
  where every subset of GPUs has the same all-to-all bandwidth, so any free ordinals will do).  A lease is live while its
  holder process is alive; a holder that died without releasing is reclaimed by the next claimer.
* ``CommandProvider`` — an external scheduler driven by argv templates from the ``[remote.provider]`` table
  (``create`` / ``phase`` / ``stop``), the form the reference hard-codes for ``cctl``.  Tests inject a fake executable.

Storage (all under ``<root>/lease/<resource>/``): ``.registry.lock`` (flock guard), ``registry.json``
(``{handle: {loop_id, task_id, claimed_at, ...}}``), ``<loop_id>.handle`` (reverse lookup for ``release``).

CLI: ``python -m forge_train_harness_b200.harness.lease claim|release|rebind|list ...``.
"""
from __future__ import annotations

import argparse
import contextlib
import datetime as _dt
import fcntl
import json
import os
import re
import shlex
import subprocess
import sys
import time
from dataclasses import dataclass, field

__all__ = ["LeaseError", "LeaseBusyError", "LeaseTimeoutError", "LeaseSpec", "LocalGpuProvider", "CommandProvider",
           "claim", "release", "rebind", "holders", "main"]

TERMINAL_PHASES = frozenset({"succeeded", "failed", "stopped", "unknown"})
READY_PHASES = frozenset({"running"})


class LeaseError(RuntimeError):
    pass


class LeaseTimeoutError(LeaseError):
    pass


class LeaseBusyError(LeaseError):
    pass


@dataclass(frozen=True)
class LeaseSpec:
    """What a loop asks for.  ``gpu_count = 0`` is a pure filesystem gateway (the reference's ``kind = "job"`` lease)."""
    gpu_count: int = 1
    labels: dict = field(default_factory=dict)  # free-form: project, pool, image, priority ... passed to the provider

    def template_vars(self) -> dict:
        out = {"gpu_count": str(self.gpu_count)}
        out.update({k: str(v) for k, v in self.labels.items()})
        return out


def _root() -> str:
    base = os.environ.get("FORGE_LEASE_DIR")
    if base:
        return base
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    return os.path.join(here, ".artifacts", "lease")


def _dir(resource: str) -> str:
    if not re.fullmatch(r"[A-Za-z0-9_.-]+", resource or ""):
        raise LeaseError(f"bad lease resource name {resource!r}")
    d = os.path.join(_root(), resource)
    os.makedirs(d, exist_ok=True)
    return d


def _reverse_path(resource: str, loop_id: str) -> str:
    if not re.fullmatch(r"[A-Za-z0-9_.-]+", loop_id or ""):
        raise LeaseError("loop_id must be non-empty and made of [A-Za-z0-9_.-]")
    return os.path.join(_dir(resource), loop_id + ".handle")


class _RegistryLock:
    """``flock`` on ``.registry.lock`` with a bounded wait (a holder that hangs must not wedge every other loop)."""

    def __init__(self, resource: str, timeout_s: float = 60.0):
        self.path = os.path.join(_dir(resource), ".registry.lock")
        self.timeout_s = timeout_s
        self.fd = None

    def __enter__(self):
        self.fd = os.open(self.path, os.O_CREAT | os.O_RDWR, 0o644)
        end = time.monotonic() + self.timeout_s
        while True:
            try:
                fcntl.flock(self.fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
                return self
            except OSError:
                if time.monotonic() >= end:
                    os.close(self.fd)
                    self.fd = None
                    raise LeaseTimeoutError(f"lease registry lock {self.path} not acquired in {self.timeout_s:.0f}s")
                time.sleep(0.05)

    def __exit__(self, *exc):
        if self.fd is not None:
            fcntl.flock(self.fd, fcntl.LOCK_UN)
            os.close(self.fd)
            self.fd = None


def _read_registry(resource: str) -> dict:
    p = os.path.join(_dir(resource), "registry.json")
    try:
        with open(p, encoding="utf-8") as f:
            data = json.load(f)
    except FileNotFoundError:
        return {}
    except json.JSONDecodeError as e:
        raise LeaseError(f"lease registry {p} is not valid JSON: {e}") from e
    if not isinstance(data, dict):
        raise LeaseError(f"lease registry {p} must hold an object")
    return data


def _write_registry(resource: str, payload: dict) -> None:
    p = os.path.join(_dir(resource), "registry.json")
    tmp = p + f".tmp{os.getpid()}"
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(payload, f, indent=1, sort_keys=True)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, p)


def _now() -> str:
    return _dt.datetime.now(_dt.timezone.utc).isoformat(timespec="seconds")


def _pid_alive(pid: int) -> bool:
    if pid <= 0:
        return False
    try:
        os.kill(pid, 0)
    except ProcessLookupError:
        return False
    except PermissionError:
        return True
    return True


def _pid_start(pid: int) -> str:
    """Start time of a process in clock ticks since boot (field 22 of /proc/<pid>/stat); "" where /proc is not available.
    Recorded with a lease so that a recycled process id is not mistaken for the holder."""
    try:
        with open(f"/proc/{int(pid)}/stat", "rb") as f:
            data = f.read().decode("ascii", "replace")
        return data[data.rindex(")") + 2:].split()[19]
    except (OSError, ValueError, IndexError):
        return ""


# ---- providers -------------------------------------------------------------------------------------------------------------
class LocalGpuProvider:
    """GPU ordinals of this node.  The handle is ``gpu-<i>[-<j>...]``; the task id is the holder's pid.

    ``allocate`` runs INSIDE the registry lock (choosing free ordinals and recording them must be one atomic step; an
    external scheduler's create, which takes minutes, runs outside it instead — see ``claim``)."""
    inside_lock = True

    def __init__(self, total_gpus: int | None = None, holder_pid: int | None = None):
        self.total = total_gpus if total_gpus is not None else self._count_gpus()
        self.holder_pid = holder_pid if holder_pid is not None else os.getpid()

    @staticmethod
    def _count_gpus() -> int:
        env = os.environ.get("FORGE_LEASE_TOTAL_GPUS")
        if env:
            return int(env)
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                return int(pynvml.nvmlDeviceGetCount())
            finally:
                pynvml.nvmlShutdown()
        except Exception:
            return 0

    @staticmethod
    def ordinals(handle: str) -> list[int]:
        if handle.startswith("gpu-none"):   # a GPU-less gateway lease ("gpu-none@<loop>")
            return []
        if not handle.startswith("gpu-"):
            raise LeaseError(f"not a local GPU lease handle: {handle!r}")
        return [int(x) for x in handle[4:].split("-")]

    def live(self, row: dict) -> bool:
        pid = int(row.get("task_id", 0) or 0)
        if not _pid_alive(pid):
            return False
        born = row.get("task_start", "")
        return not born or _pid_start(pid) in ("", born)     # same pid, other start time: the holder is gone, the pid was reused

    def allocate(self, spec: LeaseSpec, registry: dict) -> tuple[str, str, list[str]]:
        """Returns (handle, task_id, reclaimed handles).  Raises ``LeaseBusyError`` when too few ordinals are free."""
        reclaimed = [h for h, row in registry.items() if not self.live(row)]
        taken = set()
        for h, row in registry.items():
            if h not in reclaimed:
                taken.update(self.ordinals(h))
        free = [i for i in range(self.total) if i not in taken]
        if spec.gpu_count == 0:
            return "gpu-none", str(self.holder_pid), reclaimed
        if len(free) < spec.gpu_count:
            raise LeaseBusyError(f"{spec.gpu_count} GPUs wanted, {len(free)} of {self.total} free")
        # keep a lease inside one aligned group where it fits (2, 4 or 8 neighbours share a die pair / a host bridge), so
        # two 4-GPU loops split the box in halves instead of interleaving
        want = spec.gpu_count
        pick = None
        for start in range(0, self.total, max(want, 1)):
            grp = list(range(start, min(start + want, self.total)))
            if len(grp) == want and all(g in free for g in grp):
                pick = grp
                break
        pick = pick or free[:want]
        return "gpu-" + "-".join(str(i) for i in pick), str(self.holder_pid), reclaimed

    def phase(self, task_id: str) -> str:
        return "running" if _pid_alive(int(task_id or 0)) else "stopped"

    def stop(self, task_id: str) -> None:  # the holder is the loop itself; nothing to stop
        return None

    def env(self, handle: str) -> dict:
        return {"CUDA_VISIBLE_DEVICES": ",".join(str(i) for i in self.ordinals(handle))}


class CommandProvider:
    """An external scheduler behind argv templates::

        [remote.provider]
        create = ["sched", "box", "create", "--gpus", "{gpu_count}", "--pool", "{pool}"]
        id_regex = "tasks/([0-9a-f]+)"
        phase  = ["sched", "box", "get", "tasks/{task_id}", "--field", "phase"]
        stop   = ["sched", "box", "stop", "--yes", "tasks/{task_id}"]
        handle = "box-{task_id}"
        phase_map = {Running = "running", Queued = "queued", Succeeded = "succeeded", Failed = "failed"}

    A create that fails with a message matching ``retry_regex`` made no task and is re-issued (bounded), the transient
    look-up flake the reference retries (lease.py:264-295)."""
    inside_lock = False

    def __init__(self, table: dict):
        for k in ("create", "phase", "stop"):
            if not isinstance(table.get(k), list) or not table[k]:
                raise LeaseError(f"[remote.provider].{k} must be a non-empty argv list")
        self.t = table
        self.id_re = re.compile(table.get("id_regex", r"([A-Za-z0-9_.-]+)\s*$"))
        self.retry_re = re.compile(table["retry_regex"]) if table.get("retry_regex") else None
        self.handle_fmt = table.get("handle", "box-{task_id}")
        self.phase_map = {str(k).lower(): str(v) for k, v in (table.get("phase_map") or {}).items()}

    def _run(self, argv: list[str], **vars_) -> subprocess.CompletedProcess:
        try:
            cmd = [a.format(**vars_) for a in argv]
        except KeyError as e:
            raise LeaseError(f"provider template names {e} which the lease spec does not define") from e
        try:
            return subprocess.run(cmd, capture_output=True, text=True, timeout=float(self.t.get("call_timeout_s", 120)))
        except FileNotFoundError as e:
            raise LeaseError(f"provider executable not found: {cmd[0]}") from e
        except subprocess.TimeoutExpired as e:
            raise LeaseError(f"provider call timed out: {shlex.join(cmd)}") from e

    def create(self, spec: LeaseSpec, tries: int = 3) -> str:
        last = None
        for attempt in range(tries):
            r = self._run(self.t["create"], **spec.template_vars())
            if r.returncode == 0:
                m = self.id_re.search(r.stdout)
                if not m:
                    raise LeaseError(f"provider create printed no task id: {r.stdout[-300:]!r}")
                return m.group(1)
            last = (r.stderr or r.stdout)[-400:]
            if not (self.retry_re and self.retry_re.search(last)):
                break
            time.sleep(min(2.0 * (attempt + 1), 10.0) * float(self.t.get("retry_sleep_scale", 1.0)))
        raise LeaseError(f"provider create failed: {last}")

    def handle(self, task_id: str) -> str:
        return self.handle_fmt.format(task_id=task_id)

    def task_of(self, handle: str) -> str:
        pre, _, post = self.handle_fmt.partition("{task_id}")
        if handle.startswith(pre) and handle.endswith(post) and len(handle) > len(pre) + len(post):
            return handle[len(pre):len(handle) - len(post)] if post else handle[len(pre):]
        return handle

    def phase(self, task_id: str) -> str:
        r = self._run(self.t["phase"], task_id=task_id)
        if r.returncode != 0:
            return "unknown"
        raw = r.stdout.strip().splitlines()[-1].strip() if r.stdout.strip() else ""
        return self.phase_map.get(raw.lower(), raw.lower() or "unknown")

    def stop(self, task_id: str) -> None:
        r = self._run(self.t["stop"], task_id=task_id)
        if r.returncode != 0:
            raise LeaseError(f"provider stop failed: {(r.stderr or r.stdout)[-300:]}")

    def live(self, row: dict) -> bool:
        return self.phase(str(row.get("task_id", ""))) not in TERMINAL_PHASES

    def env(self, handle: str) -> dict:
        return {"FORGE_REMOTE_HANDLE": handle}


def provider_from_config(remote: dict | None):
    """``[remote]`` table -> provider.  ``kind = "local"`` (or no table) leases ordinals of this node."""
    remote = remote or {}
    kind = remote.get("kind", "local")
    if kind == "local":
        return LocalGpuProvider(total_gpus=remote.get("total_gpus"))
    if kind in ("scheduler", "job"):
        return CommandProvider(remote.get("provider") or {})
    raise LeaseError(f"[remote].kind must be 'local', 'scheduler' or 'job', not {kind!r}")


# ---- the three verbs --------------------------------------------------------------------------------------------------------
def claim(resource: str, *, spec: LeaseSpec, loop_id: str, provider=None, timeout: float = 600.0, poll_s: float = 5.0) -> str:
    """Lease an exclusive resource for ``loop_id``; returns its handle.  Idempotent: a loop that already holds a live lease
    gets the same handle back.  With a local provider and no free GPUs, waits (bounded by ``timeout``) for a release."""
    provider = provider or LocalGpuProvider()
    rev = _reverse_path(resource, loop_id)
    if os.path.exists(rev):
        handle = open(rev, encoding="utf-8").read().strip()
        with _RegistryLock(resource):
            row = _read_registry(resource).get(handle)
        if row and row.get("loop_id") == loop_id and provider.live(row):
            return handle
    end = time.monotonic() + timeout
    if provider.inside_lock:
        while True:
            with _RegistryLock(resource):
                reg = _read_registry(resource)
                try:
                    handle, task_id, reclaimed = provider.allocate(spec, reg)
                except LeaseBusyError:
                    handle = None
                if handle is not None:
                    for h in reclaimed:
                        dead = reg.pop(h, None)
                        if dead:
                            with contextlib.suppress(FileNotFoundError, LeaseError):
                                os.unlink(_reverse_path(resource, dead.get("loop_id", "")))
                    key = handle if handle != "gpu-none" else f"gpu-none@{loop_id}"
                    reg[key] = {"loop_id": loop_id, "task_id": task_id, "task_start": _pid_start(int(task_id)), "claimed_at": _now(),
                                "gpu_count": spec.gpu_count}
                    _write_registry(resource, reg)
                    with open(rev, "w", encoding="utf-8") as f:
                        f.write(key + "\n")
                    return key
            if time.monotonic() >= end:
                raise LeaseTimeoutError(f"no {spec.gpu_count} free GPUs for loop {loop_id} within {timeout:.0f}s")
            time.sleep(poll_s)
    # external scheduler: the slow create and the wait for readiness happen outside the lock
    task_id = provider.create(spec)
    while True:
        ph = provider.phase(task_id)
        if ph in READY_PHASES:
            break
        if ph in TERMINAL_PHASES:
            raise LeaseError(f"leased task {task_id} ended in phase {ph!r} before it was ready")
        if time.monotonic() >= end:
            with contextlib.suppress(LeaseError):
                provider.stop(task_id)
            raise LeaseTimeoutError(f"leased task {task_id} not ready within {timeout:.0f}s (stopped)")
        time.sleep(poll_s)
    handle = provider.handle(task_id)
    with _RegistryLock(resource):
        reg = _read_registry(resource)
        reg[handle] = {"loop_id": loop_id, "task_id": task_id, "claimed_at": _now(), "gpu_count": spec.gpu_count}
        _write_registry(resource, reg)
        with open(rev, "w", encoding="utf-8") as f:
            f.write(handle + "\n")
    return handle


def release(resource: str, *, loop_id: str, provider=None) -> None:
    """Drop ``loop_id``'s registry row, then stop what it leased.  Best effort: nothing held -> returns silently."""
    provider = provider or LocalGpuProvider()
    rev = _reverse_path(resource, loop_id)
    if not os.path.exists(rev):
        return
    handle = open(rev, encoding="utf-8").read().strip()
    with _RegistryLock(resource):
        reg = _read_registry(resource)
        row = reg.get(handle)
        if row is not None and row.get("loop_id") == loop_id:
            reg.pop(handle)
            _write_registry(resource, reg)
        else:
            row = None  # the handle was re-leased to somebody else meanwhile: theirs to stop, not ours
        with contextlib.suppress(FileNotFoundError):
            os.unlink(rev)
    if row and row.get("task_id"):
        with contextlib.suppress(LeaseError):
            provider.stop(str(row["task_id"]))


def rebind(resource: str, *, loop_id: str, handle: str, provider=None) -> None:
    """Point ``loop_id``'s lease at ``handle`` (a machine re-created after the leased one dropped) WITHOUT stopping the old
    one — it is gone already, which is why recovery ran — so that ``release`` later stops the machine actually in use."""
    if not handle:
        raise LeaseError("handle must be non-empty")
    provider = provider or LocalGpuProvider()
    rev = _reverse_path(resource, loop_id)
    task_id = provider.task_of(handle) if hasattr(provider, "task_of") else str(getattr(provider, "holder_pid", os.getpid()))
    with _RegistryLock(resource):
        reg = _read_registry(resource)
        other = reg.get(handle)
        if other and other.get("loop_id") != loop_id and provider.live(other):
            raise LeaseBusyError(f"{handle} is leased to loop {other.get('loop_id')}")
        if os.path.exists(rev):
            old = open(rev, encoding="utf-8").read().strip()
            if reg.get(old, {}).get("loop_id") == loop_id:
                reg.pop(old, None)
        reg[handle] = {"loop_id": loop_id, "task_id": task_id, "claimed_at": _now()}
        _write_registry(resource, reg)
        with open(rev, "w", encoding="utf-8") as f:
            f.write(handle + "\n")


def holders(resource: str) -> dict:
    with _RegistryLock(resource):
        return _read_registry(resource)


# ---- CLI --------------------------------------------------------------------------------------------------------------------
def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="lease")
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("claim")
    c.add_argument("resource")
    c.add_argument("--loop-id", required=True)
    c.add_argument("--gpus", type=int, default=1)
    c.add_argument("--timeout", type=float, default=600.0)
    c.add_argument("--holder-pid", type=int, default=0, help="process whose life the lease follows (default: the parent shell)")
    c.add_argument("--label", action="append", default=[], help="key=value passed to the provider's templates")
    r = sub.add_parser("release")
    r.add_argument("resource")
    r.add_argument("--loop-id", required=True)
    b = sub.add_parser("rebind")
    b.add_argument("resource")
    b.add_argument("--loop-id", required=True)
    b.add_argument("--handle", required=True)
    ls = sub.add_parser("list")
    ls.add_argument("resource")
    for p in (c, r, b):
        p.add_argument("--remote-toml", default="", help="file with a [remote] table; default: local GPU ordinals")
    a = ap.parse_args(argv)
    try:
        prov = None
        if a.cmd != "list":
            remote = {}
            if a.remote_toml:
                import tomllib
                with open(a.remote_toml, "rb") as f:
                    remote = tomllib.load(f).get("remote", {})
            prov = provider_from_config(remote)
            if isinstance(prov, LocalGpuProvider) and a.cmd == "claim":
                prov.holder_pid = a.holder_pid or os.getppid()
        if a.cmd == "claim":
            labels = dict(x.split("=", 1) for x in a.label)
            print(claim(a.resource, spec=LeaseSpec(a.gpus, labels), loop_id=a.loop_id, provider=prov, timeout=a.timeout))
        elif a.cmd == "release":
            release(a.resource, loop_id=a.loop_id, provider=prov)
        elif a.cmd == "rebind":
            rebind(a.resource, loop_id=a.loop_id, handle=a.handle, provider=prov)
        else:
            print(json.dumps(holders(a.resource), indent=1, sort_keys=True))
    except LeaseBusyError as e:
        print(f"lease: busy: {e}", file=sys.stderr)
        return 3
    except LeaseTimeoutError as e:
        print(f"lease: timeout: {e}", file=sys.stderr)
        return 4
    except LeaseError as e:
        print(f"lease: {e}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
