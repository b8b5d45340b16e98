"""Workspace plumbing of the control plane: external-resource manifest, workspace-contract probe, workspace sync, corpus
prefetch and run-directory retention.

* **Resources** (harness/resources.py:89-261 in the reference): ``configs/external_resources.toml`` declares every artefact
  the runs need from outside the tree (tokenizer, corpus, reference checkpoint) as ``[[entry]]`` tables with a ``kind``
  (``file`` | ``tree``), an optional ``sha256`` and a list of ``file://`` sources.  ``provision`` links the first source that
  verifies to ``<workspace>/<canonical_relpath>``; network schemes are refused unless ``FORGE_ALLOW_NETWORK_RESOURCES=1``
  (and there is no network here).  A swapped artefact fails provisioning instead of silently feeding a run other bytes.
* **Workspace contract** (harness/workspace_contract.py): invariants checked before GPU time is spent: the package that
  gets imported is THIS tree (no installed copy shadowing it), the extension is built and newer than its sources, a
  child interpreter resolves the same configuration bytes as this one, the resources are provisioned.
* **Sync** (harness/remote_sync.py): rsync-style push of the workspace to an execution directory, honouring an ignore
  file, with stale ``__pycache__`` removed on the far side.  The execution host here is a local path (or ``host:path``
  when ``rsync`` and a route exist).
* **Prefetch** (tools/prefetch_data.py): stage a corpus next to the trainer; with no network, the source is a local path
  and the step verifies and links it.
* **Retention** (harness/app.py:667): before a new run directory is made, all but the newest N of the same suite go.
"""
from __future__ import annotations

import fnmatch
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tomllib
from dataclasses import dataclass

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
NETWORK_SCHEMES = ("hf://", "git+ssh://", "git+https://", "https://", "http://")


# ---- resources -------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Resource:
    name: str
    kind: str
    sha256: str
    canonical_relpath: str
    sources: tuple


class ResourceError(RuntimeError):
    pass


def load_manifest(path: str | None = None) -> list[Resource]:
    path = path or os.path.join(ROOT, "configs", "external_resources.toml")
    if not os.path.isfile(path):
        return []
    with open(path, "rb") as f:
        doc = tomllib.load(f)
    out = []
    for raw in doc.get("entry", []):
        for k in ("name", "kind", "canonical_relpath", "sources"):
            if k not in raw:
                raise ResourceError(f"manifest entry lacks {k!r}: {raw}")
        if raw["kind"] not in ("file", "tree"):
            raise ResourceError(f"{raw['name']}: kind must be 'file' or 'tree'")
        rel = raw["canonical_relpath"]
        if rel.startswith("/") or ".." in rel.split("/"):
            raise ResourceError(f"{raw['name']}: canonical_relpath must stay inside the workspace")
        out.append(Resource(raw["name"], raw["kind"], raw.get("sha256", ""), rel, tuple(raw["sources"])))
    return out


def sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def sha256_tree(root: str) -> str:
    h = hashlib.sha256()
    for d, _, files in sorted(os.walk(root)):
        for fn in sorted(files):
            p = os.path.join(d, fn)
            h.update(os.path.relpath(p, root).encode() + b"\0" + sha256_file(p).encode() + b"\n")
    return h.hexdigest()


def verify(res: Resource, target: str) -> tuple[bool, str]:
    if res.kind == "file" and not os.path.isfile(target):
        return False, "not a file"
    if res.kind == "tree" and not os.path.isdir(target):
        return False, "not a directory"
    if res.sha256:
        got = sha256_file(target) if res.kind == "file" else sha256_tree(target)
        if got != res.sha256:
            return False, f"sha256 {got[:12]}... does not match the manifest"
    return True, ""


def provision(workspace: str | None = None, manifest: str | None = None) -> list[dict]:
    ws = workspace or ROOT
    allow_net = os.environ.get("FORGE_ALLOW_NETWORK_RESOURCES") == "1"
    report = []
    for res in load_manifest(manifest):
        dest = os.path.join(ws, res.canonical_relpath)
        chosen, reasons = None, []
        for src in res.sources:
            src = os.path.expandvars(src)
            if src.startswith(NETWORK_SCHEMES):
                reasons.append(f"{src}: network source " + ("unreachable here" if allow_net else "not allowed (FORGE_ALLOW_NETWORK_RESOURCES)"))
                continue
            path = src[7:] if src.startswith("file://") else src
            ok, why = verify(res, path)
            if ok:
                chosen = path
                break
            reasons.append(f"{src}: {why}")
        if chosen is None:
            raise ResourceError(f"{res.name}: no source verifies ({'; '.join(reasons) or 'no sources'})")
        os.makedirs(os.path.dirname(dest), exist_ok=True)
        if os.path.islink(dest) or os.path.exists(dest):
            if os.path.islink(dest) or os.path.isfile(dest):
                os.unlink(dest)
            else:
                shutil.rmtree(dest)
        os.symlink(os.path.abspath(chosen), dest)
        report.append({"name": res.name, "linked": dest, "source": chosen})
    return report


def assert_provisioned(workspace: str | None = None, manifest: str | None = None) -> list[str]:
    ws = workspace or ROOT
    missing = []
    for res in load_manifest(manifest):
        ok, why = verify(res, os.path.join(ws, res.canonical_relpath))
        if not ok:
            missing.append(f"{res.name}: {why}")
    return missing


# ---- workspace contract ------------------------------------------------------------------------------------------------------
def env_probe(config_path: str | None = None) -> dict:
    """Returns ``{"passed": bool, "checks": {name: {"ok": bool, "detail": str}}}``."""
    checks = {}

    def put(name, ok, detail=""):
        checks[name] = {"ok": bool(ok), "detail": detail}

    import forge_train_harness_b200 as pkg
    here = os.path.realpath(os.path.join(ROOT, "forge_train_harness_b200"))
    put("package_is_this_tree", os.path.realpath(os.path.dirname(pkg.__file__)) == here, os.path.dirname(pkg.__file__))
    so = os.path.join(here, "_C.so")
    csrc = os.path.join(here, "csrc")
    if os.path.isfile(so):
        newest = max(os.path.getmtime(os.path.join(csrc, f)) for f in os.listdir(csrc) if f.endswith((".cu", ".cuh", ".cpp", ".h")))
        put("extension_built_and_current", os.path.getmtime(so) >= newest, "rebuild with python -m forge_train_harness_b200.csrc.build"
            if os.path.getmtime(so) < newest else "")
    else:
        put("extension_built_and_current", False, "forge_train_harness_b200/_C.so is missing")
    cfg = config_path or os.path.join(ROOT, "configs", "tiny_cpu_dp2.toml")
    try:
        mine = canonical_config_sha(cfg)
        child = subprocess.run([sys.executable, "-c", "import sys; sys.path.insert(0, sys.argv[1]); "
                                "from forge_train_harness_b200.harness.workspace import canonical_config_sha as f; print(f(sys.argv[2]))",
                                ROOT, cfg], capture_output=True, text=True, timeout=120, cwd="/")
        put("subprocess_config_isomorphic", child.returncode == 0 and child.stdout.strip() == mine,
            child.stderr[-300:] if child.returncode else "")
    except Exception as e:  # noqa: BLE001
        put("subprocess_config_isomorphic", False, f"{type(e).__name__}: {e}")
    try:
        missing = assert_provisioned()
        put("resources_provisioned", not missing, "; ".join(missing))
    except ResourceError as e:
        put("resources_provisioned", False, str(e))
    return {"passed": all(c["ok"] for c in checks.values()), "checks": checks}


def canonical_config_sha(path: str) -> str:
    """sha256 of the canonical bytes of a resolved run configuration (what ``echo-config`` prints)."""
    import dataclasses

    from ..config import schema
    cfg = schema.load(path)
    doc = {k: dataclasses.asdict(getattr(cfg, k)) for k in ("model", "optim", "parallel", "train", "data", "ckpt")}
    return hashlib.sha256(json.dumps(doc, sort_keys=True).encode()).hexdigest()


# ---- sync --------------------------------------------------------------------------------------------------------------------
def _ignored(rel: str, patterns: list[str]) -> bool:
    parts = rel.split(os.sep)
    return any(fnmatch.fnmatch(rel, p) or any(fnmatch.fnmatch(x, p.rstrip("/")) for x in parts) for p in patterns)


def sync_push(dest: str, src: str | None = None, ignore_file: str | None = None) -> dict:
    """Copy the workspace to ``dest`` (a directory), skipping ignored paths; files that vanished locally are removed on the
    far side and stale ``__pycache__`` directories are cleaned.  Returns counts."""
    src = src or ROOT
    pats = ["__pycache__", ".git", ".artifacts", "*.pyc"]
    ig = ignore_file or os.path.join(src, ".syncignore")
    if os.path.isfile(ig):
        pats += [ln.strip() for ln in open(ig) if ln.strip() and not ln.startswith("#")]
    copied = removed = 0
    seen = set()
    for d, dirs, files in os.walk(src):
        rel_d = os.path.relpath(d, src)
        dirs[:] = [x for x in dirs if not _ignored(os.path.normpath(os.path.join(rel_d, x)), pats)]
        for fn in files:
            rel = os.path.normpath(os.path.join(rel_d, fn))
            if _ignored(rel, pats):
                continue
            seen.add(rel)
            s, t = os.path.join(src, rel), os.path.join(dest, rel)
            if not os.path.isfile(t) or os.path.getmtime(t) < os.path.getmtime(s) or os.path.getsize(t) != os.path.getsize(s):
                os.makedirs(os.path.dirname(t), exist_ok=True)
                shutil.copy2(s, t)
                copied += 1
    for d, dirs, files in os.walk(dest, topdown=False):
        if os.path.basename(d) == "__pycache__":
            shutil.rmtree(d, ignore_errors=True)
            continue
        for fn in files:
            rel = os.path.normpath(os.path.relpath(os.path.join(d, fn), dest))
            if rel not in seen and not _ignored(rel, pats):
                os.unlink(os.path.join(d, fn))
                removed += 1
    ok = os.path.isfile(os.path.join(dest, "forge_train_harness_b200", "__init__.py"))
    return {"passed": ok, "copied": copied, "removed": removed, "dest": dest}


# ---- prefetch ------------------------------------------------------------------------------------------------------------------
def prefetch(source_prefix: str, data_dir: str, target_gb: float = 0.0) -> dict:
    """Stage ``<source_prefix>.bin/.idx`` into ``data_dir`` (link when on the same filesystem, else copy) and check that the
    index parses.  ``target_gb`` > 0 stops early when the corpus is smaller than asked for."""
    from ..data.sources import MegatronBinary
    os.makedirs(data_dir, exist_ok=True)
    out = {}
    for ext in (".bin", ".idx"):
        s = source_prefix + ext
        if not os.path.isfile(s):
            return {"passed": False, "reason": f"{s} does not exist (no network: the corpus must already be on this host)"}
        t = os.path.join(data_dir, os.path.basename(s))
        if os.path.lexists(t):
            os.unlink(t)
        try:
            os.link(s, t)
        except OSError:
            shutil.copy2(s, t)
        out[ext] = t
    size_gb = os.path.getsize(out[".bin"]) / 1e9
    src = MegatronBinary(out[".bin"][:-4], 16, 1, 0, 1, 0)
    ok = src.n_local > 0 and (target_gb <= 0 or size_gb >= target_gb)
    return {"passed": ok, "prefix": out[".bin"][:-4], "size_gb": size_gb, "windows_of_17_tokens": int(src.n_local)}


# ---- retention -------------------------------------------------------------------------------------------------------------------
def prune_old_runs(runs_root: str, suite: str, keep: int) -> list[str]:
    """Delete all but the newest ``keep`` directories ``<runs_root>/<suite>-*`` (0 = keep everything)."""
    if keep <= 0 or not os.path.isdir(runs_root):
        return []
    mine = sorted((d for d in os.listdir(runs_root) if d.startswith(suite + "-") and os.path.isdir(os.path.join(runs_root, d))),
                  key=lambda d: os.path.getmtime(os.path.join(runs_root, d)))
    gone = mine[:-keep] if len(mine) > keep else []
    for d in gone:
        shutil.rmtree(os.path.join(runs_root, d), ignore_errors=True)
    return gone
