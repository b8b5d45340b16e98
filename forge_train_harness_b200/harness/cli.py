"""Harness command line (the counterpart of ``bin/harness`` -> harness/cli.py:70-213).

    python -m forge_train_harness_b200.harness run <suite> [--registry configs/eval/dense_training.toml] [--timeout S] [--arg k=v]
    python -m forge_train_harness_b200.harness guard | anti-proxy | unit | info | doctor | echo-config <toml> | render <gate.toml> ...
    python -m forge_train_harness_b200.harness sweep [--stage stage1] [--max-gpus N] | budget <suite> | env-probe | resources provision|verify | prefetch <prefix> <dir> | sync push <dest>
    python -m forge_train_harness_b200.harness op-inventory | op-status | op-long <op> --config <toml> [--steps N --window A B --nproc N]
    python -m forge_train_harness_b200.harness lease claim|release|rebind|list ... | job <suite> --outer S [--poll] | loop run|report|fork ... | tools canonical|recipe-env|data-check|capture-batch ...

``FORGE_EVAL_FAMILY`` picks the suite registry (dense_training | dense_training_1b | dense_training_8b | dense_training_qwen3).

Local suites (``guard``, ``anti-proxy``, ``unit``) run in-process / as a pytest child; gate suites go request -> dispatcher ->
result JSON between the result markers.  Timeout precedence: ``--timeout`` > ``HARNESS_RUN_TIMEOUT_S`` > the registry value.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

from ..config import schema
from . import dispatcher, guards, render, stage2, workspace
from . import run_schema as RS

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _timeout(cli_value, registry_value):
    if cli_value:
        return float(cli_value)
    env = os.environ.get("HARNESS_RUN_TIMEOUT_S")
    return float(env) if env else float(registry_value)


def _registry_default() -> str:
    """Suite registry of the active eval family: ``FORGE_EVAL_FAMILY`` = dense_training (0.5B, default) | dense_training_1b |
    dense_training_8b | dense_training_qwen3 (config/eval/<family>/<family>.toml in the reference)."""
    fam = os.environ.get("FORGE_EVAL_FAMILY", "dense_training")
    return os.path.join(ROOT, "configs", "eval", fam + ".toml")


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv[:1] == ["lease"]:      # GPU lease registry, short-lived GPU jobs and the development loop keep their own parsers
        from . import lease
        return lease.main(argv[1:])
    if argv[:1] == ["job"]:
        from . import jobs
        return jobs.main(argv[1:])
    if argv[:1] == ["loop"]:
        from . import loop
        return loop.main(argv[1:])
    if argv[:1] == ["tools"]:      # canonical | recipe-env | data-check | capture-batch
        from . import tools
        return tools.main(argv[1:])
    ap = argparse.ArgumentParser(prog="harness")
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run")
    r.add_argument("suite")
    r.add_argument("--registry", default=_registry_default())
    r.add_argument("--timeout", type=float, default=0.0)
    r.add_argument("--arg", action="append", default=[])
    r.add_argument("--artifacts", default=os.path.join(ROOT, ".artifacts", "runs"))
    for name in ("guard", "anti-proxy", "unit", "info", "doctor", "env", "env-probe", "op-inventory", "op-status"):
        sub.add_parser(name)
    sw = sub.add_parser("sweep", help="run every suite of a stage (optionally only those needing no GPU) and print one table")
    sw.add_argument("--registry", default=_registry_default())
    sw.add_argument("--stage", default="stage1")
    sw.add_argument("--max-gpus", type=int, default=-1, help="skip suites that need more GPUs than this (-1: whatever is visible)")
    sw.add_argument("--only", default="", help="comma-separated suite names")
    sw.add_argument("--artifacts", default=os.path.join(ROOT, ".artifacts", "runs"))
    b = sub.add_parser("budget")
    b.add_argument("suite")
    b.add_argument("--registry", default=_registry_default())
    b.add_argument("--json", action="store_true")
    rs = sub.add_parser("resources")
    rs.add_argument("action", choices=["provision", "verify"])
    pf = sub.add_parser("prefetch")
    pf.add_argument("source_prefix")
    pf.add_argument("data_dir")
    pf.add_argument("--target-gb", type=float, default=0.0)
    sy = sub.add_parser("sync")
    sy.add_argument("action", choices=["push"])
    sy.add_argument("dest")
    ol = sub.add_parser("op-long")
    ol.add_argument("op")
    ol.add_argument("--config", required=True)
    ol.add_argument("--steps", type=int, default=200)
    ol.add_argument("--window", type=int, nargs=2, default=[101, 201])
    ol.add_argument("--nproc", type=int, default=1)
    ol.add_argument("--version", default=None)
    ol.add_argument("--set", action="append", default=[])
    e = sub.add_parser("echo-config")
    e.add_argument("path")
    rn = sub.add_parser("render")
    rn.add_argument("gate")
    rn.add_argument("--model", required=True)
    rn.add_argument("--optim", required=True)
    rn.add_argument("--registry", default=_registry_default())
    a = ap.parse_args(argv)

    if a.cmd == "guard":
        res = guards.framework_guard()
        print(json.dumps(res))
        return 0 if res["passed"] else 1
    if a.cmd == "anti-proxy":
        res = guards.anti_proxy_guard()
        print(json.dumps(res))
        return 0 if res["passed"] else 1
    if a.cmd == "unit":
        return subprocess.call([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests"), "-q", "-m", "not gpu"])
    if a.cmd == "env":
        from . import env_check
        return env_check.main([])
    if a.cmd == "env-probe":
        res = workspace.env_probe()
        print(json.dumps(res, indent=1))
        return 0 if res["passed"] else 2
    if a.cmd == "budget":
        gate = render.load_toml(a.registry).get("evals", {}).get(a.suite)
        if gate is None:
            print(f"unknown suite {a.suite!r}", file=sys.stderr)
            return 1
        env = os.environ.get("HARNESS_RUN_TIMEOUT_S")
        t, src = (float(env), "HARNESS_RUN_TIMEOUT_S") if env else (float(gate.get("timeout_s", 600)), "registry")
        print(json.dumps({"suite": a.suite, "timeout_s": t, "source": src}) if a.json else int(t))
        return 0
    if a.cmd == "resources":
        try:
            if a.action == "provision":
                print(json.dumps(workspace.provision(), indent=1))
                return 0
            missing = workspace.assert_provisioned()
            print(json.dumps({"missing": missing}))
            return 0 if not missing else 1
        except workspace.ResourceError as e:
            print(str(e), file=sys.stderr)
            return 1
    if a.cmd == "prefetch":
        res = workspace.prefetch(a.source_prefix, a.data_dir, a.target_gb)
        print(json.dumps(res))
        return 0 if res["passed"] else 1
    if a.cmd == "sync":
        res = workspace.sync_push(a.dest)
        print(json.dumps(res))
        return 0 if res["passed"] else 1
    if a.cmd in ("op-inventory", "op-status"):
        r = stage2.op_inventory() if a.cmd == "op-inventory" else stage2.op_status()
        RS.emit_result(stage2.as_result(a.cmd, r), sys.stdout)
        return 0 if r["passed"] else 1
    if a.cmd == "op-long":
        r = stage2.op_long(a.op, a.config, a.steps, tuple(a.window), nproc=a.nproc, version=a.version, extra_sets=a.set)
        RS.emit_result(stage2.as_result("op-long", r), sys.stdout)
        return 0 if r.get("passed") else 1
    if a.cmd == "info":
        print(json.dumps({"result_markers": [RS.RESULT_BEGIN, RS.RESULT_END], "runner_metrics": RS.RUNNER_METRICS,
                          "schema_version": RS.RUN_SCHEMA_VERSION}, indent=1))
        return 0
    if a.cmd == "doctor":
        import torch
        info = {"torch": torch.__version__, "cuda_available": torch.cuda.is_available(),
                "extension_built": os.path.isfile(os.path.join(ROOT, "forge_train_harness_b200", "_C.so")),
                "reference_installed": os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "training_engine_tensor"))}
        if torch.cuda.is_available():
            info["gpus"] = [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())]
        print(json.dumps(info, indent=1))
        return 0
    if a.cmd == "echo-config":
        import dataclasses
        cfg = schema.load(a.path)
        print(json.dumps({k: dataclasses.asdict(getattr(cfg, k)) for k in ("model", "optim", "parallel", "train", "data", "ckpt")}, indent=1))
        return 0
    if a.cmd == "render":
        reg = render.load_toml(a.registry)
        prods = render.render_gate(render.load_toml(a.gate), render.load_toml(a.model)["model"], render.load_toml(a.optim)["optim"],
                                   reg.get("env", {}), reg.get("defaults", {}).get("seed", 1234))
        for side in ("ref", "ours"):
            print(f"# ---- {side} product ----\n" + render.dumps_product(prods[side]))
        return 0
    if a.cmd == "sweep":
        # the reference's env/gate_sweep_torch.sh: every gate of the ladder in milestone order, one line each
        reg = render.load_toml(a.registry)
        have = a.max_gpus
        if have < 0:
            try:
                import torch
                have = torch.cuda.device_count()
            except Exception:
                have = 0
        order = (reg.get(a.stage) or {}).get("milestone_order", [])
        rank = {m: i for i, m in enumerate(order)}
        names = [n for n, g in reg.get("evals", {}).items() if g.get("stage", "stage1") == a.stage]
        if a.only:
            names = [n for n in names if n in a.only.split(",")]
        names.sort(key=lambda n: (rank.get(str(reg["evals"][n].get("milestone", "")).split(".")[0], 99), n))
        rows, failed = [], 0
        for n in names:
            g = reg["evals"][n]
            if int(g.get("gpu_count", 0)) > have and not (have == 0 and "tiny_cpu" in json.dumps(g)):
                rows.append((n, g.get("milestone", "-"), "skipped", f"needs {g.get('gpu_count')} GPUs, {have} visible"))
                continue
            rc = main(["run", n, "--registry", a.registry, "--artifacts", a.artifacts])
            failed += rc != 0
            rows.append((n, g.get("milestone", "-"), "passed" if rc == 0 else "FAILED", ""))
        print("\n| suite | milestone | status | note |\n|---|---|---|---|")
        for r in rows:
            print("| " + " | ".join(r) + " |")
        return 1 if failed else 0
    # run <suite>
    reg = render.load_toml(a.registry)
    gate = reg.get("evals", {}).get(a.suite, {})
    args = dict(kv.split("=", 1) for kv in a.arg)
    args["timeout_s"] = _timeout(a.timeout, gate.get("timeout_s", 600))
    req = RS.make_run_request(a.suite, args, gate.get("gpu_count", 1))
    # sliding-window retention: all but the newest N run directories of this suite go before the new one is made
    workspace.prune_old_runs(a.artifacts, a.suite, int(reg.get("artifacts", {}).get("retention", {}).get("per_suite", 0)))
    art = os.path.join(a.artifacts, req["run_id"])
    os.makedirs(art, exist_ok=True)
    with open(os.path.join(art, "request.json"), "w") as f:
        json.dump(req, f, indent=1)
    res = dispatcher.run_suite(req, reg, ROOT, art, cache_dir=os.path.join(ROOT, ".artifacts", "ref_cache"))
    from . import mfu
    mfu.record_result(res)
    RS.emit_result(res, sys.stdout)
    return 0 if res["status"] == "passed" else 1


if __name__ == "__main__":
    sys.exit(main())
