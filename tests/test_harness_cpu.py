"""Harness control plane on CPU: schema, renderer, guards, MFU bar, dispatcher with fake side scripts, real CPU gates."""
import json
import os
import sys

import pytest

from forge_train_harness_b200.harness import dispatcher, guards, mfu, render
from forge_train_harness_b200.harness import run_schema as RS
from forge_train_harness_b200.harness.cli import main as cli_main

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_run_schema_roundtrip_and_validation():
    req = RS.make_run_request("long-train", {"x": 1})
    RS.validate_run_request(req)
    bad = dict(req, artifact_relpath="../escape")
    with pytest.raises(ValueError):
        RS.validate_run_request(bad)
    res = RS.make_run_result("long-train", True, "ok", {"mean_rel_diff": 0.0, "max_rel_diff": 0.0, "threshold": 0.01})
    RS.validate_run_result(res, "long_train")
    with pytest.raises(ValueError):
        RS.validate_run_result(RS.make_run_result("x", True, "ok", {}), "long_train")
    import io
    buf = io.StringIO()
    RS.emit_result(res, buf)
    assert RS.extract_result("noise\n" + buf.getvalue() + "more") == res and RS.extract_result("nothing") is None


def test_render_layers_overrides_unset_and_transport_split():
    gate = render.load_toml(os.path.join(ROOT, "configs", "eval", "gate_config", "long-train.toml"))
    reg = render.load_toml(os.path.join(ROOT, "configs", "eval", "dense_training.toml"))
    model = {"num_layers": 24, "hidden_size": 1024}
    optim = {"lr": 3e-4, "lr_warmup_iters": 2000}
    p = render.render_gate(gate, model, optim, reg["env"], 1234)
    assert p["ref"]["cli"]["micro_batch_size"] == 2 and p["ours"]["cli"]["micro_batch_size"] == 4  # side override wins
    assert p["ref"]["cli"]["grad_accum_steps"] == 20 and p["ours"]["cli"]["grad_accum_steps"] == 10
    assert p["ours"]["cli"]["lr_warmup_iters"] == 0 and p["ours"]["cli"]["seed"] == 1234
    assert "NCCL_NVLS_ENABLE" in p["ref"]["env"] and "NCCL_NVLS_ENABLE" not in p["ours"]["env"]  # "@unset" tombstone
    assert p["ours"]["env"]["NUM_PROCS"] == 2 and p["ours"]["env"]["DETERMINISTIC"] is False
    assert not any(k.startswith("review_") or k.startswith("mfu_elastic") for k in p["ours"]["cli"])  # review-only keys stripped
    text = render.dumps_product(p["ours"])
    import tomllib
    assert tomllib.loads(text)["cli"]["gate_window"] == [101, 201]
    env = render.product_env({"cli": {"a": True, "w": [1, 2], "r": "<runtime>", "p": "<auto-port>"}, "env": {"X": "y"}}, lambda: 4242)
    assert env == ["export A='1'", "export W='1 2'", "export P='4242'", "export X='y'"]


def test_guards_pass_on_engine_and_catch_violations(tmp_path):
    assert guards.framework_guard()["passed"] and guards.anti_proxy_guard()["passed"]
    (tmp_path / "models").mkdir()
    (tmp_path / "models" / "bad.py").write_text('"""torch.optim in a docstring is fine"""\nimport torch\n# loss.backward( in a comment is fine\n'
                                                "opt = torch.optim.AdamW([])\nx.sum().backward()\nimport training_engine_tensor\n")
    v = {w for _, w in guards.framework_guard(str(tmp_path))["violations"]}
    assert v == {"torch.optim", ".backward("}
    assert not guards.anti_proxy_guard(str(tmp_path))["passed"]


def test_mfu_history_and_elastic_bar(tmp_path):
    h = str(tmp_path / "mfu_history.jsonl")
    for suite, v, ok in [("long-train", 37.0, True), ("long-train-smoke", 50.0, True), ("long-train", 38.4, True),
                         ("long-train", 45.0, False), ("long-train", 38.6, True), ("long-train", 38.5, None)]:
        mfu.record(h, suite, v, ok)
    s = mfu.qualifying(mfu.load(h))
    assert s == [37.0, 38.4, 38.6, 38.5]  # smoke runs and failed-loss runs never count
    assert mfu.evaluate(s, 38.0) == (True, "STRICT_PASS")
    assert mfu.evaluate(s, 40.0) == (True, "ELASTIC_PASS")          # plateau within 2 pp of the bar, spread <= 0.5
    assert mfu.evaluate(s[:2], 40.0) == (False, "IN_BAND_INSUFFICIENT_HISTORY")
    assert mfu.evaluate([36.0, 38.4, 39.9], 40.0) == (False, "IN_BAND_UNSTABLE")
    assert mfu.evaluate(s, 45.0) == (False, "BELOW_BAND") and mfu.evaluate([], 1.0) == (False, "NO_QUALIFYING_RUNS")


def _fake(lines, rc=0, sleep=0.0):
    body = "import sys,time\n" + "".join(f"print({ln!r})\n" for ln in lines) + f"time.sleep({sleep})\nsys.exit({rc})\n"
    return [sys.executable, "-c", body]


def _loss(step, v, tag="LOSS"):
    return f"[{tag}] step={step} global_loss={v:.9e} grad_norm=1.000000000e+00 time_s=0.1 mfu_e2e_standard=40.0"


def test_dispatcher_three_steps_cache_and_failure_classes(tmp_path):
    ref = [_loss(i, 5.0 - 0.01 * i) for i in range(1, 31)]
    reg = {"evals": {"lt": {"needs_ref": True, "verdict": "long_train", "gate_window": [1, 31], "loss_rel_threshold": 0.01,
                            "ref_cmd": _fake(ref), "ours_cmd": _fake([_loss(i, (5.0 - 0.01 * i) * 1.002) for i in range(1, 31)])},
                     "bad": {"needs_ref": True, "verdict": "long_train", "gate_window": [1, 31], "ref_cmd": _fake(ref),
                             "ours_cmd": _fake(["RuntimeError: CUDA out of memory"], rc=1)},
                     "slow": {"needs_ref": False, "verdict": "resume_startup", "timeout_s": 1, "ours_cmd": _fake([], sleep=30)}}}
    cache = str(tmp_path / "cache")
    r1 = dispatcher.run_suite(RS.make_run_request("lt"), reg, ROOT, str(tmp_path / "a"), cache)
    assert r1["status"] == "passed" and r1["details"]["ref_cache"] == "miss" and abs(r1["metrics"]["mean_rel_diff"] - 0.002) < 1e-6
    RS.validate_run_result(r1, "long_train")
    r2 = dispatcher.run_suite(RS.make_run_request("lt"), reg, ROOT, str(tmp_path / "b"), cache)
    assert r2["details"]["ref_cache"] == "hit" and os.path.isfile(tmp_path / "b" / "result.json")
    r3 = dispatcher.run_suite(RS.make_run_request("bad"), reg, ROOT, str(tmp_path / "c"), cache)
    assert r3["status"] == "failed" and r3["details"]["failure_class"] == "training_failure" and r3["details"]["side"] == "ours"
    r4 = dispatcher.run_suite(RS.make_run_request("slow", {"timeout_s": 1}), reg, ROOT, str(tmp_path / "d"), None)
    assert r4["status"] == "failed" and r4["details"]["failure_class"] == "timeout"
    assert dispatcher.run_suite(RS.make_run_request("nope"), reg, ROOT, str(tmp_path / "e"))["status"] == "failed"


def test_cli_runs_real_cpu_gates(tmp_path, capsys):
    rc = cli_main(["run", "resume-gate", "--artifacts", str(tmp_path)])
    out = capsys.readouterr().out
    res = RS.extract_result(out)
    assert rc == 0 and res["status"] == "passed" and res["metrics"]["max_abs_loss_diff"] == 0.0, res
    rc = cli_main(["run", "production-train", "--artifacts", str(tmp_path)])
    res = RS.extract_result(capsys.readouterr().out)
    assert rc == 0 and res["metrics"]["missing"] == [], res
    assert cli_main(["guard"]) == 0 and cli_main(["info"]) == 0


def test_launch_summary_groups_kernels_and_reports_delta(tmp_path):
    from forge_train_harness_b200.utils import launch_summary as LS
    csv_text = '''==PROF== Connected to process 1
"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"
"0","1","python","h","void fth::gemm_bf16_kernel<256, 4, 0, 0, 0>(CUtensorMap)","1","7","(192, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","ns","200,000"
"1","1","python","h","fth::rope_kernel(__nv_bfloat16 *, int)","1","7","(256, 1, 1)","(1184, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","us","28.5"
"2","1","python","h","void fth::gemm_bf16_kernel<256, 4, 0, 0, 0>(CUtensorMap)","1","7","(192, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","ns","100,000"
'''
    launches = LS.parse_launches(csv_text.splitlines(keepends=True))
    assert launches == [("void fth::gemm_bf16_kernel<256, 4, 0, 0, 0>", 200.0), ("fth::rope_kernel", 28.5),
                        ("void fth::gemm_bf16_kernel<256, 4, 0, 0, 0>", 100.0)]
    s = LS.summarise(launches)
    assert s["launches"] == 3 and abs(s["total_us"] - 328.5) < 1e-6
    assert s["kernels"][0]["kernel"].startswith("void fth::gemm") and s["kernels"][0]["launches"] == 2
    prev = {"total_us": 400.0, "kernels": [{"kernel": "fth::rope_kernel", "launches": 1, "us": 60.0, "share": 0.15},
                                          {"kernel": "fth::old_kernel", "launches": 1, "us": 340.0, "share": 0.85}]}
    d = LS.with_delta(s, prev)
    rope = [k for k in d["kernels"] if k["kernel"] == "fth::rope_kernel"][0]
    assert rope["delta_us"] == -31.5 and d["kernels"][0]["delta_us"] is None and d["gone"] == ["fth::old_kernel"]
    md = LS.to_markdown(d)
    assert "delta us" in md and "no longer launched" in md and "-31.5" in md
    p = tmp_path / "l.csv"
    p.write_text(csv_text)
    assert LS.main([str(p), "--json", str(tmp_path / "s.json"), "--md", str(tmp_path / "s.md")]) == 0
    assert (tmp_path / "s.json").exists() and (tmp_path / "s.md").read_text().startswith("3 launches")


def test_env_check_reports_pins_and_toolkit():
    from forge_train_harness_b200.harness import env_check
    rows = env_check.checks(nvcc_output="Cuda compilation tools, release 12.9, V12.9.86")
    names = {r[0]: r for r in rows}
    assert names["python"][1] and names["torch"][1] and names["cuda toolkit (nvcc, sm_100a)"][1]
    bad = {r[0]: r for r in env_check.checks(nvcc_output="Cuda compilation tools, release 11.8, V11.8.89")}
    assert not bad["cuda toolkit (nvcc, sm_100a)"][1]


def test_step_profile_summary_and_delta(tmp_path, monkeypatch):
    """One env var profiles one step of one rank; the summary has per-kernel totals, busy / idle time and a delta."""
    from forge_train_harness_b200.utils import step_profile as sp
    agg = {"gemm": {"launches": 2, "us": 30.0}, "norm": {"launches": 1, "us": 5.0}}
    cur = sp._finish(dict(agg), [(0.0, 10.0), (5.0, 25.0), (40.0, 45.0)])
    assert cur["busy_us"] == 30.0 and cur["span_us"] == 45.0 and cur["idle_us"] == 15.0 and cur["n_launches"] == 3
    prev = sp._finish({"gemm": {"launches": 2, "us": 40.0}, "old": {"launches": 1, "us": 1.0}}, [(0.0, 41.0)])
    md = sp.render_md(cur, prev)
    assert "| `gemm` | 2 | 30 |" in md and "-10 |" in md and "new |" in md and "no longer launched: `old`" in md
    # the hook in the training loop: CPU run, step 2 profiled (CPU activities only; the file is still written)
    import forge_train_harness_b200 as fth
    monkeypatch.setenv("FORGE_PROFILE_STEP", "2")
    monkeypatch.setenv("FORGE_PROFILE_DIR", str(tmp_path))
    cfg = fth.RunConfig(model=fth.preset("tiny"), optim=fth.OptimConfig(lr=1e-3, lr_schedule="constant"),
                        train=fth.TrainConfig(num_steps=2, micro_batch_size=1, grad_accum_steps=1, dtype="fp32", cuda_graph=False),
                        data=fth.DataConfig(prefetch_size=0)).replace(model={"seq_length": 32, "padded_vocab_size": 256})
    import io
    fth.run_training_loop(cfg, out=io.StringIO())
    assert (tmp_path / "step_2_rank0.json").exists() and (tmp_path / "step_2_rank0.md").exists()


def test_stage2_inventory_status_and_op_long(tmp_path, monkeypatch):
    """The per-op registry agrees with the op router; op-long swaps exactly one op and compares the loss window."""
    import copy
    from forge_train_harness_b200.harness import stage2
    inv = stage2.op_inventory()
    assert inv["passed"] and inv["ops_registered"] == inv["ops_total"], inv["problems"]
    reg = copy.deepcopy(stage2.load_registry())
    reg["ops"]["swiglu_fwd"]["env_var"] = "OP_SWIGLU"          # not what the router reads
    reg["ops"]["rope_fwd_"]["kernel"] = "forge_train_harness_b200/csrc/elementwise.cu::no_such_kernel"
    del reg["ops"]["sumsq"]
    bad = stage2.op_inventory(reg)
    assert not bad["passed"] and len(bad["problems"]) == 3
    monkeypatch.setattr(stage2, "_results_dir", lambda: str(tmp_path / "op_long"))
    st = stage2.op_status()
    assert st["counts"]["not_started"] == 0 and st["counts"]["unverified"] == 21 and st["passed"]   # every op has a hand-written version
    # op-long on CPU: the candidate's one swapped op resolves to the same PyTorch code, so the windows agree exactly
    r = stage2.op_long("swiglu_fwd", os.path.join(ROOT, "configs", "tiny_cpu_dp2.toml"), steps=6, window=(2, 7), version="baseline",
                       out_dir=str(tmp_path / "run"), extra_sets=["parallel.use_distributed_optimizer=false", "train.micro_batch_size=1",
                                                                   "train.global_batch_size=1"])
    assert r["passed"] and r["mean_rel_diff"] == 0.0, r
    st = stage2.op_status()
    assert st["ops"]["swiglu_fwd"]["state"] == "merged" and st["counts"]["merged"] == 1
    assert not stage2.op_long("swiglu_fwd", "x.toml", version="nope")["passed"]


def test_workspace_resources_sync_prefetch_retention(tmp_path):
    import numpy as np
    from forge_train_harness_b200.data.sources import write_megatron_binary
    from forge_train_harness_b200.harness import workspace as W
    # resources: the first source that verifies is linked; a digest mismatch fails instead of feeding other bytes
    tok = tmp_path / "src" / "tokenizer.model"
    tok.parent.mkdir()
    tok.write_bytes(b"tokenizer-bytes")
    man = tmp_path / "external_resources.toml"
    man.write_text(f'''[meta]\nversion = 1\n[[entry]]\nname = "tok"\nkind = "file"\nsha256 = "{W.sha256_file(str(tok))}"\n'''
                   f'''canonical_relpath = ".resources/tok/tokenizer.model"\nsources = ["hf://org/repo#tokenizer.model", "file://{tmp_path}/nope", "file://{tok}"]\n''')
    ws = tmp_path / "ws"
    rep = W.provision(str(ws), str(man))
    assert rep[0]["source"] == str(tok) and (ws / ".resources/tok/tokenizer.model").read_bytes() == b"tokenizer-bytes"
    assert W.assert_provisioned(str(ws), str(man)) == []
    tok.write_bytes(b"swapped")
    with pytest.raises(W.ResourceError, match="no source verifies"):
        W.provision(str(ws), str(man))
    # sync: ignored paths stay behind, vanished files are removed on the far side
    src = tmp_path / "tree"
    (src / "forge_train_harness_b200").mkdir(parents=True)
    (src / "forge_train_harness_b200" / "__init__.py").write_text("x = 1\n")
    (src / "scratch_out").mkdir()
    (src / "scratch_out" / "big.log").write_text("log")
    (src / ".syncignore").write_text("# stays behind\nscratch_out/\n")
    (src / "a.txt").write_text("a")
    dst = tmp_path / "remote"
    r1 = W.sync_push(str(dst), str(src))
    assert r1["passed"] and r1["copied"] == 3 and not (dst / "scratch_out").exists()
    (src / "a.txt").unlink()
    (dst / "forge_train_harness_b200" / "__pycache__").mkdir()
    r2 = W.sync_push(str(dst), str(src))
    assert r2["removed"] == 1 and not (dst / "a.txt").exists() and not (dst / "forge_train_harness_b200" / "__pycache__").exists()
    # prefetch: the corpus is staged next to the trainer and its index parses
    docs = [np.arange(100, dtype=np.int32) for _ in range(5)]
    write_megatron_binary(str(tmp_path / "corpus"), docs)
    pf = W.prefetch(str(tmp_path / "corpus"), str(tmp_path / "data"))
    assert pf["passed"] and pf["windows_of_17_tokens"] == 500 // 17
    assert not W.prefetch(str(tmp_path / "missing"), str(tmp_path / "data"))["passed"]
    # retention: all but the newest two run directories of a suite go
    runs = tmp_path / "runs"
    for i in range(4):
        d = runs / f"long-train-{i}"
        d.mkdir(parents=True)
        os.utime(d, (1000 + i, 1000 + i))
    (runs / "resume-gate-0").mkdir()
    assert W.prune_old_runs(str(runs), "long-train", 2) == ["long-train-0", "long-train-1"]
    assert sorted(os.listdir(runs)) == ["long-train-2", "long-train-3", "resume-gate-0"]
    probe = W.env_probe()
    assert probe["checks"]["package_is_this_tree"]["ok"] and probe["checks"]["subprocess_config_isomorphic"]["ok"]


def test_wsd_sft_suite_with_host_side_kills(tmp_path, capsys):
    """``harness run wsd-sft``: the three-phase run is SIGKILLed from outside once per phase and restarted; its banners and
    per-phase trajectories equal a clean run's, and the run directory retention keeps only the newest runs."""
    rc = cli_main(["run", "wsd-sft", "--artifacts", str(tmp_path / "runs")])
    res = RS.extract_result(capsys.readouterr().out)
    assert rc == 0 and res["status"] == "passed", res
    assert all(p["passed"] and p["complete"] and p["max_abs_loss_diff"] == 0.0 for p in res["metrics"]["phases"].values())
    log = open(os.path.join(res["details"]["run_dir"], "ours", "ours.log")).read()
    assert log.count("[PHASE]") >= 6          # three phases, re-announced after each of the three kills


def test_axis_directories_gate_sources_and_resolve_deploy():
    """Every gate source renders against every model x optim axis file; <runtime> sentinels are filled at freeze time."""
    axes = render.load_axes(os.path.join(ROOT, "configs", "axes"))
    assert {"minicpm4_0.5b", "minicpm4_8b", "tiny"} <= set(axes["model"]) and "pretrain_cosine" in axes["optim"]
    reg = render.load_toml(os.path.join(ROOT, "configs", "eval", "dense_training.toml"))
    gdir = os.path.join(ROOT, "configs", "eval", "gate_config")
    gates = sorted(f for f in os.listdir(gdir) if f.endswith(".toml"))
    assert len(gates) >= 7
    for g in gates:
        for mname, model in axes["model"].items():
            prods = render.render_gate(render.load_toml(os.path.join(gdir, g)), model, axes["optim"]["pretrain_cosine"], reg["env"])
            ours = prods["ours"]
            assert ours["cli"]["num_layers"] >= 1 and ours["env"]["NUM_PROCS"] == ours["cli"].get("world_size", 1), (g, mname)
            assert ours["cli"]["grad_accum_steps"] * ours["cli"]["micro_batch_size"] * ours["env"]["NUM_PROCS"] == ours["cli"]["global_batch_size"]
    dptp = render.render_gate(render.load_toml(os.path.join(gdir, "dptp.toml")), axes["model"]["minicpm4_8b"],
                              axes["optim"]["pretrain_cosine"], reg["env"])["ours"]
    assert dptp["cli"]["num_layers"] == 4 and dptp["cli"]["tensor_parallel_size"] == 2 and dptp["cli"]["lr_warmup_iters"] == 0
    prod = {"cli": dict(dptp["cli"], data_path=render.RUNTIME), "env": {"MASTER_PORT": render.RUNTIME}}
    frozen = render.resolve_deploy(prod, {"data_path": "/data/corpus", "MASTER_PORT": 29511})
    assert frozen["cli"]["data_path"] == "/data/corpus" and frozen["env"]["MASTER_PORT"] == 29511
    with pytest.raises(KeyError, match="no value was given"):
        render.resolve_deploy(prod, {"data_path": "/data/corpus"})
    with pytest.raises(KeyError, match="match no <runtime>"):
        render.resolve_deploy(prod, {"data_path": "x", "MASTER_PORT": 1, "typo": 2})


def test_stage2_fan_out_bounds_concurrency_and_skips_exhausted_ops(tmp_path, monkeypatch):
    """[automation].max_concurrent workers at a time; an op whose last max_op_long_failures op-long runs failed is skipped."""
    from forge_train_harness_b200.harness import stage2
    monkeypatch.setattr(stage2, "_results_dir", lambda: str(tmp_path / "op_long"))
    ops = sorted(stage2.load_registry()["ops"])[:5]
    for _ in range(3):
        stage2._record(ops[0], {"passed": False})
    stage2._record(ops[1], {"passed": False})
    stage2._record(ops[1], {"passed": True})        # a pass resets the count
    assert stage2.op_long_failures(ops[0]) == 3 and stage2.op_long_failures(ops[1]) == 0
    marks = tmp_path / "marks"
    marks.mkdir()
    worker = tmp_path / "w.py"
    worker.write_text("import os, sys, time\nd = sys.argv[2]\nopen(os.path.join(d, sys.argv[1] + '.start'), 'w').close()\n"
                      "time.sleep(0.4)\nn = len([f for f in os.listdir(d) if f.endswith('.start')]) - len([f for f in os.listdir(d) if f.endswith('.end')])\n"
                      "open(os.path.join(d, sys.argv[1] + '.end'), 'w').write(str(n))\nsys.exit(3 if sys.argv[1] == os.environ['FAIL_OP'] else 0)\n")
    monkeypatch.setenv("FAIL_OP", ops[2])
    res = stage2.fan_out([sys.executable, str(worker), "{op}", str(marks)], ops=ops, max_concurrent=2, max_failures=3,
                         log_dir=str(tmp_path / "logs"))
    assert res["ops"][ops[0]]["state"] == "exhausted" and not os.path.exists(marks / (ops[0] + ".start"))
    assert res["ops"][ops[2]] == {"state": "failed", "rc": 3, "failures": 0} and res["ops"][ops[1]]["state"] == "done"
    assert res["peak_running"] == 2 and not res["passed"]
    assert max(int(open(marks / f).read()) for f in os.listdir(marks) if f.endswith(".end")) <= 2   # never more than 2 alive
    with pytest.raises(KeyError):
        stage2.fan_out(["true"], ops=["no_such_op"])


def test_gate_runs_feed_the_mfu_history_of_their_loop(tmp_path, capsys):
    """A long-train result carries the window's mean MFU; the runner appends it to the loop's history (and says so loudly when
    there is no loop to record it for), and the elastic bar reads that history."""
    from forge_train_harness_b200.gates import verdicts as V
    from forge_train_harness_b200.utils import wire
    lines = "\n".join(wire.format_loss_line(s, 5.0 - 0.01 * s, 1.0, 0.5, 40.0 + 0.1 * s) for s in range(1, 11))
    recs = wire.parse_loss_lines(lines, strict=False)
    m = V.long_train(recs, recs, (3, 9), 0.01)
    assert m["passed"] and abs(m["avg_mfu_e2e_standard"] - 40.55) < 1e-6 and "mfu_target" not in m
    assert not V.long_train(recs, recs, (3, 9), 0.01, mfu_floor=45.0)["passed"]          # a floor gates, its absence does not
    res = RS.make_run_result("long-train", True, "ok", m, {})
    assert mfu.record_result(res, env={}) is None and "SKIPPED" in capsys.readouterr().err
    row = mfu.record_result(res, env={"FORGE_LOOP_DIR": str(tmp_path)})
    assert row["suite"] == "long-train" and row["loss_passed"] is True and abs(row["mfu_avg"] - 40.55) < 1e-6
    assert mfu.record_result(RS.make_run_result("resume-gate", True, "ok", {"passed": True}, {}), env={"FORGE_LOOP_DIR": str(tmp_path)}) is None
    hist = mfu.load(str(tmp_path / "mfu_history.jsonl"))
    assert len(hist) == 1 and mfu.evaluate(mfu.qualifying(hist), 40.0)[0]


def test_profile_snapshot_suite_runs_end_to_end_on_cpu(tmp_path):
    """The suite's plumbing (environment prefix, profile directory inside the run directory, verdict) with the tiny CPU model;
    on CPU the snapshot names no device kernel, which the registry entry has to allow explicitly."""
    reg = {"evals": {"profile-snapshot": {
        "needs_ref": False, "gpu_count": 0, "timeout_s": 300, "verdict": "profile", "require_kernels": False,
        "ours_cmd": ["env", "FORGE_PROFILE_STEP=2", "FORGE_PROFILE_RANK=0", "FORGE_PROFILE_DIR={run_dir}/ours/profile", "CUDA_VISIBLE_DEVICES=",
                     "{python}", "-m", "forge_train_harness_b200.train", "--config", "{repo}/configs/tiny_cpu_dp2.toml",
                     "--set", "train.num_steps=3", "--set", "parallel.use_distributed_optimizer=false"]}}}
    req = RS.make_run_request("profile-snapshot", {}, 0)
    art = tmp_path / req["run_id"]
    res = dispatcher.run_suite(req, reg, ROOT, str(art))
    assert res["status"] == "passed", res
    assert os.path.isfile(art / "ours" / "profile" / "step_2_rank0.json") and os.path.isfile(art / "ours" / "profile" / "step_2_rank0.md")
    assert res["metrics"]["n_kernels"] == 0 and res["metrics"]["snapshot"].endswith("step_2_rank0.json")
    reg["evals"]["profile-snapshot"]["require_kernels"] = True
    req2 = RS.make_run_request("profile-snapshot", {}, 0)
    res2 = dispatcher.run_suite(req2, reg, ROOT, str(tmp_path / req2["run_id"]))
    assert res2["status"] != "passed" and "no device kernel" in json.dumps(res2)


def test_loss_gate_verdict_needs_its_threshold(tmp_path):
    from forge_train_harness_b200.utils import wire
    run = tmp_path / "run"
    for side, bias in (("ref", 0.0), ("ours", 0.002)):
        (run / side).mkdir(parents=True)
        (run / side / f"{side}.log").write_text("\n".join(wire.format_loss_line(s, 5.0 - 0.01 * s + bias, 1.0, 0.5, 41.0) for s in range(1, 21)))
    gate = {"gate_window": [11, 21], "max_avg_relative_loss_diff": 0.01}
    ok, m = dispatcher._verdict("loss_gate", gate, str(run))
    assert ok and m["mean_rel_diff"] < 1e-3 and abs(m["avg_mfu_e2e_standard"] - 41.0) < 1e-9 and m["threshold"] == 0.01
    assert not dispatcher._verdict("loss_gate", dict(gate, max_avg_relative_loss_diff=1e-5), str(run))[0]
    with pytest.raises(KeyError, match="max_avg_relative_loss_diff"):
        dispatcher._verdict("loss_gate", {"gate_window": [11, 21]}, str(run))
