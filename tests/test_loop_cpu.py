"""Development loop: retry matrix, milestone parsing / advancing, review gating, timeouts, lease release, offline report
(reference contract: agent-loop.sh, tools/agent_loop_milestone.sh, tools/agent_loop_retry.sh, tools/loop_report.py)."""
import json
import os
import subprocess
import sys

import pytest

from forge_train_harness_b200.harness import lease, loop, mfu

ORDER = ["alignment", "bitwise-singlecard", "resume", "long-horizon", "production"]


def test_retry_matrix():
    for rc in (0, 130, 143, 137, 64, 78, 124):
        assert not loop.should_retry(rc)
    for rc in (1, 2, 75, 139, 255):
        assert loop.should_retry(rc)
    assert "SIGTERM" in loop.classify_failure(143)
    assert loop.classify_failure(9) == "rc=9; no diagnostic available"


def test_classify_failure_quotes_the_last_log_line(tmp_path):
    p = tmp_path / "w.log"
    p.write_text("a\nAI Model Not Found: model name is not valid\n\n")
    assert loop.classify_failure(1, str(p)) == "rc=1; last log line: AI Model Not Found: model name is not valid"


def test_declared_milestone_parsing_and_successor():
    bodies = ("fix\n\nMILESTONE_STATUS: alignment PASS\n\x00other\nMILESTONE_STATUS: resume PASS  \n"
              "MILESTONE_STATUS: nonsense PASS\n  MILESTONE_STATUS: production PASS\nMILESTONE_STATUS: long-horizon FAIL\n")
    assert loop.parse_declared_milestone(bodies, ORDER) == "resume"  # indented / unknown / non-PASS lines do not count
    assert loop.parse_declared_milestone("nothing here", ORDER) == ""
    assert loop.next_milestone_after("resume", "alignment", ORDER) == "long-horizon"
    assert loop.next_milestone_after("alignment", "resume", ORDER) == ""  # never moves backwards
    assert loop.next_milestone_after("production", "long-horizon", ORDER) == "production"  # capped at the last
    assert loop.next_milestone_after("production", "production", ORDER) == ""


def _workspace(tmp_path):
    ws = tmp_path / "ws"
    ws.mkdir()
    env = dict(os.environ, GIT_AUTHOR_NAME="t", GIT_AUTHOR_EMAIL="t@t", GIT_COMMITTER_NAME="t", GIT_COMMITTER_EMAIL="t@t")
    for cmd in (["git", "init", "-q"], ["git", "commit", "-q", "--allow-empty", "-m", "base"]):
        subprocess.run(cmd, cwd=ws, check=True, env=env)
    reg = tmp_path / "registry.toml"
    reg.write_text('[stage1]\nmilestone_order = ["alignment", "bitwise-singlecard", "long-horizon", "production"]\n'
                   '[evals.forward-align]\nmilestone = "alignment.forward"\ngpu_count = 0\ntimeout_s = 30\n'
                   '[evals.backward-align]\nmilestone = "alignment.backward"\ngpu_count = 0\ntimeout_s = 30\n'
                   '[evals.multistep]\nmilestone = "bitwise-singlecard"\ngpu_count = 0\ntimeout_s = 30\n')
    return ws, reg


WORKER = r'''
import os, subprocess, sys
rnd = int(os.environ["FORGE_ROUND"]); ms = os.environ["FORGE_MILESTONE"]
script = {script!r}
act = script.get(rnd, "noop")
if act.startswith("fail"):
    flag = os.path.join(os.environ["FORGE_LOOP_DIR"], "failed_once_%d" % rnd)
    if not os.path.exists(flag):
        open(flag, "w").close(); print("transient: rate limit"); sys.exit(int(act[4:] or 1))
    act = "declare"
if act == "hang":
    import time; time.sleep(60)
if act in ("declare", "declare_gated"):
    env = dict(os.environ, GIT_AUTHOR_NAME="t", GIT_AUTHOR_EMAIL="t@t", GIT_COMMITTER_NAME="t", GIT_COMMITTER_EMAIL="t@t")
    subprocess.run(["git", "commit", "-q", "--allow-empty", "-m", "round %d\n\nMILESTONE_STATUS: %s PASS" % (rnd, ms)], check=True, env=env)
'''


def _cfg(tmp_path, ws, reg, script, **kw):
    w = tmp_path / "worker.py"
    w.write_text(WORKER.format(script=script))
    base = dict(worker_cmd=[sys.executable, str(w)], registry=str(reg), workspace=str(ws), loops_dir=str(tmp_path / "loops"),
                retry_backoff_s=0.0, round_timeout_s=20.0, review_gated=["long-horizon"])
    base.update(kw)
    return loop.LoopConfig(**base)


def _events(lp):
    return [json.loads(x) for x in open(os.path.join(lp.dir, "events.jsonl"))]


def test_loop_advances_on_declarations_retries_and_withholds_gated(tmp_path):
    ws, reg = _workspace(tmp_path)
    # round 1 declares alignment; round 2 fails once (transient) then declares; round 3 declares the gated milestone
    cfg = _cfg(tmp_path, ws, reg, {1: "declare", 2: "fail1", 3: "declare_gated"})
    lp = loop.Loop(cfg, loop_id="L1")
    assert lp.run(max_rounds=3) == 0
    ev = _events(lp)
    adv = [(e["from"], e["to"]) for e in ev if e["subtype"] == "milestone_advanced"]
    assert adv == [("alignment", "bitwise-singlecard"), ("bitwise-singlecard", "long-horizon")]
    assert all(e.get("commit") for e in ev if e["subtype"] == "milestone_advanced")
    fails = [e for e in ev if e["subtype"] == "agent_failed"]
    assert len(fails) == 1 and fails[0]["round"] == 2 and "rate limit" in fails[0]["text"]
    assert [e["milestone"] for e in ev if e["subtype"] == "milestone_advance_withheld"] == ["long-horizon"]
    assert lp.milestone == "long-horizon"  # the declaration alone did not move a review-gated milestone
    assert ev[-1]["subtype"] == "loop_exit" and ev[-1]["cause"] == "round limit reached"
    # a restart resumes: same milestone, round counter continues
    lp2 = loop.Loop(cfg, loop_id="L1")
    assert lp2.milestone == "long-horizon" and lp2.run(max_rounds=1) == 0
    assert [e["round"] for e in _events(lp2) if e["subtype"] == "round_started"] == [1, 2, 3, 4]
    # prompts name the milestone and its suites
    txt = open(os.path.join(lp.dir, "round_001.prompt.md")).read()
    assert "active milestone: alignment" in txt and "forward-align" in txt and "backward-align" in txt


def test_review_override_advances_gated_milestone_and_finishes(tmp_path):
    ws, reg = _workspace(tmp_path)
    review = tmp_path / "review.py"
    review.write_text("import os,sys\nopen(sys.argv[1],'w').write('REVIEW_STATUS: PASS\\nMILESTONE_OVERRIDE: %s\\n' % os.environ['FORGE_MILESTONE'])\n")
    cfg = _cfg(tmp_path, ws, reg, {}, review_cmd=[sys.executable, str(review), "{review_file}"])
    lp = loop.Loop(cfg, loop_id="L2")
    lp._write("stage1.milestone", "long-horizon")
    assert lp.run(max_rounds=1) == 0
    assert lp.milestone == "production"
    assert [e["subtype"] for e in _events(lp) if e["subtype"].startswith("milestone")] == ["milestone_auto_advanced"]
    # a FAIL review never advances, whatever it writes
    review.write_text("import os,sys\nopen(sys.argv[1],'w').write('REVIEW_STATUS: FAIL\\nMILESTONE_OVERRIDE: long-horizon\\n')\n")
    lp3 = loop.Loop(cfg, loop_id="L3")
    lp3._write("stage1.milestone", "long-horizon")
    assert lp3.run(max_rounds=1) == 0 and lp3.milestone == "long-horizon"
    assert [e["verdict"] for e in _events(lp3) if e["subtype"] == "review_finished"] == ["FAIL"]


def test_no_retry_codes_stop_the_loop_and_timeouts_start_a_fresh_round(tmp_path):
    ws, reg = _workspace(tmp_path)
    cfg = _cfg(tmp_path, ws, reg, {1: "fail78"})
    w = tmp_path / "worker.py"
    w.write_text("import sys; sys.exit(78)\n")
    lp = loop.Loop(cfg, loop_id="L4")
    assert lp.run(max_rounds=5) == 78
    ev = _events(lp)
    assert len([e for e in ev if e["subtype"] == "agent_failed"]) == 1  # not retried
    assert "configuration error" in ev[-1]["cause"]
    # a round that overruns its cap is killed (its whole process group), reported as a timeout, and the loop moves on
    cfg2 = _cfg(tmp_path, ws, reg, {1: "hang", 2: "declare"}, round_timeout_s=0.5)
    lp2 = loop.Loop(cfg2, loop_id="L5")
    assert lp2.run(max_rounds=2) == 0
    st = [(e["round"], e["status"]) for e in _events(lp2) if e["subtype"] == "round_finished"]
    assert st == [(1, "timeout"), (2, "ok")] and lp2.milestone == "bitwise-singlecard"


class _Sched:
    def __init__(self, verdicts):
        self.verdicts, self.entries, self.n = verdicts, [], 0

    def submit(self, entry, *, gpus, nodes=1, env=None):
        self.entries.append(entry)
        self.n += 1
        return f"j{self.n}"

    def phase(self, job_id):
        suite = next(s for s in self.verdicts if f" {s} " in self.entries[int(job_id[1:]) - 1] + " ")
        return "succeeded" if self.verdicts[suite] else "failed"

    def stop(self, job_id, reason=""):
        pass

    def logs(self, job_id):
        return ""


def test_gates_mode_advances_only_when_every_suite_of_the_milestone_passes(tmp_path, monkeypatch):
    monkeypatch.setenv("FORGE_JOBS_DIR", str(tmp_path / "jobs"))
    ws, reg = _workspace(tmp_path)
    cfg = _cfg(tmp_path, ws, reg, {}, advance="gates", gate_poll_s=0.01)
    s = _Sched({"forward-align": True, "backward-align": False, "multistep": True})
    lp = loop.Loop(cfg, loop_id="L6", scheduler=s)
    assert lp.run(max_rounds=1) == 0 and lp.milestone == "alignment"  # half of the milestone failed
    s.verdicts["backward-align"] = True
    subprocess.run(["git", "commit", "-q", "--allow-empty", "-m", "fix"], cwd=ws, check=True,
                   env=dict(os.environ, GIT_AUTHOR_NAME="t", GIT_AUTHOR_EMAIL="t@t", GIT_COMMITTER_NAME="t", GIT_COMMITTER_EMAIL="t@t"))
    assert lp.run(max_rounds=1) == 0 and lp.milestone == "bitwise-singlecard"
    runs = [(e["suite"], e["rc"]) for e in _events(lp) if e["subtype"] == "gate_run"]
    assert runs == [("forward-align", 0), ("backward-align", 1), ("forward-align", 0), ("backward-align", 0)]


def test_lease_is_released_on_every_exit_path_and_report_reads_files_only(tmp_path, monkeypatch):
    monkeypatch.setenv("FORGE_LEASE_DIR", str(tmp_path / "lease"))
    ws, reg = _workspace(tmp_path)
    w = tmp_path / "worker.py"
    cfg = _cfg(tmp_path, ws, reg, {1: "declare"}, gpus=2, remote={"kind": "local", "total_gpus": 4})
    w.write_text("import os,sys\nprint(os.environ['CUDA_VISIBLE_DEVICES']); sys.exit(64)\n")
    lp = loop.Loop(cfg, loop_id="L7")
    assert lp.run(max_rounds=2) == 64
    assert lease.holders("gpu") == {}
    assert open(os.path.join(lp.dir, "round_001.worker.log")).read().strip() == "0,1"
    sub = [e["subtype"] for e in _events(lp)]
    assert sub.index("lease_claimed") < sub.index("round_started") < sub.index("lease_released") < sub.index("loop_exit")
    mfu.record(os.path.join(lp.dir, "mfu_history.jsonl"), "long-train", 41.0, True)
    mfu.record(os.path.join(lp.dir, "mfu_history.jsonl"), "long-train", 43.5, True)
    rep = loop.report(lp.dir)
    assert not rep["live"] and rep["exit"]["rc"] == 64 and rep["rounds"][0]["status"] == "failed"
    assert [round(t["delta"], 2) if t["delta"] is not None else None for t in rep["mfu"]] == [None, 2.5]
    md = loop.report_markdown(rep)
    assert "| alignment | - |" in md and "usage error" in md and "+2.50" in md


def test_loop_config_file_and_cli(tmp_path):
    ws, reg = _workspace(tmp_path)
    cfgp = tmp_path / "loop.toml"
    cfgp.write_text(f'[loop]\nworker_cmd = ["true"]\nregistry = "{reg}"\nworkspace = "{ws}"\nloops_dir = "{tmp_path}/loops"\nmax_rounds = 1\n')
    r = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.harness.loop", "run", "--config", str(cfgp), "--loop-id", "cli"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.harness.loop", "report", str(tmp_path / "loops" / "cli")],
                       capture_output=True, text=True)
    assert r.returncode == 0 and "## rounds" in r.stdout and "round limit reached" in r.stdout
    cfgp.write_text('[loop]\nworker_cmd = ["true"]\nbogus = 1\n')
    with pytest.raises(ValueError, match="bogus"):
        loop.LoopConfig.load(str(cfgp))
    # the shipped loop config parses, and the shipped registry has a milestone order whose every suite maps into it
    shipped = loop.LoopConfig.load(os.path.join(loop.ROOT, "configs", "loop.toml"))
    order = loop.milestone_order(shipped.registry)
    assert order[0] == "alignment" and order[-1] == "production"
    for m in order:
        assert loop.suites_of_milestone(shipped.registry, m), m


def test_every_eval_family_registry_is_routable():
    """Four families (0.5B, 1B, 8B, Qwen3), each with a milestone order that its suites cover and verdict kinds the dispatcher knows."""
    import inspect
    import tomllib

    from forge_train_harness_b200.harness import dispatcher
    kinds = set(__import__("re").findall(r'kind == "([a-z_]+)"', inspect.getsource(dispatcher._verdict)))
    for fam in ("dense_training", "dense_training_1b", "dense_training_8b", "dense_training_qwen3"):
        path = os.path.join(loop.ROOT, "configs", "eval", fam + ".toml")
        doc = tomllib.load(open(path, "rb"))
        assert doc["family"]["name"] == fam
        order = loop.milestone_order(path)
        for m in order:
            assert loop.suites_of_milestone(path, m), (fam, m)
        for name, gate in doc["evals"].items():
            assert gate["verdict"] in kinds, (fam, name, gate["verdict"])
            assert gate.get("stage") in ("stage1", "stage2", "aux"), (fam, name)     # aux: not part of any milestone (profile snapshot)
            ms = gate.get("milestone", "")
            assert gate["stage"] != "stage1" or ms.split(".")[0] in order, (fam, name, ms)
    d8 = tomllib.load(open(os.path.join(loop.ROOT, "configs", "eval", "dense_training_8b.toml"), "rb"))
    assert "hf-oracle" in d8["evals"] and "dptp" in d8["evals"] and "--model" in d8["evals"]["long-train"]["ours_cmd"]
    dq = tomllib.load(open(os.path.join(loop.ROOT, "configs", "eval", "dense_training_qwen3.toml"), "rb"))
    assert "qwen3_0.6b" in dq["evals"]["long-train"]["ours_cmd"] and "dptp" not in dq["evals"]


def test_fork_continues_from_the_milestone_after_the_anchor(tmp_path):
    ws, reg = _workspace(tmp_path)
    cfg = _cfg(tmp_path, ws, reg, {1: "declare", 2: "declare"})
    lp = loop.Loop(cfg, loop_id="src")
    assert lp.run(max_rounds=2) == 0 and lp.milestone == "long-horizon"
    mfu.record(os.path.join(lp.dir, "mfu_history.jsonl"), "long-train", 40.0, True)
    assert lp.backfill_mfu_events() == 1 and lp.backfill_mfu_events() == 0  # cursor: each row becomes one event, once
    assert [e["mfu_avg"] for e in _events(lp) if e["subtype"] == "mfu_record"] == [40.0]
    # fork at the first milestone: anchor = the commit that declared it (from the event), state = the milestone after it
    info = loop.fork(cfg, "src", "alignment", new_loop_id="forked", workspace_dst=str(tmp_path / "ws2"))
    assert info["anchor_source"] == "event" and info["next_milestone"] == "bitwise-singlecard" and info["round"] == 1
    head2 = subprocess.run(["git", "-C", str(tmp_path / "ws2"), "rev-parse", "HEAD"], capture_output=True, text=True).stdout.strip()
    assert head2 == info["anchor"] and head2 != lp.head()  # history cut at the anchor; the source keeps its later commits
    import dataclasses
    lp2 = loop.Loop(dataclasses.replace(cfg, workspace=str(tmp_path / "ws2")), loop_id="forked")
    assert lp2.milestone == "bitwise-singlecard" and os.path.isfile(os.path.join(lp2.dir, "mfu_history.jsonl"))
    assert lp2.run(max_rounds=1) == 0  # round counter continues: this is round 2, whose script entry declares
    assert [e["round"] for e in _events(lp2) if e["subtype"] == "round_started"] == [2] and lp2.milestone == "long-horizon"
    with pytest.raises(ValueError, match="already exists"):
        loop.fork(cfg, "src", "alignment", new_loop_id="forked")
    with pytest.raises(ValueError, match="not in the milestone order"):
        loop.fork(cfg, "src", "nonsense")
    # without events the one declaring commit is found in the history; an undeclared sha is refused
    os.unlink(os.path.join(lp.dir, "events.jsonl"))
    assert loop.fork(cfg, "src", "bitwise-singlecard", new_loop_id="f3")["anchor_source"] == "git-fallback"
    with pytest.raises(ValueError, match="does not"):
        loop.fork(cfg, "src", "alignment", new_loop_id="f4", at_sha=lp.head())


def test_builtin_review_applies_the_elastic_mfu_bar_to_the_gated_milestone(tmp_path):
    ws, reg = _workspace(tmp_path)
    cfg = _cfg(tmp_path, ws, reg, {}, review_mfu_target=40.0)
    lp = loop.Loop(cfg, loop_id="R1")
    lp._write("stage1.milestone", "long-horizon")
    hist = os.path.join(lp.dir, "mfu_history.jsonl")
    mfu.record(hist, "long-train", 36.0, True)                     # below the band
    assert lp.run(max_rounds=1) == 0 and lp.milestone == "long-horizon"
    mfu.record(hist, "long-train", 38.6, True)                     # in the band, too little history
    assert lp.run(max_rounds=1) == 0 and lp.milestone == "long-horizon"
    mfu.record(hist, "long-train", 38.9, True)
    mfu.record(hist, "long-train", 38.7, True)                     # three in-band samples within 0.5: a plateau
    assert lp.run(max_rounds=1) == 0 and lp.milestone == "production"
    ev = _events(lp)
    codes = [e["contract"]["code"] for e in ev if e["subtype"] == "review_finished"]
    assert codes == ["BELOW_BAND", "IN_BAND_INSUFFICIENT_HISTORY", "ELASTIC_PASS"]
    assert [e["text"] for e in ev if e["subtype"] == "milestone_auto_advanced"] == ["ELASTIC_PASS"]
    assert [e["mfu_avg"] for e in ev if e["subtype"] == "mfu_record"] == [36.0, 38.6, 38.9, 38.7]
    # a failed loss verdict disqualifies a sample; milestones that are not review-gated are never touched by the bar
    lp2 = loop.Loop(_cfg(tmp_path, ws, reg, {}, review_mfu_target=40.0), loop_id="R2")
    mfu.record(os.path.join(lp2.dir, "mfu_history.jsonl"), "long-train", 55.0, False)
    lp2._write("stage1.milestone", "long-horizon")
    assert lp2.run(max_rounds=1) == 0 and lp2.milestone == "long-horizon"
    lp3 = loop.Loop(_cfg(tmp_path, ws, reg, {}, review_mfu_target=40.0), loop_id="R3")
    mfu.record(os.path.join(lp3.dir, "mfu_history.jsonl"), "long-train", 55.0, True)
    assert lp3.run(max_rounds=1) == 0 and lp3.milestone == "alignment"


def test_stage2_fans_workers_out_per_operator_until_every_op_is_merged(tmp_path, monkeypatch):
    """After stage 1 the loop re-fans one worker per not-yet-merged operator each round; a worker 'merges' its op here by
    recording a passing op-long for it, the way the real gate does."""
    from forge_train_harness_b200.harness import stage2
    res_dir = tmp_path / "op_long"
    monkeypatch.setattr(stage2, "_results_dir", lambda: str(res_dir))
    ws, reg = _workspace(tmp_path)
    worker = tmp_path / "s2.py"
    worker.write_text("import json, os, sys\nop, d, rnd = sys.argv[1], sys.argv[2], int(os.environ['FORGE_ROUND'])\nos.makedirs(d, exist_ok=True)\n"
                      "ok = not (op == os.environ.get('SLOW_OP') and rnd == 1)\n"
                      "json.dump({'passed': ok, 'mean_rel_diff': 1e-4, 'steps': 200, 'consecutive_failures': 0 if ok else 1}, open(os.path.join(d, op + '.json'), 'w'))\n"
                      "sys.exit(0 if ok else 1)\n")
    ops = sorted(stage2.load_registry()["ops"])
    monkeypatch.setenv("SLOW_OP", ops[3])
    cfg = _cfg(tmp_path, ws, reg, {}, stage2_worker_cmd=[sys.executable, str(worker), "{op}", str(res_dir)])
    lp = loop.Loop(cfg, loop_id="S2")
    lp._write("stage1.status", "finished")
    assert lp.run() == 0
    ev = [e for e in _events(lp) if e["subtype"].startswith("stage2") or e["subtype"] == "stage_finished"]
    assert [e["subtype"] for e in ev] == ["stage2_round_started", "stage2_round_finished", "stage2_round_started", "stage2_round_finished",
                                          "stage2_round_started", "stage_finished"]
    assert len(ev[0]["pending"]) == len(ops) and ev[2]["pending"] == [ops[3]] and ev[4]["pending"] == []   # only the failed op is re-run
    assert ev[1]["ops"][ops[3]] == "failed" and ev[3]["ops"] == {ops[3]: "done"} and ev[1]["peak_running"] <= 6
    assert lp._read("stage2.status") == "finished" and lp.run() == 0                                        # and it stays finished
