"""Capture layer, verdicts, wire format, config schema, schedules, data sources (CPU)."""
import dataclasses
import math
import os

import numpy as np
import pytest
import torch

import forge_train_harness_b200 as fth
from forge_train_harness_b200.config import schema
from forge_train_harness_b200.data import sources
from forge_train_harness_b200.gates import capture as cap
from forge_train_harness_b200.gates import verdicts as V
from forge_train_harness_b200.optim.schedule import compute_lr, wsd_lr
from forge_train_harness_b200.parallel.pipeline import build_schedule
from forge_train_harness_b200.utils import wire
from tests.test_parallel_cpu import base_cfg


# ---- wire ---------------------------------------------------------------------------------------------
def test_wire_roundtrip_and_trailing_fields():
    line = wire.format_loss_line(7, 3.14159265, 0.5, 1.25, 42.0, tokens_per_sec_per_gpu=1234.5)
    r = wire.parse_loss_line(line)
    assert (r.step, r.tag) == (7, "LOSS") and abs(r.loss - 3.14159265) < 1e-9 and r.mfu == 42.0
    assert r.extra["tokens_per_sec_per_gpu"].startswith("1234.5")
    assert wire.parse_loss_line("[LOSS_RES] step=3 global_loss=1.0e+00 grad_norm=2.0e+00").tag == "LOSS_RES"
    with pytest.raises(ValueError):
        wire.parse_loss_line("[LOSS] step=1 global_loss=nan grad_norm=1.0")
    assert wire.parse_loss_line("[LOSS] step=1 global_loss=nan grad_norm=1.0", strict=False) is not None
    ph = wire.parse_phase_line(wire.format_phase_line("decay", 20, 1e-3, 0.0, 0, 40, 20, False, "synthetic"))
    assert ph["name"] == "decay" and ph["start_step"] == "20" and ph["init_weights_only"] == "0"
    recs = wire.parse_loss_lines(" iteration 5/ 10 | lm loss: 2.5E+00 | grad norm: 1.5 |", megatron_fallback=True)
    assert recs[0].step == 5 and recs[0].loss == 2.5


# ---- config --------------------------------------------------------------------------------------------
def test_schema_aliases_products_and_rejection(tmp_path):
    doc = {"model": {"scale_emb": 10, "dim_model_base": 128, "scale_depth": 2.0, "hidden_size": 256},
           "cli": {"num_steps": 5, "micro_batch_size": 3, "lr": 0.5, "tensor_parallel_size": 1, "world_size": 2, "gate_window": [1, 2]},
           "env": {"NCCL_ALGO": "Tree"}}
    c = schema.from_dict(doc)
    assert c.model.mup_emb_scale == 10 and c.model.mup_base_hidden_size == 128 and c.model.width_mult == 2.0
    assert c.train.num_steps == 5 and c.train.micro_batch_size == 3 and c.optim.lr == 0.5
    with pytest.raises(KeyError):
        schema.from_dict({"model": {"no_such_key": 1}})
    with pytest.raises(KeyError):
        schema.from_dict({"nonsense": {}})
    for name in ("tiny", "minicpm4_0.5b", "minicpm4_8b", "minicpm5_1b", "qwen3_0.6b"):
        assert schema.preset(name).qkv_dim > 0
    # FLOPs per token of the two benchmark shapes (training, x3)
    assert abs(schema.preset("minicpm4_0.5b").flops_per_token(False) / 3.207e9 - 1) < 1e-3
    assert abs(schema.preset("minicpm4_8b").flops_per_token(False) / 50.53e9 - 1) < 1e-3


def test_lr_schedules():
    assert wsd_lr(5, 1.0, 0.1, 10, 100, 20) == 0.5
    assert wsd_lr(50, 1.0, 0.1, 10, 100, 20) == 1.0
    assert abs(wsd_lr(90, 1.0, 0.1, 10, 100, 20) - (0.1 + (2 * 0.5 ** 0.5 - 1) * 0.9)) < 1e-12
    assert wsd_lr(100, 1.0, 0.1, 10, 100, 20) == pytest.approx(0.1)
    assert wsd_lr(101, 1.0, 0.1, 10, 100, 20) == 0.1
    oc = fth.OptimConfig(lr=1.0, min_lr=0.0, lr_warmup_iters=10, lr_decay_iters=110, lr_schedule="cosine")
    assert compute_lr(5, oc) == 0.5 and abs(compute_lr(60, oc) - 0.5) < 1e-12 and compute_lr(200, oc) == 0.0


# ---- data ----------------------------------------------------------------------------------------------
def test_megatron_binary_roundtrip_and_cursor(tmp_path):
    rng = np.random.RandomState(0)
    docs = [rng.randint(0, 1000, size=n).astype(np.int32) for n in (50, 200, 333, 17)]
    prefix = str(tmp_path / "corpus")
    sources.write_megatron_binary(prefix, docs)
    a = sources.MegatronBinary(prefix, seq_len=16, micro_batch=2, dp_rank=0, dp_size=2, seed=3)
    b = sources.MegatronBinary(prefix, seq_len=16, micro_batch=2, dp_rank=1, dp_size=2, seed=3)
    flat = np.concatenate(docs)
    x = next(a)
    assert x["tokens"].shape == (2, 16) and torch.equal(x["tokens"][:, 1:], x["labels"][:, :-1])
    win = flat[: len(flat) // 17 * 17].reshape(-1, 17)
    assert any((win[:, :-1] == x["tokens"][0].numpy()).all(1))
    assert not torch.equal(x["tokens"], next(b)["tokens"])
    seq = [next(a)["tokens"].clone() for _ in range(30)]  # crosses epochs
    st = a.state_dict()
    nxt = next(a)["tokens"]
    c = sources.MegatronBinary(prefix, 16, 2, 0, 2, 3)
    c.load_state_dict(st)
    assert torch.equal(next(c)["tokens"], nxt)  # O(1) restore, no replay
    d = sources.MegatronBinary(prefix, 16, 2, 0, 2, 3)
    d.seek_microbatches(31)
    assert torch.equal(next(d)["tokens"], nxt)


def test_prefetcher_skips_all_masked_batches_and_tracks_consumer_state():
    class Src:
        def __init__(self):
            self.i = 0

        def state_dict(self):
            return {"i": self.i}

        def __next__(self):
            self.i += 1
            m = torch.zeros(1, 4) if self.i % 2 else torch.ones(1, 4)
            return {"tokens": torch.full((1, 4), self.i), "labels": torch.zeros(1, 4, dtype=torch.long), "loss_mask": m}
    pf = sources.Prefetcher(Src(), depth=4)
    got = [int(pf.get()["tokens"][0, 0]) for _ in range(3)]
    assert got == [2, 4, 6] and pf.state_dict() == {"i": 6}
    pf.stop()
    ids, lab, mk = torch.arange(8).view(1, 8), torch.arange(1, 9).view(1, 8), torch.ones(1, 8)
    mi, ml, mm = sources.build_mtp_tensors(ids, lab, mk)
    assert torch.equal(mi, lab) and ml[0, -1] == 0 and mm[0, -1] == 0 and torch.equal(ml[0, :-1], lab[0, 1:])


# ---- pipeline schedule -----------------------------------------------------------------------------------
@pytest.mark.parametrize("pp,vpp,n_mb", [(2, 1, 4), (4, 1, 8), (2, 2, 4), (4, 2, 8), (2, 2, 2)])
def test_schedule_is_complete_and_causal(pp, vpp, n_mb):
    for p in range(pp):
        acts = build_schedule(pp, p, vpp, n_mb)
        f = [(v, i) for k, v, i in acts if k == "F"]
        b = [(v, i) for k, v, i in acts if k == "B"]
        assert sorted(f) == sorted(b) == sorted((v, i) for v in range(vpp) for i in range(n_mb))
        seen = set()
        for k, v, i in acts:
            if k == "F":
                seen.add((v, i))
            else:
                assert (v, i) in seen  # a backward never precedes its forward
        inflight = peak = 0
        for k, _, _ in acts:
            inflight += 1 if k == "F" else -1
            peak = max(peak, inflight)
        assert peak <= (pp - p - 1) * (2 if vpp > 1 else 1) + (vpp - 1) * pp + 1 or n_mb == pp


# ---- capture + verdicts --------------------------------------------------------------------------------------
def _run_with_capture(tmp_path, tag, level, perturb=False):
    cfg = base_cfg(steps=2)
    out = str(tmp_path / f"{tag}.json")
    sess = cap.CaptureSession(out, level=level, rank=0)
    tr = fth.Trainer(cfg, device="cpu", quiet=True, capture=sess)
    if perturb:
        tr.store.p("layers.1.wo.weight").mul_(1.0001)
        tr.opt.sync_master_from_params()
    for _ in range(2):
        tr.train_step()
    sess.dump()
    tr.close()
    return out


def test_capture_key_families_and_alignment_verdict(tmp_path):
    a = _run_with_capture(tmp_path, "ref", 2)
    b = _run_with_capture(tmp_path, "ours", 2)
    c = _run_with_capture(tmp_path, "bad", 2, perturb=True)
    recs = cap.load_merged(a)
    keys = set(recs)
    assert "step_0.rank0.mb0.fwd.layers.0.wqkv#0" in keys and "step_1.rank0.mb1.bwd.layers.3.w2#0" in keys
    assert "step_0.rank0.mb0.loss.per_token.preallreduce" in keys and "step_0.rank0.loss.scalar.postallreduce" in keys
    assert "step_1.rank0.grad.tok_embeddings.weight.preallreduce" in keys
    assert recs["step_0.rank0.mb0.loss.per_token.preallreduce"]["shape"] == [2, 32]
    assert len(recs["step_0.rank0.grad.norm.weight.postallreduce"]["hash"]) == 32
    assert V.align(a, b, ".fwd.")["passed"] and V.align(a, b, ".grad.", backward=True)["passed"]
    bad = V.align(a, c, ".fwd.")
    assert not bad["passed"] and any("layers.1.wo" in k for k in bad["mismatched"])
    assert not cap.diff_captures({"x": {"hash": "1"}}, {"y": {"hash": "1"}})["passed"]  # zero overlap fails
    lvl1 = cap.load_merged(_run_with_capture(tmp_path, "l1", 1))
    assert not any(".fwd." in k for k in lvl1) and any(".grad." in k for k in lvl1)
    assert cap.load_merged(_run_with_capture(tmp_path, "l0", 0)) == {}
    t = torch.arange(10, dtype=torch.float32)
    flipped = t.clone()
    flipped.view(torch.int32)[3] ^= 1  # one mantissa bit
    assert cap.hash_tensor(t)["hash"] != cap.hash_tensor(flipped)["hash"]


def _recs(losses, tag="LOSS"):
    return [wire.LossRecord(tag, i + 1, l, 1.0, 0.1, 40.0) for i, l in enumerate(losses)]


def test_long_train_and_trajectory_verdicts():
    ref = [5.0 - 0.01 * i for i in range(40)]
    ok = V.long_train(_recs(ref), _recs([x * 1.004 for x in ref]), (1, 41), 0.01, mfu_floor=30.0)
    assert ok["passed"] and ok["mean_rel_diff"] == pytest.approx(0.004) and ok["drift_warning"] is None
    bad = V.long_train(_recs(ref), _recs([x * 1.03 for x in ref]), (1, 41), 0.01)
    assert not bad["passed"] and "systematic bias" in bad["drift_warning"]
    grow = V.window_loss_diff_metrics({i: 5.0 for i in range(40)}, {i: 5.0 + 0.0005 * (i + 1) for i in range(40)}, range(40))
    assert "monotonically positive" in grow["drift_warning"]
    assert not V.long_train(_recs(ref[:10]), _recs(ref), (1, 41))["passed"]  # missing window steps
    assert V.trajectory(_recs(ref), _recs(ref))["passed"]
    assert not V.trajectory(_recs(ref), _recs([ref[0] + 1e-9] + ref[1:]))["passed"]  # bitwise rule
    assert V.trajectory(_recs(ref), _recs([ref[0] + 1e-9] + ref[1:]), rtol=1e-6)["passed"]  # tolerance rule
    text = "\n".join(wire.format_loss_line(r.step, r.loss, 1.0, 0.1, 1.0, "LOSS_REF") for r in _recs(ref)) + "\n" + \
           "\n".join(wire.format_loss_line(r.step, r.loss, 1.0, 0.1, 1.0, "LOSS_RES") for r in _recs(ref)[10:])
    assert V.resume(text, (11, 41))["passed"]
    # a resumed run that printed one step of the window and died must not pass, nor a run that exited non-zero
    cut = "\n".join(wire.format_loss_line(r.step, r.loss, 1.0, 0.1, 1.0, "LOSS_REF") for r in _recs(ref)) + "\n" + \
          wire.format_loss_line(11, _recs(ref)[10].loss, 1.0, 0.1, 1.0, "LOSS_RES")
    trunc = V.resume(cut, (11, 41))
    assert not trunc["passed"] and "candidate lacks 29" in trunc["reason"]
    died = V.resume(text, (11, 41), returncode=1)
    assert not died["passed"] and died["script_succeeded"] is False
    assert V.resume(text, (11, 41), returncode=0)["passed"]
    assert not V.trajectory(_recs(ref), _recs(ref[:5]), window=(1, 41))["passed"]
    assert V.resume_startup("[RESUME_STARTUP] seconds=7.16", 18)["passed"] and not V.resume_startup("x", 18)["passed"]
    assert V.classify_failure("", timed_out=True) == "timeout" and V.classify_failure("NCCL error: unhandled") == "network"
    assert V.classify_failure("CUDA out of memory") == "training_failure"


def test_hf_stream_packer_is_deterministic_sharded_and_resumable(tmp_path, monkeypatch, capsys):
    import json
    import torch
    """Local parquet + JSON-lines sources, weighted mix, shuffle buffer, DP split, packing, [DATAHASH] lines, resume."""
    import pyarrow as pa
    import pyarrow.parquet as pq
    from forge_train_harness_b200.data.hf_stream import HFStream, build_modelbest, parse_data_path
    a, b = tmp_path / "a", tmp_path / "b"
    a.mkdir()
    b.mkdir()
    for i in range(2):
        pq.write_table(pa.table({"content": [f"doc a{i}-{j} " + "x" * (j % 7) for j in range(40)] + [""]}), a / f"part{i}.parquet")
    with open(b / "qa.jsonl", "w") as f:
        for j in range(30):
            f.write(json.dumps({"question": f"what is {j}+{j}?", "answer": str(2 * j)}) + "\n")
    monkeypatch.setenv("CORPUS_A", str(a))
    monkeypatch.setenv("CORPUS_B", str(b))
    path = f"2.0 hf://org/a?split=train&text=content&local_env=CORPUS_A&tokenizer=bytes 1.0 hf://org/b?split=train&template=gsm8k_qa&local_env=CORPUS_B&glob=*.jsonl"
    specs = parse_data_path(path)
    assert [s.repo for s in specs] == ["org/a", "org/b"] and specs[1].template == "gsm8k_qa"

    def take(rank, dp, n, state=None):
        s = HFStream(parse_data_path(path), 32, 2, rank, dp, seed=5, buffer_size=16)
        if state is not None:
            s.load_state_dict(state)
        out = [next(s) for _ in range(n)]
        return out, s.state_dict()
    x, st = take(0, 1, 6)
    y, _ = take(0, 1, 6)
    assert all(torch.equal(p["tokens"], q["tokens"]) and torch.equal(p["labels"], q["labels"]) for p, q in zip(x, y))
    assert x[0]["tokens"].shape == (2, 32) and torch.equal(x[0]["tokens"][:, 1:], x[0]["labels"][:, :-1])
    assert int(torch.cat([p["tokens"].reshape(-1) for p in x]).eq(256).sum()) > 0          # EOS between documents
    first3, st3 = take(0, 1, 3)
    rest, _ = take(0, 1, 3, st3)
    assert all(torch.equal(p["tokens"], q["tokens"]) for p, q in zip(first3 + rest, x))      # resume = uninterrupted
    r0, _ = take(0, 2, 3)
    r1, _ = take(1, 2, 3)
    assert not torch.equal(r0[0]["tokens"], r1[0]["tokens"])                                  # ranks read different documents
    monkeypatch.setenv("FORGE_HF_DATA_DUMP", "1")
    take(0, 1, 2)
    assert capsys.readouterr().out.count("[DATAHASH] rank=0 batch=") == 2
    monkeypatch.delenv("CORPUS_A")
    with pytest.raises(FileNotFoundError, match="no network access"):
        take(0, 1, 1)
    with pytest.raises(RuntimeError, match="modelbest_sdk"):
        build_modelbest("x")


def test_tolerance_alignment_of_tensor_captures(tmp_path):
    """forward-/backward-align in tolerance mode: relative L2 per key, known scales, fitted scales, missing overlap."""
    import torch
    from forge_train_harness_b200.gates.capture import CaptureSession, diff_tensors, family_key
    assert family_key("step_3.rank0.mb1.fwd.layers.0.wqkv#0") == "fwd.layers.0.wqkv"
    assert family_key("step_0.rank0.grad.layers.1.w2.weight.preallreduce") == "grad.layers.1.w2.weight"
    assert family_key("step_0.rank0.grad.x.weight.postallreduce") == "grad.x.weight.postallreduce"
    g = torch.Generator().manual_seed(0)
    ref = {"fwd.a": torch.randn(64, 32, generator=g), "fwd.emb": torch.randn(16, 8, generator=g), "bwd.a": torch.randn(64, 32, generator=g)}
    sess = CaptureSession(str(tmp_path / "ours.pt"), level=2, rank=0, mode="tensor")
    sess.begin_step(0)
    sess.module_hook("fwd", "a", (ref["fwd.a"] * (1 + 2e-3 * torch.randn(64, 32, generator=g))).to(torch.bfloat16))
    sess.module_hook("fwd", "emb", ref["fwd.emb"] * 12.0)
    sess.module_hook("bwd", "a", ref["bwd.a"] * 0.37)
    sess.dump()
    torch.save(ref, tmp_path / "ref.pt")
    ok = V.align_tolerance(str(tmp_path / "ref.pt"), str(tmp_path / "ours.pt"), "fwd", 1e-2, scales={"fwd.emb": 1 / 12.0})
    assert ok["passed"] and ok["checks_total"] == 2 and ok["worst_rel_err"] < 6e-3
    assert not V.align_tolerance(str(tmp_path / "ref.pt"), str(tmp_path / "ours.pt"), "fwd", 1e-2)["passed"]   # the x12 shows
    assert not V.align_tolerance(str(tmp_path / "ref.pt"), str(tmp_path / "ours.pt"), "bwd", 1e-2)["passed"]
    fit = V.align_tolerance(str(tmp_path / "ref.pt"), str(tmp_path / "ours.pt"), "bwd", 1e-2, fit_scale=True)
    assert fit["passed"] and fit["worst_rel_err"] < 1e-6
    assert not diff_tensors(ref, {}, family="fwd", rel_tol=1.0)["passed"]                                        # no overlap


def test_prepare_corpus_matches_the_streaming_encode_contract(tmp_path):
    import json
    import numpy as np
    from forge_train_harness_b200.data import prepare
    from forge_train_harness_b200.data.sources import MegatronBinary
    f = tmp_path / "qa.jsonl"
    with open(f, "w") as fh:
        for j in range(20):
            fh.write(json.dumps({"question": f"q{j}", "answer": f"a{j}"}) + "\n")
        fh.write(json.dumps({"question": "", "answer": ""}) + "\n")
    assert prepare.main([str(f), "--out", str(tmp_path / "c"), "--tokenizer", "bytes", "--template", "gsm8k_qa"]) == 0
    src = MegatronBinary(str(tmp_path / "c"), 8, 1, 0, 1, 0)
    flat = np.concatenate([w for w in src.windows])
    assert int((flat == 256).sum()) >= 10 and flat.max() <= 256          # one EOS per document, byte ids otherwise
    text = bytes(int(x) for x in flat[:9]).decode()
    assert text.startswith("Question")


def test_profile_snapshot_verdict_compares_with_the_previous_snapshot(tmp_path):
    import json
    from forge_train_harness_b200.gates import verdicts as V

    def snap(run, kernels, span):
        d = tmp_path / run / "ours" / "profile"
        d.mkdir(parents=True)
        (d / "step_5_rank0.json").write_text(json.dumps({"kernels": kernels, "span_us": span, "busy_us": 0.9 * span, "idle_us": 0.1 * span,
                                                          "n_launches": sum(k["launches"] for k in kernels.values())}))
        return str(tmp_path / run)
    old = snap("profile-snapshot-20260101T000000-aaaaaa", {"gemm": {"launches": 10, "us": 5000.0}, "attn": {"launches": 4, "us": 3000.0}}, 10000.0)
    new = snap("profile-snapshot-20260102T000000-bbbbbb", {"gemm": {"launches": 10, "us": 4000.0}, "attn": {"launches": 4, "us": 3100.0},
                                                           "norm": {"launches": 8, "us": 200.0}}, 9000.0)
    first = V.profile(old)
    assert first["passed"] and first["n_kernels"] == 2 and "previous" not in first and abs(first["busy_pct"] - 90.0) < 1e-6
    r = V.profile(new)
    assert r["passed"] and r["previous"].startswith(old) and abs(r["delta_span_ms"] + 1.0) < 1e-9
    assert r["moved_most_ms"][0] == ["gemm", -1.0] and ["norm", 0.2] in r["moved_most_ms"] and r["top"][0][0] == "gemm"
    empty = snap("profile-snapshot-20260103T000000-cccccc", {}, 0.0)
    assert not V.profile(empty)["passed"] and V.profile(empty, require_kernels=False)["passed"]
    assert not V.profile(str(tmp_path / "nothing"))["passed"]


def test_hash_capture_is_switched_on_by_the_configuration(tmp_path):
    """train.hash_capture_level / train.hash_output (a gate product's keys) make the public entry point write per-rank hash dumps."""
    import subprocess
    import sys
    ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "ours_hash_dump.json"
    r = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.train", "--config", os.path.join(ROOT, "configs", "tiny_cpu_dp2.toml"),
                        "--set", "train.num_steps=2", "--set", "parallel.use_distributed_optimizer=false", "--set", "train.hash_capture_level=1",
                        "--set", f"train.hash_output={out}"], cwd=ROOT, capture_output=True, text=True, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stderr[-1500:]
    keys = cap.load_merged(str(out))
    assert any(".grad." in k and k.endswith("preallreduce") for k in keys) and any("loss.scalar.postallreduce" in k for k in keys)
    assert not any(".fwd." in k for k in keys)          # level 1: no per-module activations
    assert {k.split(".")[0] for k in keys} == {"step_0", "step_1"}   # keyed by the number of completed steps
