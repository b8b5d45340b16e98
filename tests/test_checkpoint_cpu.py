"""Save -> resume equivalence (bitwise), legacy codec, resharding across TP/PP/DP layouts, crash tolerance."""
import json
import os

import pytest
import torch

import forge_train_harness_b200 as fth
from forge_train_harness_b200.ckpt import manager as ckpt
from tests._mp import run_ranks
from tests.test_parallel_cpu import base_cfg


def _run(cfg, n):
    tr = fth.Trainer(cfg, device="cpu", quiet=True)
    return tr, [tuple(float(x) for x in (r["loss"], r["grad_norm"])) for r in (tr.train_step() for _ in range(n))]


@pytest.mark.parametrize("fmt", ["megatron_dist", "legacy"])
def test_resume_bitwise(tmp_path, fmt):
    cfg = base_cfg(steps=6).replace(ckpt={"format": fmt})
    tr, full = _run(cfg, 6)
    tr.close()
    tr, first = _run(cfg, 3)
    ckpt.save(tr, str(tmp_path))
    tr.close()
    tr2 = fth.Trainer(cfg, device="cpu", quiet=True)
    assert ckpt.load(tr2, str(tmp_path)) == 3
    rest = [tuple(float(x) for x in (r["loss"], r["grad_norm"])) for r in (tr2.train_step() for _ in range(3))]
    tr2.close()
    assert first + rest == full  # bitwise: identical floats


def test_weights_only_load_resets_optimizer(tmp_path):
    cfg = base_cfg(steps=2)
    tr, _ = _run(cfg, 2)
    ckpt.save(tr, str(tmp_path))
    w = tr.store.flat_param.clone()
    tr.close()
    tr2 = fth.Trainer(cfg.replace(train={"seed": 99}), device="cpu", quiet=True)
    ckpt.load(tr2, str(tmp_path), weights_only=True)
    assert torch.equal(tr2.store.flat_param, w)
    assert tr2.step == 0 and tr2.opt.step_count == 0 and float(tr2.opt.m.abs().sum()) == 0.0
    tr2.close()


def test_incomplete_checkpoint_is_ignored(tmp_path):
    cfg = base_cfg(steps=2)
    tr, _ = _run(cfg, 2)
    ckpt.save(tr, str(tmp_path))
    tr.close()
    os.makedirs(tmp_path / "iter_0000009.tmp" / "mp_rank_00")  # a writer died mid-save
    os.makedirs(tmp_path / "iter_0000007")  # no metadata.json -> incomplete
    (tmp_path / ckpt.TRACKER).write_text("7")  # tracker points at the broken one
    assert ckpt.latest_iteration(str(tmp_path)) == 2


def _save_layout(rank, world, cfg, path, n):
    tr = fth.Trainer(cfg, device="cpu", quiet=True)
    out = [float(tr.train_step()["loss"]) for _ in range(n)]
    ckpt.save(tr, path)
    tr.close()
    return out


def _load_layout(rank, world, cfg, path, n):
    tr = fth.Trainer(cfg, device="cpu", quiet=True)
    ckpt.load(tr, path)
    out = [float(tr.train_step()["loss"]) for _ in range(n)]
    tr.close()
    return out


def test_reshard_tp2pp2_to_dp2_zero_and_single(tmp_path):
    a = base_cfg(tensor_parallel_size=2, pipeline_parallel_size=2, sequence_parallel=True, gbs=8)
    full = run_ranks(4, _save_layout, a.replace(train={"num_steps": 5}), str(tmp_path / "full"), 5)[0]
    first = run_ranks(4, _save_layout, a, str(tmp_path / "ck"), 3)[0]
    b = base_cfg(use_distributed_optimizer=True, gbs=8, ddp_bucket_elems=20000)
    rest = run_ranks(2, _load_layout, b, str(tmp_path / "ck"), 2)[0]
    for x, y in zip(full, first + rest):
        assert abs(x - y) / abs(x) < 2e-4
    c = base_cfg(gbs=8)
    tr = fth.Trainer(c, device="cpu", quiet=True)
    assert ckpt.load(tr, str(tmp_path / "ck")) == 3
    l4 = float(tr.train_step()["loss"])
    tr.close()
    assert abs(l4 - full[3]) / abs(full[3]) < 2e-4


def test_legacy_codec_round_trips_with_the_reference(tmp_path):
    """``step_<N>/training_state.pt`` written here is read by the reference's own ``load_checkpoint`` and the other way
    round (weights, both moments, step counters and all four RNG states); run in a child process because the reference
    reads its model geometry from the environment when it is imported."""
    import subprocess
    import sys
    ref_root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "training_engine_tensor")):
        pytest.skip("the reference is not installed under baseline/_ref")
    env = dict(os.environ, NUM_LAYERS="4", HIDDEN_SIZE="64", NUM_ATTENTION_HEADS="4", NUM_QUERY_GROUPS="2", HEAD_DIM="16",
               FFN_HIDDEN_SIZE="128", PADDED_VOCAB_SIZE="512", MAX_POSITION_EMBEDDINGS="64", NORM_EPSILON="1e-5",
               ROTARY_BASE="10000")
    r = subprocess.run([sys.executable, os.path.join(os.path.dirname(__file__), "_legacy_codec_worker.py"), str(tmp_path)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "LEGACY_CODEC_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_megatron_binary_cursor_moves_between_dp_degrees(tmp_path):
    """The saved data position of an indexed corpus is a per-rank count: loading it at another DP degree must resume at
    the same GLOBAL position (same set of consumed samples), or refuse when that is impossible."""
    import numpy as np
    from forge_train_harness_b200.data.sources import MegatronBinary, write_megatron_binary
    rng = np.random.RandomState(0)
    docs = [rng.randint(0, 1000, size=rng.randint(40, 90)).astype(np.int32) for _ in range(300)]
    prefix = str(tmp_path / "corpus")
    write_megatron_binary(prefix, docs)
    S, mbs, seed = 16, 2, 11

    def consume(dp, steps_mb, states=None):
        """Run all ranks of a dp-way group for ``steps_mb`` micro-batches each; returns (rows seen, state of rank 0)."""
        seen, st0 = [], None
        for r in range(dp):
            src = MegatronBinary(prefix, S, mbs, r, dp, seed)
            if states is not None:
                src.load_state_dict(states)
            for _ in range(steps_mb):
                b = next(src)
                seen += [tuple(row.tolist()) for row in b["tokens"]]
            if r == 0:
                st0 = src.state_dict()
        return seen, st0

    first, st = consume(2, 6)                      # 2 ranks x 6 micro-batches x 2 = 24 samples
    assert st["consumed_in_epoch"] == 24 and st["dp_size"] == 2
    rest4, _ = consume(4, 2, st)                   # resume on 4 ranks
    ref_all, _ = consume(1, 20)                    # one rank reading the same shared order: first 40 samples
    assert sorted(first) == sorted(ref_all[:24])
    assert sorted(rest4) == sorted(ref_all[24:40])
    bad = dict(st, pos=5, consumed_in_epoch=10)    # 10 samples do not split over 4 ranks
    with pytest.raises(ValueError, match="do not split evenly"):
        MegatronBinary(prefix, S, mbs, 0, 4, seed).load_state_dict(bad)
    with pytest.raises(ValueError, match="epoch 1"):
        MegatronBinary(prefix, S, mbs, 0, 4, seed).load_state_dict(dict(st, epoch=1))
    same = MegatronBinary(prefix, S, mbs, 1, 2, seed)
    same.load_state_dict(dict(st, epoch=1))        # same layout: any epoch restores directly
    assert same.epoch == 1 and same.pos == st["pos"]


def _load_layout_stats(rank, world, cfg, path, n):
    tr = fth.Trainer(cfg, device="cpu", quiet=True)
    ckpt.load(tr, path)
    out = [float(tr.train_step()["loss"]) for _ in range(n)]
    stats = (getattr(tr, "last_load_bytes", 0), int(tr.opt.master.numel()) * 4 * 3)
    tr.close()
    return out, stats


def test_distributed_payload_reshards_tp2pp2dp2_to_tp4_and_dp4_and_exports(tmp_path):
    """Every DP rank writes its own optimizer shard; another layout reads only the slices it needs (here: at most a few
    times its own shard, not the whole checkpoint), continues with the same losses, and the exporter rewrites the
    checkpoint under Megatron names at a chosen TP x PP."""
    a = base_cfg(tensor_parallel_size=2, pipeline_parallel_size=2, sequence_parallel=True, use_distributed_optimizer=True, gbs=16,
                 ddp_bucket_elems=20000)
    full = run_ranks(8, _save_layout, a.replace(train={"num_steps": 5}), str(tmp_path / "full"), 5)[0]
    first = run_ranks(8, _save_layout, a, str(tmp_path / "ck"), 3)[0]
    it = tmp_path / "ck" / "iter_0000003"
    shards = sorted(p.name for p in (it / "mp_rank_00_000").iterdir())
    assert shards == ["distrib_optim_dp000.pt", "distrib_optim_dp001.pt", "layout.json", "model_optim_rng.pt"]
    one = torch.load(it / "mp_rank_00_000" / "distrib_optim_dp001.pt", weights_only=False)
    assert one["dp_rank"] == 1 and one["dp_world"] == 2 and "rng_state" in one and one["master"].dim() == 1
    meta = json.load(open(it / "metadata.json"))
    assert meta["version"] == 2 and set(meta["mp"]) == {"mp_rank_00_000", "mp_rank_01_000", "mp_rank_00_001", "mp_rank_01_001"}
    total_bytes = sum(l["numel"] for l in meta["mp"].values()) * 4 * 3
    b = base_cfg(tensor_parallel_size=4, sequence_parallel=True, gbs=16)
    res = run_ranks(4, _load_layout_stats, b, str(tmp_path / "ck"), 2)
    for x, y in zip(full, first + res[0][0]):
        assert abs(x - y) / abs(x) < 2e-4
    for _, (asked, own) in res:
        assert 0 < asked < 0.6 * total_bytes      # a TP-4 rank needs its rows of every tensor, not the whole checkpoint
    c = base_cfg(use_distributed_optimizer=True, gbs=16, ddp_bucket_elems=20000)
    res4 = run_ranks(4, _load_layout_stats, c, str(tmp_path / "ck"), 2)
    for x, y in zip(full, first + res4[0][0]):
        assert abs(x - y) / abs(x) < 2e-4
    # exporter: Megatron names, TP 2 x PP 2, shapes of the local shards
    from forge_train_harness_b200.ckpt.export_megatron import export, megatron_name
    out = export(str(tmp_path / "ck"), str(tmp_path / "mg"), tp=2, pp=2, impl="te", dtype="fp32")
    sd = torch.load(os.path.join(out, "mp_rank_01_001", "model_optim_rng.pt"), weights_only=False)
    m = a.model
    names = set(sd["model"])
    assert "decoder.final_layernorm.weight" in names and "output_layer.weight" in names and "embedding.word_embeddings.weight" not in names
    assert sd["model"]["decoder.layers.0.self_attention.linear_qkv.weight"].shape == (m.qkv_dim // 2, m.hidden_size)
    assert sd["model"]["decoder.layers.1.mlp.linear_fc1.weight"].shape == (2 * m.ffn_hidden_size // 2, m.hidden_size)
    assert sd["model"]["decoder.layers.0.mlp.linear_fc2.weight"].shape == (m.hidden_size, m.ffn_hidden_size // 2)
    assert sd["args"]["tensor_model_parallel_size"] == 2 and sd["iteration"] == 3
    s0 = torch.load(os.path.join(out, "mp_rank_00_000", "model_optim_rng.pt"), weights_only=False)
    assert "embedding.word_embeddings.weight" in s0["model"] and "decoder.layers.1.self_attention.linear_proj.weight" in s0["model"]
    assert megatron_name("layers.3.ffn_norm.weight", 1, "local") == "decoder.layers.1.pre_mlp_layernorm.weight"


def test_weights_round_trip_through_megatron_layout_and_hf_names(tmp_path):
    """Export a trained checkpoint as Megatron per-rank files at TP 2 x PP 2, import it back: every master weight returns bit
    for bit, and an engine started from the imported file holds exactly the trained weights.  Same through HF names."""
    import dataclasses
    from forge_train_harness_b200.ckpt import hf_names, import_weights, manager
    from forge_train_harness_b200.ckpt.export_megatron import export
    from forge_train_harness_b200.models import params as P
    m = fth.ModelConfig(name="rt", num_layers=4, hidden_size=128, ffn_hidden_size=256, num_attention_heads=4, num_query_groups=2, head_dim=32,
                        seq_length=32, padded_vocab_size=512, tie_embeddings=False)
    cfg = fth.RunConfig(model=m, optim=fth.OptimConfig(lr=2e-3, lr_schedule="constant"),
                        train=fth.TrainConfig(num_steps=2, micro_batch_size=2, seed=1, dtype="fp32", cuda_graph=False),
                        data=fth.DataConfig(prefetch_size=0))
    tr = fth.Trainer(cfg, device="cpu")
    tr.start_data()
    tr.train_step()
    tr.train_step()
    manager.save(tr, str(tmp_path / "ck"))
    trained = {k: v.detach().clone() for k, v in tr.store.params.items()}
    tr.close()
    export(str(tmp_path / "ck"), str(tmp_path / "mg"), tp=2, pp=2, impl="local", dtype="fp32")
    back = import_weights.from_megatron(str(tmp_path / "mg"), m, impl="local")
    assert set(back) == set(trained) and all(torch.equal(back[k], trained[k]) for k in trained)
    import_weights.write_canonical(back, str(tmp_path / "canon"))
    tr2 = fth.Trainer(cfg.replace(ckpt={"checkpoint_root": str(tmp_path / "canon")}), device="cpu")
    assert all(torch.equal(tr2.store.params[k], trained[k]) for k in trained)
    tr2.close()
    # wrong implementation flavour / wrong shape are errors, not silent partial loads
    with pytest.raises(KeyError, match="layer_norm_weight"):
        import_weights.from_megatron(str(tmp_path / "mg"), m, impl="te")
    with pytest.raises((ValueError, KeyError)):
        import_weights.from_megatron(str(tmp_path / "mg"), dataclasses.replace(m, ffn_hidden_size=512), impl="local")
    # HF names: there and back
    hf = hf_names.engine_to_hf(trained, m)
    eng = import_weights.from_hf(hf, m)
    assert all(torch.equal(eng[k], trained[k]) for k in trained)
    del hf["model.layers.2.mlp.up_proj.weight"]
    with pytest.raises(KeyError):
        import_weights.from_hf(hf, m)
    # the command line
    torch.save(hf_names.engine_to_hf(trained, m), tmp_path / "hf.pt")
    assert len([s for s in P.full_param_specs(m)]) == len(trained)
