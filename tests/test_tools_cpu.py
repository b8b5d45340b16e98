"""Operator tools: canonical-state bootstrap, recipe -> shell env, data determinism check, batch capture
(reference: tools/bootstrap_canonical.py, tools/train_recipe_to_env.py, tools/hf_data_bitwise_check.py,
tools/capture_profile_batch.py)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import forge_train_harness_b200 as fth
from forge_train_harness_b200.data.sources import write_megatron_binary
from forge_train_harness_b200.harness import tools

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_canonical_bootstrap_matches_the_engine_reference_init(tmp_path):
    m = fth.preset("tiny")
    p1 = tools.write_canonical(m, str(tmp_path), seed=7, init_ones=True)
    p0 = tools.write_canonical(m, str(tmp_path), seed=7, init_ones=False)
    assert p1.endswith(os.path.join("ones", "canonical_state_fp32.pt")) and p0.endswith(os.path.join("no1", "canonical_state_fp32.pt"))
    s1, s0 = torch.load(p1, weights_only=True), torch.load(p0, weights_only=True)
    assert float(s1["norm.weight"][0]) == 1.0 and abs(float(s0["norm.weight"][0]) - 0.97) < 1e-7
    assert torch.equal(s1["layers.0.wqkv.weight"], s0["layers.0.wqkv.weight"])
    # an engine that loads it holds exactly what one initialised from the same seed holds
    cfg = fth.RunConfig(model=m, optim=fth.OptimConfig(), train=fth.TrainConfig(seed=7, dtype="fp32", cuda_graph=False), data=fth.DataConfig(prefetch_size=0))
    a = fth.Trainer(cfg, device="cpu")
    b = fth.Trainer(cfg.replace(ckpt={"checkpoint_root": os.path.dirname(p1)}), device="cpu")
    assert all(torch.equal(a.store.params[k], b.store.params[k]) for k in a.store.params)
    a.close(), b.close()


def test_recipe_env_lets_the_environment_win_and_rejects_unknown_tables(tmp_path):
    import tomllib
    rec = tomllib.load(open(os.path.join(ROOT, "configs", "eval", "recipe_wsd_sft_tiny.toml"), "rb"))
    lines = tools.recipe_env_lines(rec)
    assert 'export ORDER="${ORDER:-stable decay sft}"' in lines and 'export SFT_INIT_WEIGHTS_ONLY="${SFT_INIT_WEIGHTS_ONLY:-1}"' in lines
    assert 'export DECAY_LR_WSD_DECAY_ITERS="${DECAY_LR_WSD_DECAY_ITERS:-4}"' in lines
    sh = "\n".join(lines) + '\necho "$STABLE_LR|$DECAY_MIN_LR|$ORDER"\n'
    out = subprocess.run(["bash", "-c", sh], capture_output=True, text=True, env=dict(os.environ, STABLE_LR="9e-9")).stdout.strip()
    assert out == "9e-9|0.0002|stable decay sft"  # an exported variable beats the recipe; the rest are defaults
    with pytest.raises(ValueError, match="unknown recipe table"):
        tools.recipe_env_lines({"phazes": {"a": {"x": 1}}})
    assert tools.recipe_env_lines({"launch": {"gpus_per_node": 8}, "common": {"note": 'a "q" $x'}}) == \
        ['export GPUS_PER_NODE="${GPUS_PER_NODE:-8}"', 'export NOTE="${NOTE:-a \\"q\\" \\$x}"']


def _run_cfg(tmp_path):
    rng = np.random.RandomState(0)
    docs = [rng.randint(0, 8000, size=4000).astype(np.int32) for _ in range(6)]
    prefix = str(tmp_path / "corpus")
    write_megatron_binary(prefix, docs, np.int32)
    cfgp = tmp_path / "run.toml"
    cfgp.write_text(f'[model]\nname = "tiny"\nseq_length = 64\n[train]\nmicro_batch_size = 2\nseed = 5\n[data]\ndata_loader = "megatron_binary"\n'
                    f'data_path = {json.dumps(prefix)}\n')
    return str(cfgp)


def test_data_check_and_capture_batch(tmp_path):
    cfgp = _run_cfg(tmp_path)
    r = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.harness.tools", "data-check", "--config", cfgp, "--dp", "2", "--batches", "6"],
                       capture_output=True, text=True, cwd=ROOT)
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert r.returncode == 0 and res["passed"] and res["ranks"] == 2 and not res["ranks_share_samples"], r.stderr
    out = tmp_path / "in" / "captured_batch.pt"
    r = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.harness.tools", "capture-batch", "--config", cfgp, "--out", str(out)],
                       capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stderr
    b = torch.load(out, weights_only=True)
    assert b["tokens"].shape == (2, 64) and torch.equal(b["tokens"][:, 1:], b["labels"][:, :-1]) and float(b["loss_mask"].min()) == 1.0
    # a non-deterministic source is caught
    from forge_train_harness_b200.config import schema
    from forge_train_harness_b200.data import sources
    cfg = schema.load(cfgp)
    real = sources.MegatronBinary.__next__

    def noisy(self):
        b = real(self)
        b["tokens"] = b["tokens"] + torch.randint(0, 2, b["tokens"].shape)
        return b
    try:
        sources.MegatronBinary.__next__ = noisy
        assert not tools.data_check(cfg, 1, 4)["passed"]
    finally:
        sources.MegatronBinary.__next__ = real


def test_canonical_preflight_finds_what_would_waste_a_gate_run(tmp_path):
    m = fth.preset("tiny")
    path = tools.write_canonical(m, str(tmp_path), seed=3, init_ones=True)
    ok = tools.canonical_preflight(m, path)
    assert ok["passed"] and ok["tensors"] == len(list(fth.models.params.full_param_specs(m))) if hasattr(fth, "models") else ok["passed"]
    open(path + ".sha256", "w").write(ok["sha256"] + "  canonical_state_fp32.pt\n")
    assert tools.canonical_preflight(m, path)["passed"]
    state = torch.load(path, weights_only=True)
    state["layers.0.wo.weight"][0, 0] = float("nan")
    state["layers.1.w2.weight"] = state["layers.1.w2.weight"][:, :-1].contiguous()
    del state["norm.weight"]
    torch.save(state, path)
    bad = tools.canonical_preflight(m, path)
    text = " ".join(bad["problems"])
    assert not bad["passed"] and "sha256" in text and "missing norm.weight" in text and "not finite" in text and "layers.1.w2.weight: shape" in text
    import dataclasses
    assert not tools.canonical_preflight(dataclasses.replace(m, num_layers=3), str(tmp_path / "nope.pt"))["passed"]


def test_gate_sweep_runs_the_cpu_suites_in_milestone_order(tmp_path):
    from forge_train_harness_b200.harness.cli import main as cli_main
    import contextlib, io
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        rc = cli_main(["sweep", "--only", "multistep,production-train,dptp", "--max-gpus", "0", "--artifacts", str(tmp_path / "runs")])
    table = buf.getvalue().split("| suite | milestone | status | note |")[-1]
    assert rc == 0, buf.getvalue()[-3000:]
    lines = [ln for ln in table.splitlines() if ln.startswith("| ") and "---" not in ln]
    assert [ln.split("|")[1].strip() for ln in lines] == ["multistep", "dptp", "production-train"]   # milestone order
    assert "passed" in lines[0] and "skipped" in lines[1] and "needs 4 GPUs" in lines[1] and "passed" in lines[2]


def test_set_overrides_parse_every_field_kind():
    from forge_train_harness_b200.config import schema
    from forge_train_harness_b200.train import _apply_sets
    cfg = schema.load(os.path.join(ROOT, "configs", "minicpm4_8b_tp4pp2.toml"))
    assert cfg.parallel.pipeline_layer_split == (17, 15)
    c2 = _apply_sets(cfg, ["parallel.pipeline_layer_split=none", "parallel.pipeline_parallel_size=1", "parallel.sequence_parallel=false",
                           "train.init_mode=device", "optim.lr=3e-4", "train.num_steps=7", "train.save_path=none"])
    assert c2.parallel.pipeline_layer_split == () and c2.parallel.pipeline_parallel_size == 1 and c2.parallel.sequence_parallel is False
    assert c2.train.init_mode == "device" and c2.optim.lr == 3e-4 and c2.train.num_steps == 7 and c2.train.save_path is None
    assert _apply_sets(cfg, ["parallel.pipeline_layer_split=16,16"]).parallel.pipeline_layer_split == (16, 16)
    with pytest.raises(ValueError):
        _apply_sets(cfg, ["parallel.pipeline_layer_split=20,20"])      # must sum to the layer count


def test_reference_environment_surface_maps_onto_the_config():
    from forge_train_harness_b200.config import schema
    from forge_train_harness_b200.config.ref_env import apply_reference_env, op_env_from_reference
    cfg = schema.load(os.path.join(ROOT, "configs", "tiny_cpu_dp2.toml"))
    env = {"NUM_LAYERS": "3", "HIDDEN_SIZE": "128", "NUM_ATTENTION_HEADS": "2", "NUM_QUERY_GROUPS": "1", "HEAD_DIM": "64", "FFN_HIDDEN_SIZE": "256",
           "PADDED_VOCAB_SIZE": "1024", "MAX_POSITION_EMBEDDINGS": "64", "SEQ_LENGTH": "64", "NORM_EPSILON": "1e-5", "ROTARY_BASE": "10000",
           "LR": "3e-4", "MIN_LR": "3e-5", "LR_WARMUP_ITERS": "7", "CLIP_GRAD": "0.5", "DETERMINISTIC": "1", "ENABLE_ZERO_OPTIMIZER": "1",
           "ENABLE_CUDA_GRAPH": "0", "ENABLE_DL_PREFETCH": "0", "DL_PREFETCH_SIZE": "128", "FORGE_INIT_ONES": "0", "MTP_NUM_LAYERS": "0",
           "NCCL_ALGO": "Tree", "ENABLE_TRITON_ROPE_FWD": "0", "ENABLE_TRITON_RMSNORM_FWD": "1"}
    c = apply_reference_env(cfg, env)
    assert (c.model.num_layers, c.model.hidden_size, c.model.head_dim, c.model.padded_vocab_size, c.model.seq_length) == (3, 128, 64, 1024, 64)
    assert c.optim.lr == 3e-4 and c.optim.min_lr == 3e-5 and c.optim.lr_warmup_iters == 7 and c.optim.clip_grad == 0.5
    assert c.train.deterministic and not c.train.cuda_graph and not c.train.forge_init_ones and c.parallel.use_distributed_optimizer
    assert c.data.prefetch_size == 0                         # prefetch switched off beats its size
    assert c.optim.weight_decay == cfg.optim.weight_decay    # absent variables leave the file's value
    assert apply_reference_env(cfg, {}) is cfg
    assert op_env_from_reference(env) == {"OP_ROPE_FWD": "baseline", "OP_RMSNORM_FWD": "sm100", "OP_RESIDUAL_RMSNORM_FWD": "sm100"}
    with pytest.raises(ValueError, match="HIDDEN_SIZE"):
        apply_reference_env(cfg, {"HIDDEN_SIZE": "wide"})
    # and the engine trains from such an environment through its public entry point
    r = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.train", "--config", os.path.join(ROOT, "configs", "tiny_cpu_dp2.toml"),
                        "--reference-env", "--set", "train.num_steps=2", "--set", "parallel.use_distributed_optimizer=false"],
                       cwd=ROOT, capture_output=True, text=True, env=dict(os.environ, CUDA_VISIBLE_DEVICES="", NUM_LAYERS="1", LR="1e-3", SEQ_LENGTH="32",
                                                                          MAX_POSITION_EMBEDDINGS="32"))
    assert r.returncode == 0 and r.stdout.count("[LOSS]") == 2, r.stderr[-1500:]
    assert "lr=0.001" in r.stdout                            # the [PHASE] banner shows the variable's value
