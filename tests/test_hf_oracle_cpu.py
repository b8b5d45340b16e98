"""The Hugging Face single-card oracle (the reference's framework-native cross-check of the 8B model, ref/reference/
train_minicpm4_8b_hf_singlecard.py) against this engine, on CPU in fp32 at a shrunken width, plus the name / layout map."""
import json
import os
import subprocess
import sys

import pytest
import torch

import forge_train_harness_b200 as fth
from forge_train_harness_b200.ckpt import hf_names

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))
import hf_oracle  # noqa: E402


def test_name_map_round_trip_is_exact():
    m = fth.ModelConfig(num_layers=2, hidden_size=256, ffn_hidden_size=512, num_attention_heads=4, num_query_groups=2, head_dim=64,
                        seq_length=64, padded_vocab_size=512, qk_norm=True)
    from forge_train_harness_b200.models import params as P
    g = torch.Generator().manual_seed(0)
    state = {s.name: torch.randn(s.full_shape, generator=g) for s in P.full_param_specs(m)}
    hf = hf_names.engine_to_hf(state, m)
    assert hf["model.layers.1.self_attn.q_proj.weight"].shape == (256, 256) and hf["model.layers.1.self_attn.k_proj.weight"].shape == (128, 256)
    assert "model.layers.0.self_attn.q_norm.weight" in hf and "lm_head.weight" in hf
    back = hf_names.hf_to_engine(hf, m)
    assert set(back) == set(state) and all(torch.equal(back[k], state[k]) for k in state)
    # head h of q_proj is query head (h % g) of KV group (h // g) in the fused layout
    q = hf["model.layers.0.self_attn.q_proj.weight"].view(4, 64, 256)
    fused = state["layers.0.wqkv.weight"].view(2, 4, 64, 256)
    assert torch.equal(q[3], fused[1, 1]) and torch.equal(hf["model.layers.0.self_attn.v_proj.weight"].view(2, 64, 256)[0], fused[0, 3])


@pytest.mark.timeout(600)
def test_training_trajectory_matches_the_hf_oracle(tmp_path):
    why = hf_oracle.available()
    if why:
        pytest.skip(why)
    env = dict(os.environ, HF_MODULES_CACHE=str(tmp_path / "hf_modules"))
    r = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.gates.run_hf_oracle", "--layers", "2", "--hidden", "256", "--seq", "64",
                        "--vocab", "512", "--steps", "10", "--window", "4", "11", "--mbs", "2", "--accum", "2", "--lr", "3e-3",
                        "--warmup", "2", "--device", "cpu", "--dtype", "fp32", "--threshold", "1e-3", "--first-tol", "1e-5",
                        "--out", str(tmp_path / "out")], cwd=ROOT, env=env, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    res = json.loads(r.stdout.strip().splitlines()[-1])
    # model, muP scaling, loss, clipping, AdamW groups, schedule and data order all agree with the independent implementation
    assert res["passed"] and res["first_step"]["rel_diff"] < 1e-6 and res["trend"]["mean_rel_diff"] < 2e-4, res
    gn = res["grad_norm_first"]
    assert abs(gn["ref"] - gn["ours"]) / gn["ref"] < 1e-5


def test_exported_checkpoint_loads_into_the_hf_model_and_gives_the_same_loss(tmp_path, monkeypatch):
    """A trained checkpoint exported under HF names (``python -m forge_train_harness_b200.ckpt.hf_names``) is a drop-in state
    dict of the bundled ``MiniCPMForCausalLM``: strict load, same loss on the same batch."""
    why = hf_oracle.available()
    if why:
        pytest.skip(why)
    from forge_train_harness_b200.ckpt import manager
    monkeypatch.setenv("HF_MODULES_CACHE", str(tmp_path / "hf_modules"))
    m = fth.ModelConfig(name="exp", num_layers=2, hidden_size=256, ffn_hidden_size=512, num_attention_heads=4, num_query_groups=2, head_dim=64,
                        seq_length=64, padded_vocab_size=512, norm_epsilon=1e-6, tie_embeddings=False)
    cfg = fth.RunConfig(model=m, optim=fth.OptimConfig(lr=2e-3, lr_schedule="constant"),
                        train=fth.TrainConfig(num_steps=2, micro_batch_size=2, seed=3, dtype="fp32", cuda_graph=False),
                        data=fth.DataConfig(prefetch_size=0))
    tr = fth.Trainer(cfg, device="cpu")
    tr.start_data()
    tr.train_step()
    tr.train_step()
    manager.save(tr, str(tmp_path / "ckpt"))
    out = tmp_path / "hf_state.pt"
    r = subprocess.run([sys.executable, "-m", "forge_train_harness_b200.ckpt.hf_names", str(tmp_path / "ckpt"), str(out), "--dtype", "fp32"],
                       cwd=ROOT, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    hf, _ = hf_oracle.build_model(m, 0, "cpu", torch.float32)
    hf.load_state_dict(torch.load(out, weights_only=True), strict=True)
    batch = tr.stager.stage(tr.prefetch.get())
    batch = {k: (v.clone() if hasattr(v, "clone") else v) for k, v in batch.items()}
    tr.store.zero_grad()
    stats = tr._fwd_bwd(batch)
    logits = hf(input_ids=batch["ids"].long().view(2, 64)).logits
    nll = torch.nn.functional.cross_entropy(logits.view(-1, 512).float(), batch["labels"].long().view(-1), reduction="none")
    ref = float((nll * batch["mask"].float().view(-1)).sum().detach())
    assert abs(float(stats[0]) - ref) / ref < 2e-6, (float(stats[0]), ref)
    tr.close()
