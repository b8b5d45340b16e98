"""The engine against the reference's own L0 models, live, on CPU in fp32: the Qwen3 variant and MiniCPM4 with muP + MTP.

The MiniCPM model (ref/reference/model_pure_mup_mtp.py:326-436: fused wqkv, muP embedding / depth / width scales, one MTP
layer with its two input norms, the 2H -> H projection, a transformer layer and a final norm, LM head shared by both
branches) uses this engine's parameter names, so weights and gradients map one to one; the objective is the reference
trainer's ``lm_sum + weight * mtp_sum`` (train_pure_mup_mtp.py:752-765).

Qwen3:

The reference model (ref/reference/model_qwen3.py:102-269: separate q / k / v projections, per-head RMSNorm on q and k before
RoPE, tied embeddings, standard parameterisation) is imported UNMODIFIED from the installed reference tree; only the library
attention call it makes (``flash_attn.flash_attn_func``, GPU-only) is replaced by the same math in plain PyTorch.  Its weights
are copied into this engine (q / k / v rows interleaved per KV group into the fused ``wqkv``), both run one forward +
backward on the same batch, and the loss and EVERY parameter gradient must agree."""
import dataclasses
import importlib
import math
import os
import sys
import types

import pytest
import torch

import forge_train_harness_b200 as fth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref", "ref", "reference")

GEOM = dict(NUM_LAYERS=2, HIDDEN_SIZE=128, NUM_ATTENTION_HEADS=4, NUM_QUERY_GROUPS=2, HEAD_DIM=64, FFN_HIDDEN_SIZE=256,
            PADDED_VOCAB_SIZE=512, MAX_POSITION_EMBEDDINGS=64, NORM_EPSILON=1e-6, ROTARY_BASE=1000000)


def _attention_stub():
    def flash_attn_func(q, k, v, causal=True, deterministic=False, **kw):
        B, S, H, D = q.shape
        g = H // k.shape[2]
        kk, vv = k.repeat_interleave(g, dim=2), v.repeat_interleave(g, dim=2)
        s = torch.einsum("bshd,bthd->bhst", q, kk) / math.sqrt(D)
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
        return torch.einsum("bhst,bthd->bshd", s.softmax(-1), vv)
    m = types.ModuleType("flash_attn")
    m.flash_attn_func = flash_attn_func
    return m


@pytest.fixture()
def ref_qwen3(monkeypatch):
    if not os.path.isfile(os.path.join(REF, "model_qwen3.py")):
        pytest.skip("the reference tree is not installed under baseline/_ref")
    for k, v in GEOM.items():
        monkeypatch.setenv(k, str(v))
    monkeypatch.setitem(sys.modules, "flash_attn", _attention_stub())
    monkeypatch.syspath_prepend(REF)
    for name in ("model_qwen3", "model_pure_mup_mtp"):
        sys.modules.pop(name, None)
    mod = importlib.import_module("model_qwen3")
    yield mod
    for name in ("model_qwen3", "model_pure_mup_mtp"):
        sys.modules.pop(name, None)


def test_qwen3_variant_matches_the_reference_model(ref_qwen3):
    torch.manual_seed(0)
    ref = ref_qwen3.Qwen3Dense().float()
    ref.init_weights(init_std=0.02, seed=7)
    # norm weights away from 1 so that a wrong q_norm / k_norm wiring cannot hide
    g = torch.Generator().manual_seed(3)
    for n, p in ref.named_parameters():
        if p.ndim == 1:
            p.data.copy_(1.0 + 0.2 * torch.randn(p.shape, generator=g))

    m = dataclasses.replace(fth.preset("qwen3_0.6b"), num_layers=2, hidden_size=128, ffn_hidden_size=256, num_attention_heads=4,
                            num_query_groups=2, head_dim=64, seq_length=64, padded_vocab_size=512, max_position_embeddings=64)
    cfg = fth.RunConfig(model=m, optim=fth.OptimConfig(lr=1e-3, lr_schedule="constant"),
                        train=fth.TrainConfig(num_steps=1, micro_batch_size=2, seed=0, dtype="fp32", cuda_graph=False),
                        data=fth.DataConfig(prefetch_size=0))
    tr = fth.Trainer(cfg, device="cpu")
    sd = dict(ref.named_parameters())
    nkv, gq, d = m.num_query_groups, m.q_per_kv, m.head_dim

    def fuse(li):
        wq, wk, wv = (sd[f"layers.{li}.{n}.weight"].data for n in ("wq", "wk", "wv"))
        rows = []
        for j in range(nkv):
            rows += [wq[j * gq * d:(j + 1) * gq * d], wk[j * d:(j + 1) * d], wv[j * d:(j + 1) * d]]
        return torch.cat(rows, 0)

    def unfuse_grad(gw):
        gw = gw.view(nkv, gq + 2, d, -1)
        return gw[:, :gq].reshape(nkv * gq * d, -1), gw[:, gq].reshape(nkv * d, -1), gw[:, gq + 1].reshape(nkv * d, -1)

    for name, p in tr.store.params.items():
        if name.endswith("wqkv.weight"):
            p.copy_(fuse(int(name.split(".")[1])))
        else:
            p.copy_(sd[name].data)
    tr.weights_changed()

    tr.start_data()
    batch = tr.stager.stage(tr.prefetch.get())
    stats = tr._fwd_bwd(batch)
    ours_loss = float(stats[0])

    ids = batch["ids"].long().view(2, 64)
    labels, mask = batch["labels"].long().view(-1), batch["mask"].float().view(-1)
    rope = ref_qwen3.precompute_rope_freqs(64, device="cpu")
    logits, _ = ref(ids, rope)
    nll = torch.nn.functional.cross_entropy(logits.view(-1, 512).float(), labels, reduction="none")
    loss = (nll * mask).sum()
    loss.backward()
    ref_loss = float(loss.detach())
    assert abs(ours_loss - ref_loss) / abs(ref_loss) < 2e-6, (ours_loss, ref_loss)

    def ref_grad(name):
        p = sd[name]
        mg = getattr(p, "main_grad", None)  # weight gradients go to the fp32 side buffer, the rest to .grad
        return mg if mg is not None else p.grad

    worst = {}
    for name, gw in tr.store.grads.items():
        if name.endswith("wqkv.weight"):
            li = int(name.split(".")[1])
            pairs = zip(unfuse_grad(gw), (ref_grad(f"layers.{li}.{n}.weight") for n in ("wq", "wk", "wv")))
        else:
            pairs = [(gw, ref_grad(name))]
        for a, b in pairs:
            assert b is not None, name
            worst[name] = max(worst.get(name, 0.0), float((a - b).norm() / (b.norm() + 1e-30)))
    assert set(n.replace("wqkv", "wq") for n in worst) >= {"layers.0.q_norm.weight", "layers.1.k_norm.weight", "tok_embeddings.weight"}
    bad = {k: v for k, v in worst.items() if v > 2e-5}
    assert not bad, bad
    tr.close()


@pytest.fixture()
def ref_minicpm(monkeypatch):
    if not os.path.isfile(os.path.join(REF, "model_pure_mup_mtp.py")):
        pytest.skip("the reference tree is not installed under baseline/_ref")
    geom = dict(GEOM, HIDDEN_SIZE=128, NORM_EPSILON=1e-5, ROTARY_BASE=10000)
    for k, v in geom.items():
        monkeypatch.setenv(k, str(v))
    monkeypatch.setitem(sys.modules, "flash_attn", _attention_stub())
    monkeypatch.syspath_prepend(REF)
    sys.modules.pop("model_pure_mup_mtp", None)
    mod = importlib.import_module("model_pure_mup_mtp")
    yield mod
    sys.modules.pop("model_pure_mup_mtp", None)


def test_minicpm_mup_mtp_matches_the_reference_model(ref_minicpm):
    ref = ref_minicpm.MiniCPM4MupMtp(eagle_num_layers=1).float()
    ref.init_weights(init_std=0.05, seed=11, init_ones=True)
    g = torch.Generator().manual_seed(5)
    for n, p in ref.named_parameters():
        if p.ndim == 1:
            p.data.copy_(1.0 + 0.2 * torch.randn(p.shape, generator=g))
    m = fth.ModelConfig(name="mtp_tiny", num_layers=2, hidden_size=128, ffn_hidden_size=256, num_attention_heads=4, num_query_groups=2,
                        head_dim=64, seq_length=64, padded_vocab_size=512, norm_epsilon=1e-5, rotary_base=10000.0,
                        mtp_num_layers=1, mtp_loss_weight=0.3, tie_embeddings=False)
    cfg = fth.RunConfig(model=m, optim=fth.OptimConfig(lr=1e-3, lr_schedule="constant"),
                        train=fth.TrainConfig(num_steps=1, micro_batch_size=2, seed=0, dtype="fp32", cuda_graph=False),
                        data=fth.DataConfig(prefetch_size=0))
    tr = fth.Trainer(cfg, device="cpu")
    sd = dict(ref.named_parameters())
    assert set(tr.store.params) == set(sd), set(tr.store.params) ^ set(sd)
    for name, p in tr.store.params.items():
        p.copy_(sd[name].data)
    tr.weights_changed()
    tr.start_data()
    batch = tr.stager.stage(tr.prefetch.get())
    stats = tr._fwd_bwd(batch)

    ids = batch["ids"].long().view(2, 64)
    labels, mask = batch["labels"].long().view(2, 64), batch["mask"].float().view(2, 64)
    # the reference trainer's own MTP shift (train_pure_mup_mtp.py:456-471), restated
    mtp_in = labels.clone()
    mtp_lab = torch.zeros_like(labels)
    mtp_lab[:, :-1] = labels[:, 1:]
    mtp_mask = torch.zeros_like(mask)
    mtp_mask[:, :-1] = mask[:, :-1] * mask[:, 1:]
    assert torch.equal(batch["mtp_ids"].long().view(2, 64), mtp_in) and torch.equal(batch["mtp_labels"].long().view(2, 64), mtp_lab)
    rope = ref_minicpm.precompute_rope_freqs(64, device="cpu") if "device" in ref_minicpm.precompute_rope_freqs.__code__.co_varnames \
        else ref_minicpm.precompute_rope_freqs(64)
    logits, logits_mtp = ref(ids, rope, mtp_input_ids=mtp_in)
    ce = torch.nn.functional.cross_entropy
    lm = (ce(logits.view(-1, 512), labels.view(-1), reduction="none") * mask.view(-1)).sum()
    mt = (ce(logits_mtp.view(-1, 512), mtp_lab.view(-1), reduction="none") * mtp_mask.view(-1)).sum()
    (lm + 0.3 * mt).backward()
    assert abs(float(stats[0]) - float(lm.detach())) / float(lm.detach()) < 2e-6
    assert abs(float(stats[2]) - float(mt.detach())) / float(mt.detach()) < 2e-6
    bad = {}
    for name, gw in tr.store.grads.items():
        p = sd[name]
        b = getattr(p, "main_grad", None)
        b = b if b is not None else p.grad
        assert b is not None, name
        err = float((gw - b).norm() / (b.norm() + 1e-30))
        if err > 2e-5:
            bad[name] = err
    assert not bad, bad
    tr.close()


def test_reference_order_init_is_bit_identical_for_both_model_families(ref_qwen3):
    """``init_reference`` must reproduce the reference's own ``init_weights`` (same generator, same draw order): it is what lets
    a gate start both sides from equal weights without exchanging a file."""
    from forge_train_harness_b200.ckpt.hf_names import split_qkv
    from forge_train_harness_b200.models import params as P
    ref = ref_qwen3.Qwen3Dense().float()
    ref.init_weights(init_std=0.02, seed=1234)
    sd = dict(ref.named_parameters())
    m = dataclasses.replace(fth.preset("qwen3_0.6b"), num_layers=2, hidden_size=128, ffn_hidden_size=256, num_attention_heads=4,
                            num_query_groups=2, head_dim=64, seq_length=64, padded_vocab_size=512, max_position_embeddings=64)
    n = 0
    for spec, t in P.iter_full_init(m, 1234, True):
        if spec.name.endswith("wqkv.weight"):
            li = spec.name.split(".")[1]
            for part, nm in zip(split_qkv(t, m), ("wq", "wk", "wv")):
                assert torch.equal(part, sd[f"layers.{li}.{nm}.weight"].data), (spec.name, nm)
        else:
            assert torch.equal(t, sd[spec.name].data), spec.name
        n += 1
    assert n == len(P.full_param_specs(m))
