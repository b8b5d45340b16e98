"""Config 1: tiny MiniCPM4 decoder on CPU — manual backward vs autograd, training step sanity."""
import math

import torch

import forge_train_harness_b200 as fth
from forge_train_harness_b200.ops import TorchOps


def tiny_cfg(**train):
    t = dict(num_steps=3, micro_batch_size=2, grad_accum_steps=1, seed=0, dtype="fp32", cuda_graph=False)
    t.update(train)
    return fth.RunConfig(model=fth.preset("tiny"), optim=fth.OptimConfig(lr=1e-3, lr_schedule="constant"),
                         train=fth.TrainConfig(**t), data=fth.DataConfig(prefetch_size=0))


def autograd_loss(tr, batch):
    """Same network written with autograd-tracked torch ops on leaf copies of the parameters."""
    cfg = tr.cfg.model
    P = {k: v.detach().clone().double().requires_grad_(True) for k, v in tr.store.params.items()}
    ids, labels, mask = batch["ids"].long(), batch["labels"].long(), batch["mask"].double()
    S, d, nkv, g = cfg.seq_length, cfg.head_dim, cfg.num_query_groups, cfg.q_per_kv
    B = ids.numel() // S
    table = tr.rope.double()

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.norm_epsilon) * w

    def rope(t):  # [B,S,h,d]
        half = d // 2
        cos, sin = table[:S, :half].view(1, S, 1, half), table[:S, half:].view(1, S, 1, half)
        x1, x2 = t[..., :half], t[..., half:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    x = torch.nn.functional.embedding(ids, P["tok_embeddings.weight"]) * cfg.emb_scale
    ds = cfg.depth_scale()
    for li in range(cfg.num_layers):
        p = f"layers.{li}."
        qkv = (norm(x, P[p + "attention_norm.weight"]) @ P[p + "wqkv.weight"].t()).view(B, S, nkv, g + 2, d)
        q = rope(qkv[:, :, :, :g].reshape(B, S, nkv * g, d))
        k = rope(qkv[:, :, :, g])
        v = qkv[:, :, :, g + 1]
        k = k.repeat_interleave(g, dim=2)
        v = v.repeat_interleave(g, dim=2)
        s = torch.einsum("bshd,bthd->bhst", q, k) / math.sqrt(d)
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
        a = torch.einsum("bhst,bthd->bshd", s.softmax(-1), v).reshape(B * S, nkv * g * d)
        x = x + (a @ P[p + "wo.weight"].t()) * ds
        gu = norm(x, P[p + "ffn_norm.weight"]) @ P[p + "wfc1.weight"].t()
        gate, up = gu.chunk(2, -1)
        x = x + ((torch.nn.functional.silu(gate) * up) @ P[p + "w2.weight"].t()) * ds
    h = norm(x, P["norm.weight"]) / cfg.width_mult
    wout = P["tok_embeddings.weight"] if cfg.tie_embeddings else P["output.weight"]
    nll = torch.nn.functional.cross_entropy(h @ wout.t(), labels, reduction="none")
    loss = (nll * mask).sum()
    loss.backward()
    return loss.detach(), {k: v.grad for k, v in P.items()}


def test_manual_backward_matches_autograd():
    cfg = tiny_cfg()
    cfg = cfg.replace(model={"seq_length": 32, "padded_vocab_size": 512})
    tr = fth.Trainer(cfg, device="cpu")
    tr.start_data()
    batch = tr.stager.stage(tr.prefetch.get())
    # run in float64 for a tight comparison
    tr.store.flat_param = tr.store.flat_param  # fp32 params
    stats = tr._fwd_bwd(batch)
    ref_loss, ref_grads = autograd_loss(tr, batch)
    assert abs(float(stats[0]) - float(ref_loss)) / abs(float(ref_loss)) < 1e-5
    for name, g in tr.store.grads.items():
        r = ref_grads[name].float()
        err = (g - r).abs().max() / (r.abs().max() + 1e-12)
        assert err < 2e-4, (name, float(err))
    tr.close()


def test_loss_decreases():
    cfg = tiny_cfg(num_steps=6)
    cfg = cfg.replace(model={"seq_length": 64, "padded_vocab_size": 256}, optim={"lr": 3e-3})
    recs = fth.run_training_loop(cfg)
    assert len(recs) == 6
    assert recs[-1].loss < recs[0].loss
    assert all(math.isfinite(r.grad_norm) for r in recs)


def test_kernel_status_stops_the_step_before_it_is_logged_or_saved(tmp_path):
    """A kernel whose bounded wait ran out returns early and leaves wrong data behind.  The loop must raise after the
    step's sync, before the loss line is printed and before a checkpoint is written (fake status reader: code 5)."""
    import io

    import pytest
    cfg = tiny_cfg(num_steps=2, save_path=str(tmp_path / "ck"), save_interval=1)
    cfg = cfg.replace(model={"seq_length": 32, "padded_vocab_size": 256})
    tr = fth.Trainer(cfg, device="cpu", quiet=True)
    assert tr._read_status is None          # no sm_100a kernel can run here: nothing to read
    tr.verify_kernels()                      # and nothing raises
    codes = iter([0, 5])
    tr._read_status = lambda: next(codes)
    out = io.StringIO()
    with pytest.raises(RuntimeError, match="status 5.*peer flag never set"):
        fth.run_training_loop(cfg, trainer=tr, out=out)
    lines = [l for l in out.getvalue().splitlines() if l.startswith("[LOSS")]
    assert len(lines) == 1                   # the first step was fine and logged; the second was not
    assert not (tmp_path / "ck" / "iter_0000002").exists()
    tr._read_status = lambda: 3
    with pytest.raises(RuntimeError, match="accumulator never committed"):
        tr.train_step(verify=True)
    tr.close()


def test_debug_checks_catch_a_corrupt_batch():
    """``train.debug_checks``: a token id or a label outside the vocabulary stops the step with its position, instead of being
    skipped like another vocabulary shard's token."""
    import pytest
    cfg = tiny_cfg(debug_checks=True).replace(model={"seq_length": 32, "padded_vocab_size": 512})
    tr = fth.Trainer(cfg, device="cpu")
    tr.start_data()
    batch = tr.stager.stage(tr.prefetch.get())
    tr._fwd_bwd({k: (v.clone() if hasattr(v, "clone") else v) for k, v in batch.items()})   # a clean batch passes
    bad = {k: (v.clone() if hasattr(v, "clone") else v) for k, v in batch.items()}
    bad["ids"][7] = 512
    with pytest.raises(ValueError, match=r"index 512 at position 7 lies outside \[0, 512\)"):
        tr._fwd_bwd(bad)
    bad = {k: (v.clone() if hasattr(v, "clone") else v) for k, v in batch.items()}
    bad["labels"][3] = -1
    with pytest.raises(ValueError, match="position 3"):
        tr._fwd_bwd(bad)
    tr.close()
    # off by default: the same batch is accepted (the op skips the id), which is what vocabulary parallelism relies on
    tr2 = fth.Trainer(tiny_cfg().replace(model={"seq_length": 32, "padded_vocab_size": 512}), device="cpu")
    assert not tr2.chunks[0].debug_checks
    tr2.close()
