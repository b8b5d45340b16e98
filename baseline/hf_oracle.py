"""Single-card oracle built on the Hugging Face modeling code the reference bundles (its independent cross-check of the 8B
model: ref/reference/train_minicpm4_8b_hf_singlecard.py, ref/reference/minicpm4_8b_hf_singlecard/{model,optim,train}.py).

``transformers`` builds and runs ``MiniCPMForCausalLM`` from the ``hf_model/`` directory shipped inside the installed
reference tree (no download; the remote-code cache is kept inside this repository); the muP forward scaling (``scale_emb``,
``scale_depth``, ``dim_model_base``) is whatever that modeling code does, not this repository's.  The oracle trains it on one
device with the recipe the reference's script describes: low-precision parameters with fp32 master copies, AdamW with
weight decay on matrices only and the muP learning-rate rule (block matrices at ``lr / width_mult``; embeddings, head and
norms at ``lr``), gradient clipping, linear warm-up then cosine decay.

Two additions make it usable as the reference side of a gate: it reads the same ``.bin/.idx`` corpus as the engine, and it
writes its initial weights as ``canonical_state_fp32.pt`` under this engine's parameter names so that both sides start from
the same numbers.  It prints its own ``step | loss | ...`` lines and the ``[LOSS]`` wire line.

    python baseline/hf_oracle.py --model minicpm4_8b --layers 4 --steps 50 --mbs 1 --accum 8 --data-prefix <dir>/corpus \
        --ckpt-root <dir> [--device cuda:0] [--dtype bf16]
"""
from __future__ import annotations

import argparse
import dataclasses
import math
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
HF_DIR = os.path.join(HERE, "_ref", "ref", "reference", "minicpm4_8b_hf_singlecard", "hf_model")


def available() -> str:
    """Empty string if the oracle can be built here, else the reason."""
    if not os.path.isfile(os.path.join(HF_DIR, "modeling_minicpm.py")):
        return "the reference tree with hf_model/ is not installed under baseline/_ref"
    try:
        import transformers  # noqa: F401
    except ImportError:
        return "transformers is not installed"
    return ""


def _compat():
    """The bundled modeling file was written against an older transformers: two helpers it imports have since moved."""
    import transformers.pytorch_utils as pu
    import transformers.utils as U
    import transformers.utils.import_utils as iu
    if not hasattr(iu, "is_torch_fx_available"):
        iu.is_torch_fx_available = lambda: False
    if not hasattr(U, "is_torch_fx_available"):
        U.is_torch_fx_available = iu.is_torch_fx_available
    if not hasattr(pu, "is_torch_greater_or_equal_than_1_13"):
        pu.is_torch_greater_or_equal_than_1_13 = True


def build_model(m, seed: int, device: str = "cpu", dtype=None, attn_impl: str = "eager"):
    """HF ``MiniCPMForCausalLM`` with the geometry and muP constants of ``m`` (a ``ModelConfig``), random weights."""
    import torch
    cache = os.environ.setdefault("HF_MODULES_CACHE", os.path.join(ROOT, ".artifacts", "hf_modules"))
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    _compat()
    # transformers reads the cache location once, at import; if it was imported before this call the constants still point
    # at the user's home directory, so they are re-pointed here: the copied modeling files stay inside this repository
    import transformers.dynamic_module_utils as _dmu
    import transformers.utils.hub as _hub
    for mod in (_dmu, _hub):
        if getattr(mod, "HF_MODULES_CACHE", cache) != cache:
            mod.HF_MODULES_CACHE = cache
    from transformers import AutoConfig, AutoModelForCausalLM
    sys.path.insert(0, ROOT)
    from forge_train_harness_b200.ckpt.hf_names import hf_config_overrides
    if m.head_dim * m.num_attention_heads != m.hidden_size:
        raise ValueError("the HF modeling code derives head_dim = hidden_size / num_attention_heads")
    if m.qk_norm or not m.use_mup:
        raise ValueError("the bundled HF model is MiniCPM (muP, no q/k-norm)")
    config = AutoConfig.from_pretrained(HF_DIR, trust_remote_code=True)
    for k, v in hf_config_overrides(m).items():
        setattr(config, k, v)
    # no padding row: with a pad id the embedding module zero-initialises that row and freezes it, and a synthetic corpus
    # uses every id as an ordinary token (an all-zero row also sends 1/sqrt(eps) through the first RMSNorm's gradient)
    config.pad_token_id = None
    torch.manual_seed(seed)
    model = AutoModelForCausalLM.from_config(config, trust_remote_code=True, attn_implementation=attn_impl)
    model = model.to(device=device, dtype=dtype or torch.float32)
    model.train()
    return model, config


def lr_at(step: int, lr: float, min_lr: float, warmup: int, decay_iters: int) -> float:
    if warmup > 0 and step <= warmup:
        return lr * step / warmup
    if decay_iters <= warmup:
        return lr
    t = min(1.0, (step - warmup) / max(1, decay_iters - warmup))
    return min_lr + (lr - min_lr) * 0.5 * (1.0 + math.cos(math.pi * t))


def make_optimizer(model, lr: float, weight_decay: float, betas, width_mult: float, mup_lr: bool = True):
    """fp32 masters grouped by (lr scale, weight decay).  Returns (optimizer, per-group lr scales, [(param, master)])."""
    import torch
    groups, pairs = {}, []
    for name, p in model.named_parameters():
        matrix = p.dim() >= 2
        in_block = matrix and not any(s in name.lower() for s in ("embed", "lm_head", "norm"))
        scale = 1.0 / width_mult if (mup_lr and in_block) else 1.0
        master = p.detach().float().clone().requires_grad_(True)
        pairs.append((p, master))
        groups.setdefault((scale, weight_decay if matrix else 0.0), []).append(master)
    spec = [{"params": ps, "lr": lr * s, "weight_decay": wd} for (s, wd), ps in groups.items()]
    opt = torch.optim.AdamW(spec, betas=betas, eps=1e-8)
    return opt, [s for (s, _wd) in groups], pairs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="minicpm4_8b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--vocab", type=int, default=0)
    ap.add_argument("--hidden", type=int, default=0, help="shrink the width (tests); heads / ffn shrink with it")
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--mbs", type=int, default=1)
    ap.add_argument("--accum", type=int, default=8)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--min-lr", type=float, default=0.0)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--decay-iters", type=int, default=0)
    ap.add_argument("--weight-decay", type=float, default=0.1)
    ap.add_argument("--clip-grad", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--data-prefix", required=True)
    ap.add_argument("--ckpt-root", default="", help="write canonical_state_fp32.pt (engine parameter names) here")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--attn-impl", default="eager", choices=["eager", "sdpa", "flash_attention_2"])
    ap.add_argument("--no-mup-lr", dest="mup_lr", action="store_false", default=True)
    a = ap.parse_args(argv)
    why = available()
    if why:
        print(f"hf_oracle: unavailable: {why}", file=sys.stderr)
        return 3
    import torch
    sys.path.insert(0, ROOT)
    from forge_train_harness_b200.ckpt.hf_names import hf_to_engine
    from forge_train_harness_b200.config.schema import preset
    from forge_train_harness_b200.data.sources import MegatronBinary
    from forge_train_harness_b200.utils import wire

    m = dataclasses.replace(preset(a.model), num_layers=a.layers, mtp_num_layers=0, mtp_loss_weight=0.0, tie_embeddings=False)
    if a.hidden:
        heads = max(2, a.hidden // m.head_dim)
        m = dataclasses.replace(m, hidden_size=heads * m.head_dim, num_attention_heads=heads, num_query_groups=2, ffn_hidden_size=2 * a.hidden)
    if a.seq:
        m = dataclasses.replace(m, seq_length=a.seq, max_position_embeddings=a.seq)
    if a.vocab:
        m = dataclasses.replace(m, padded_vocab_size=a.vocab)
    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    model, config = build_model(m, a.seed, a.device, dt, a.attn_impl)
    width_mult = m.hidden_size / m.mup_base_hidden_size
    if a.ckpt_root:
        os.makedirs(a.ckpt_root, exist_ok=True)
        sd = {k: v.detach().float().cpu() for k, v in model.state_dict().items()}
        torch.save(hf_to_engine(sd, m), os.path.join(a.ckpt_root, "canonical_state_fp32.pt"))
    opt, scales, pairs = make_optimizer(model, a.lr, a.weight_decay, (0.9, 0.95), width_mult, a.mup_lr)
    acc = [torch.zeros_like(ms) for _, ms in pairs]
    src = MegatronBinary(a.data_prefix, m.seq_length, a.mbs, 0, 1, a.seed)
    print(f"=== HF MiniCPM single-card oracle: layers={m.num_layers} hidden={m.hidden_size} vocab={m.padded_vocab_size} "
          f"width_mult={width_mult:g} mbs={a.mbs} accum={a.accum} dtype={a.dtype} ===", flush=True)
    S = m.seq_length
    for step in range(1, a.steps + 1):
        t0 = time.time()
        lr = lr_at(step, a.lr, a.min_lr, a.warmup, a.decay_iters)
        for g, s in zip(opt.param_groups, scales):
            g["lr"] = lr * s
        for b in acc:
            b.zero_()
        nll_sum, n_tok = 0.0, 0.0
        batches = [next(src) for _ in range(a.accum)]
        total_tok = float(sum(b["loss_mask"].sum() for b in batches))
        for b in batches:
            ids = b["tokens"].view(a.mbs, S).long().to(a.device)
            labels = b["labels"].reshape(-1).long().to(a.device)
            mask = b["loss_mask"].reshape(-1).float().to(a.device)
            logits = model(input_ids=ids).logits
            nll = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels, reduction="none")
            s_ = (nll * mask).sum()
            (s_ / total_tok).backward()
            nll_sum += float(s_.detach())
            n_tok += float(mask.sum())
            with torch.no_grad():
                for (p, _ms), buf in zip(pairs, acc):
                    if p.grad is not None:
                        buf.add_(p.grad.float())
                        p.grad = None
        for (_p, ms), buf in zip(pairs, acc):
            ms.grad = buf
        gn = float(torch.nn.utils.clip_grad_norm_([ms for _, ms in pairs], a.clip_grad))
        opt.step()
        with torch.no_grad():
            for p, ms in pairs:
                p.copy_(ms)
        if a.device.startswith("cuda"):
            torch.cuda.synchronize()
        dts = time.time() - t0
        loss = nll_sum / max(n_tok, 1.0)
        print(f"step {step:5d} | loss {loss:.6f} | lr {lr:.6e} | grad_norm {gn:.4f} | tok/s {a.mbs * a.accum * S / dts:8.1f}", flush=True)
        print(wire.format_loss_line(step, loss, gn, dts, 0.0), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
