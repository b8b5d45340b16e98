"""Run the UNMODIFIED reference engine (``training_engine_tensor.run_training_loop`` from ``baseline/_ref``) as the
reference side of a gate: a given model shape, a given ``.bin/.idx`` corpus, weights from a ``canonical_state_fp32.pt``.

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 baseline/ref_engine_driver.py --model minicpm4_0.5b \
        --steps 200 --mbs 4 --accum 10 --data-prefix <dir>/corpus --ckpt-root <dir holding canonical_state_fp32.pt> --lr 1e-3

Nothing of this repository's engine runs here: the module writes what the reference reads from its environment (geometry
variables, a rendered ``[cli]`` product, a data TOML naming its Megatron-binary reader; config.py:16-25,
runtime_config.py:84-139, train_loop.py:192-229) and calls its public entry point.  The reference prints its own
``[LOSS]`` lines on rank 0.  Its single-GPU branch does not run on torch 2.11 (``torch._foreach_mul_`` with a 1-element
tensor, train_loop.py:2405); with two or more ranks it does.
"""
from __future__ import annotations

import argparse
import dataclasses
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def reference_env(m, tmp: str, *, lr: float, min_lr: float, warmup: int, decay_iters: int, wsd_decay: int = 0,
                  deterministic: bool = False, cuda_graph: bool = True) -> dict:
    """Environment + product files the reference engine reads for model shape ``m`` (a ``ModelConfig``)."""
    with open(os.path.join(tmp, "data.toml"), "w") as f:
        f.write('[data]\ndata_loader = "megatron_binary"\n')
    cli = {"num_layers": m.num_layers, "hidden_size": m.hidden_size, "ffn_hidden_size": m.ffn_hidden_size,
           "num_attention_heads": m.num_attention_heads, "num_query_groups": m.num_query_groups, "head_dim": m.head_dim,
           "seq_length": m.seq_length, "max_position_embeddings": m.seq_length, "padded_vocab_size": m.padded_vocab_size,
           "rotary_base": int(m.rotary_base), "norm_epsilon": m.norm_epsilon, "init_method_std": m.init_method_std,
           "mup_base_hidden_size": m.mup_base_hidden_size, "mup_emb_scale": m.mup_emb_scale,
           "mup_depth_scale": m.mup_depth_scale, "mtp_num_layers": 0, "mtp_loss_weight": 0.0,
           "lr": lr, "min_lr": min_lr, "lr_warmup_iters": warmup, "lr_decay_iters": decay_iters, "lr_wsd_decay_iters": wsd_decay,
           "weight_decay": 0.1, "adam_beta1": 0.9, "adam_beta2": 0.95, "clip_grad": 1.0}
    with open(os.path.join(tmp, "gate.toml"), "w") as f:
        f.write("[cli]\n" + "".join(f"{k} = {v!r}\n" for k, v in cli.items()))
    env = {k.upper(): str(v) for k, v in cli.items()}
    on = "1"
    env.update(FORGE_GATE="gate", FORGE_OURS_CONFIG_DIR=tmp, FORGE_DATA_TOML=os.path.join(tmp, "data.toml"),
               DETERMINISTIC="1" if deterministic else "0", FORGE_INIT_ONES="1", ENABLE_CUDA_GRAPH=on if cuda_graph else "0",
               ENABLE_DL_PREFETCH="1", DL_PREFETCH_SIZE="128", ENABLE_TRITON_SWIGLU_FWD=on, ENABLE_TRITON_SWIGLU_BWD=on,
               ENABLE_TRITON_RMSNORM_FWD=on, ENABLE_TRITON_RMSNORM_BWD=on, ENABLE_TRITON_ROPE_FWD=on, ENABLE_TRITON_ROPE_BWD=on,
               ENABLE_TRITON_CE_BWD=on, ENABLE_ZERO_OPTIMIZER="0", CUDA_DEVICE_MAX_CONNECTIONS="8")
    return env


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="minicpm4_0.5b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--steps", type=int, required=True)
    ap.add_argument("--mbs", type=int, default=4)
    ap.add_argument("--accum", type=int, default=2)
    ap.add_argument("--data-prefix", required=True)
    ap.add_argument("--ckpt-root", required=True)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--decay-iters", type=int, default=100000)
    ap.add_argument("--seed", type=int, default=1234)
    a = ap.parse_args(argv)
    sys.path.insert(0, os.path.dirname(HERE))
    from forge_train_harness_b200.config.schema import preset  # shape constants only
    m = preset(a.model)
    if a.layers:
        m = dataclasses.replace(m, num_layers=a.layers)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    tmp = tempfile.mkdtemp(prefix=f"refengine_r{os.environ.get('RANK', '0')}_")
    os.environ.update(reference_env(m, tmp, lr=a.lr, min_lr=a.lr * 0.1, warmup=a.warmup, decay_iters=a.decay_iters))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    sys.path.insert(0, REF)
    sys.path.insert(1, os.path.join(REF, "ref", "reference"))
    from training_engine_tensor import TrainLoopConfig, run_training_loop
    cfg = TrainLoopConfig(num_steps=a.steps, micro_batch_size=a.mbs, seq_length=m.seq_length, grad_accum_steps=a.accum,
                          seed=a.seed, world_size=world, checkpoint_root=a.ckpt_root, data_path=a.data_prefix, lr=a.lr,
                          min_lr=a.lr * 0.1, lr_warmup_iters=a.warmup, lr_decay_iters=a.decay_iters, lr_wsd_decay_iters=0,
                          teardown_exit=False)
    run_training_loop(cfg)


if __name__ == "__main__":
    main()
    sys.exit(0)
