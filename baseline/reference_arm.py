"""Reference arm of ``bench.py``: the UNMODIFIED reference engine on the benchmark's model shape.

What runs: ``training_engine_tensor.run_training_loop(TrainLoopConfig(...))`` — the reference's only public training
contract (workload/src/training_engine_tensor/__init__.py:18-20) — imported from ``baseline/_ref`` (a
``pip install --no-deps --target`` of the reference plus verbatim copies of its ``workload/src/training_engine_tensor``
and ``ref`` trees, which the reference's own packaging leaves out).  Nothing from this repository's engine, models or
kernels is on that path: this module only prepares the inputs the reference reads from its environment — the geometry
variables (config.py:16-25), a rendered product TOML (runtime_config.py:84-139), a data TOML selecting its Megatron
binary reader (train_loop.py:192-229) and a synthetic ``.bin/.idx`` corpus of seeded uniform tokens — with the
perf switches of its published configuration (workload/src/config/long-train.toml:53-79: Triton fusions on, CUDA graph
on, prefetch on, determinism off).  The reference engine has no tied-embedding mode and no distributed optimizer that
works (zero_optimizer.py, "known hang"), so its arm runs untied weights with replicated AdamW and a flat fp32 gradient
all-reduce; FLOPs per token are identical.

Timing: the reference prints one ``[LOSS]`` line per step with ``time_s`` measured by its own CUDA events around the
step (train_loop.py:2136, 2496-2498).  ``value`` sums ``time_s`` over the last K steps (device time); ``e2e`` is the
host clock between the arrival of the line that ends warm-up and the line that ends step W+K, which includes its
per-micro-batch pinned H2D copies and its per-step loss read.
"""
from __future__ import annotations

import io
import json
import os
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


class _Tee(io.TextIOBase):
    def __init__(self, inner):
        self.inner, self.lines, self._buf = inner, [], ""

    def write(self, s):
        self._buf += s
        while "\n" in self._buf:
            line, self._buf = self._buf.split("\n", 1)
            self.lines.append((time.perf_counter(), line))
        return len(s)

    def flush(self):
        pass


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def run_reference(a) -> None:
    if not os.path.isdir(os.path.join(REF, "training_engine_tensor")):
        return _unavailable("baseline/_ref is not installed (pip install --no-deps --target baseline/_ref of the reference)")
    try:
        import numpy as np
        import torch
        if not torch.cuda.is_available():
            return _unavailable("no CUDA device")
        import flash_attn  # noqa: F401  (library the reference's attention calls)
        import triton  # noqa: F401
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"missing dependency of the reference engine: {type(e).__name__}: {e}")

    sys.path.insert(0, os.path.dirname(HERE))
    from forge_train_harness_b200.config.schema import preset  # shape constants only
    from forge_train_harness_b200.data.sources import write_megatron_binary  # writes the reference's input format
    m = preset(a.model)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    steps = a.warmup + a.steps
    tmp = tempfile.mkdtemp(prefix=f"refarm_r{rank}_")
    rng = np.random.RandomState(0)
    n_windows = steps * a.accum * a.mbs * world + 64
    docs = [rng.randint(0, m.padded_vocab_size, size=(m.seq_length + 1) * 64).astype(np.int32) for _ in range((n_windows + 63) // 64)]
    write_megatron_binary(os.path.join(tmp, "synthetic"), docs, np.int32)
    with open(os.path.join(tmp, "data.toml"), "w") as f:
        f.write('[data]\ndata_loader = "megatron_binary"\n')
    cli = {"num_layers": m.num_layers, "hidden_size": m.hidden_size, "ffn_hidden_size": m.ffn_hidden_size,
           "num_attention_heads": m.num_attention_heads, "num_query_groups": m.num_query_groups, "head_dim": m.head_dim,
           "seq_length": m.seq_length, "max_position_embeddings": m.seq_length, "padded_vocab_size": m.padded_vocab_size,
           "rotary_base": int(m.rotary_base), "norm_epsilon": m.norm_epsilon, "init_method_std": m.init_method_std,
           "mup_base_hidden_size": m.mup_base_hidden_size, "mup_emb_scale": m.mup_emb_scale,
           "mup_depth_scale": m.mup_depth_scale, "mtp_num_layers": 0, "mtp_loss_weight": 0.0,
           "lr": 1e-2, "min_lr": 1e-3, "lr_warmup_iters": 100, "lr_decay_iters": 2000, "lr_wsd_decay_iters": 0,
           "weight_decay": 0.1, "adam_beta1": 0.9, "adam_beta2": 0.95, "clip_grad": 1.0}
    with open(os.path.join(tmp, "bench.toml"), "w") as f:
        f.write("[cli]\n" + "".join(f"{k} = {v!r}\n" for k, v in cli.items()))
    env = {k.upper(): str(v) for k, v in cli.items()}
    env.update(FORGE_GATE="bench", FORGE_OURS_CONFIG_DIR=tmp, FORGE_DATA_TOML=os.path.join(tmp, "data.toml"),
               DETERMINISTIC="0", FORGE_INIT_ONES="1", ENABLE_CUDA_GRAPH="1", ENABLE_DL_PREFETCH="1", DL_PREFETCH_SIZE="128",
               ENABLE_TRITON_SWIGLU_FWD="1", ENABLE_TRITON_SWIGLU_BWD="1", ENABLE_TRITON_RMSNORM_FWD="1",
               ENABLE_TRITON_RMSNORM_BWD="1", ENABLE_TRITON_ROPE_FWD="1", ENABLE_TRITON_ROPE_BWD="1", ENABLE_TRITON_CE_BWD="1",
               ENABLE_ZERO_OPTIMIZER="0", CUDA_DEVICE_MAX_CONNECTIONS="8")
    os.environ.update(env)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    sys.path.insert(0, REF)
    # the reference's trainer imports its model file as a sibling module (it is normally run as a script)
    sys.path.insert(1, os.path.join(REF, "ref", "reference"))
    try:
        from training_engine_tensor import TrainLoopConfig, run_training_loop
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"reference engine import failed: {type(e).__name__}: {e}")
    cfg = TrainLoopConfig(num_steps=steps, micro_batch_size=a.mbs, seq_length=m.seq_length, grad_accum_steps=a.accum,
                          seed=1234, world_size=world, checkpoint_root=os.path.join(tmp, "no_canonical_state"),
                          data_path=os.path.join(tmp, "synthetic"), lr=1e-2, min_lr=1e-3, lr_warmup_iters=100,
                          lr_decay_iters=2000, lr_wsd_decay_iters=0, teardown_exit=False)
    tee = _Tee(sys.stdout)
    real = sys.stdout
    stack, engine_error = "engine (training_engine_tensor.run_training_loop)", None
    sys.stdout = tee
    try:
        run_training_loop(cfg)
    except BaseException as e:  # noqa: BLE001
        import traceback
        traceback.print_exc(file=sys.stderr)
        engine_error = f"{type(e).__name__}: {str(e)[:160]}"
    finally:
        sys.stdout = real
    if engine_error is not None:
        # The reference's produced engine does not run on this torch build; fall back to the reference's own live
        # baseline, its pure-PyTorch L0 trainer (ref/reference/train_pure_mup_mtp.py), which every one of its gates
        # compares against.  Same shape, same data file, stock code path (its argparse main()).
        import gc

        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()
        gc.collect()
        torch.cuda.empty_cache()
        stack = "L0 pure-torch trainer (ref/reference/train_pure_mup_mtp.py main)"
        with open(os.path.join(tmp, "data_path.txt"), "w") as f:
            f.write(f"1.0 {os.path.join(tmp, 'synthetic')}\n")
        argv = ["train_pure_mup_mtp.py", "--data-path-file", os.path.join(tmp, "data_path.txt"), "--data-config",
                os.path.join(tmp, "data.toml"), "--train-iters", str(steps), "--micro-batch-size", str(a.mbs),
                "--global-batch-size", str(a.mbs * a.accum * world), "--lr", "1e-2", "--min-lr", "1e-3", "--lr-warmup-iters", "100",
                "--lr-decay-iters", "2000", "--weight-decay", "0.1", "--adam-beta1", "0.9", "--adam-beta2", "0.95",
                "--clip-grad", "1.0", "--seed", "1234", "--init-method-std", str(m.init_method_std), "--init-ones", "1",
                "--eagle-num-layers", "0", "--out-dir", os.path.join(tmp, "out"), "--no-deterministic"]
        tee = _Tee(sys.stdout)
        sys.stdout = tee
        old_argv = sys.argv
        sys.argv = argv
        try:
            import train_pure_mup_mtp
            train_pure_mup_mtp.main()
        except SystemExit:
            pass
        except BaseException as e:  # noqa: BLE001
            import traceback
            sys.stdout = real
            traceback.print_exc(file=sys.stderr)
            return _unavailable(f"reference engine raised {engine_error}; its L0 trainer raised {type(e).__name__}: {str(e)[:160]}")
        finally:
            sys.stdout = real
            sys.argv = old_argv
    if rank != 0:
        return
    recs = []
    for ts, line in tee.lines:
        if line.startswith("[LOSS]"):
            kv = dict(p.split("=", 1) for p in line.split()[1:] if "=" in p)
            recs.append((ts, float(kv["time_s"]), float(kv["global_loss"])))
    if len(recs) < steps:
        return _unavailable(f"reference printed {len(recs)} [LOSS] lines, expected {steps}")
    timed = recs[a.warmup:]
    tokens_per_step = a.mbs * m.seq_length * a.accum * world
    dt_dev = sum(r[1] for r in timed)
    dt_e2e = timed[-1][0] - recs[a.warmup - 1][0]
    value = tokens_per_step * a.steps / dt_dev
    from forge_train_harness_b200.utils.peaks import load_peaks
    peaks = load_peaks()
    out = {"metric": "tokens/sec (whole job; per-GPU and MFU in extras)", "value": value, "unit": "tokens/s", "n_gpus": world,
           "steps": a.steps, "warmup": a.warmup, "ms_per_step": dt_dev / a.steps * 1e3, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic seeded uniform tokens, random-init weights",
           "impl": "reference", "reference_stack": stack, "engine_error": engine_error,
           "config": {"model": a.model, "global_batch": a.mbs * a.accum * world, "seq_len": m.seq_length, "micro_batch": a.mbs,
                      "grad_accum": a.accum, "parallelism": f"dp{world}",
                      "note": "reference engine: untied embeddings, replicated AdamW, flat fp32 all-reduce, Triton + flash-attn 2 + cuBLAS, CUDA graph"},
           "tokens_per_sec_per_gpu": value / world,
           "mfu_percent_of_measured_sustained_bf16": 100.0 * m.flops_per_token(False) * value / (world * peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) * 1e12),
           "final_loss": timed[-1][2],
           "e2e": {"value": tokens_per_step * a.steps / dt_e2e, "unit": "tokens/s",
                   "h2d_bytes_per_step": 40 * a.mbs * m.seq_length * a.accum * world, "d2h_bytes_per_step": 16 * world},
           "timing": "device: sum of the reference's own per-step CUDA-event time_s on rank 0; e2e: host clock between [LOSS] lines"}
    print(json.dumps(out), flush=True)
