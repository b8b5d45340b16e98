"""Headline benchmark: MiniCPM4-0.5B-shaped pre-training step, data parallel with the distributed optimizer.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 3 --warmup 3

Config (weak scaling: per-GPU work fixed): 24 layers, hidden 1024, 16 q / 2 kv heads of 64, SwiGLU 4096, vocab 73448,
tied embeddings, seq 4096, micro-batch 4, 16 micro-batches per GPU per step (global batch 64 x N sequences = 512 at
N = 8), bf16 compute with fp32 master weights and AdamW state sharded over the DP group, synthetic seeded tokens,
random-init weights.  One line of JSON is printed by rank 0: ``value`` is whole-job tokens/s over exactly K steps, timed
on the device with CUDA events between barrier + synchronize brackets, max over ranks; ``e2e`` is the same steps timed
by the host clock through the public ``Trainer.train_step`` call including every micro-batch's pinned-memory H2D copy
and a D2H read of the loss and gradient norm every step.  ``--impl reference`` runs the unmodified reference engine from
``baseline/_ref`` on the same shape (see ``baseline/reference_arm.py``).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.rows, self.proc, self.thread = gpu_index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()  # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2])); pw.append(float(r[3]))
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        busy = [s for s, p in zip(sm, pw) if p > 300] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


def baseline_number():
    """Published reference figure to compare against: none exists for B200 (the reference's numbers are H100 MFU)."""
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            pub = json.load(f).get("published", {})
        return pub.get("tokens_per_sec") if pub else None
    except OSError:
        return None


def run_ours(a):
    import torch
    import torch.distributed as dist

    import forge_train_harness_b200 as fth
    from forge_train_harness_b200.engine import _max_over_ranks
    from forge_train_harness_b200.ops.cuda_ops import _C, check_status
    from forge_train_harness_b200.parallel.topology import init_distributed

    init_distributed()
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE is {world}"
    model = fth.preset(a.model)
    cfg = fth.RunConfig(
        model=model,
        optim=fth.OptimConfig(lr=1e-2, min_lr=1e-3, lr_warmup_iters=100, lr_decay_iters=2000, lr_schedule="cosine",
                              weight_decay=0.1, adam_beta1=0.9, adam_beta2=0.95, clip_grad=1.0),
        parallel=fth.ParallelConfig(use_distributed_optimizer=True, ddp_bucket_elems=40_000_000),
        train=fth.TrainConfig(num_steps=a.steps, micro_batch_size=a.mbs, grad_accum_steps=a.accum, seed=1234, dtype="bf16",
                              cuda_graph=not a.no_graph),
        data=fth.DataConfig(data_loader="synthetic", prefetch_size=16))
    tr = fth.Trainer(cfg, device=f"cuda:{local}", init_mode="device", quiet=rank != 0)
    tokens_per_step = a.mbs * model.seq_length * a.accum * world

    def launches():
        return _C.launch_count() + tr.graph_replays * tr.graph_launches

    for _ in range(a.warmup):
        tr.train_step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    def bracket():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed region: exactly K steps -------------------------------------------------
    bracket()
    n0 = launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        res = tr.train_step()
    e1.record()
    bracket()
    dt = _max_over_ranks(e0.elapsed_time(e1) / 1e3, tr.device)
    n_launch = launches() - n0
    loss = float(res["loss"])
    # ---- end-to-end region: host clock, loss read back every step ---------------------------------
    bracket()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        res = tr.train_step()
        loss = float(res["loss"])          # D2H 8 bytes
        gnorm = float(res["grad_norm"])    # D2H 4 bytes
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    dt_e2e = _max_over_ranks(t1 - t0, tr.device)
    bracket()
    clocks = sampler.stop() if rank == 0 else None
    check_status()
    paths = tr.paths()   # which of the fused peer-memory paths / the CUDA graph actually ran
    tr.close()
    if rank == 0:
        value = tokens_per_step * a.steps / dt
        peaks = tr.peaks
        base = baseline_number()
        out = {
            "metric": "tokens/sec (whole job; per-GPU and MFU in extras)", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": dt / a.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": (value / base) if base else None,
            "dtype": "bf16", "data": "synthetic seeded uniform tokens, random-init weights", "impl": "ours",
            "config": {"model": a.model, "global_batch": a.mbs * a.accum * world, "seq_len": model.seq_length,
                       "micro_batch": a.mbs, "grad_accum": a.accum,
                       "parallelism": f"dp{world}" + ("+zero1" if world > 1 else ""),
                       "l2": "no explicit flush: every step streams tens of GB of activations/weights/grads, far above the 126 MB L2",
                       "cuda_graph": tr._graph is not None, "paths": paths},
            "tokens_per_sec_per_gpu": value / world,
            "mfu_percent_of_measured_sustained_bf16": 100.0 * tr.flops_per_token * value / (world * peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) * 1e12),
            "peaks_source": peaks.get("source"), "final_loss": loss, "grad_norm": gnorm,
            "clocks": clocks,
            "e2e": {"value": tokens_per_step * a.steps / dt_e2e, "unit": "tokens/s",
                    "h2d_bytes_per_step": tr.stager.nbytes * a.accum * world, "d2h_bytes_per_step": 12 * world},
            "gpu_launches": int(n_launch),
        }
        print(json.dumps(out), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="minicpm4_0.5b")
    ap.add_argument("--mbs", type=int, default=4)
    ap.add_argument("--accum", type=int, default=16)
    ap.add_argument("--no-graph", action="store_true")
    a = ap.parse_args()
    if a.warmup < 3:
        a.warmup = 3
    if a.impl == "reference":
        from baseline.reference_arm import run_reference
        run_reference(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
