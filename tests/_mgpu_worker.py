"""Worker for the multi-GPU tests: trains a small bf16 model for a few steps and prints the losses as JSON on rank 0."""
import dataclasses
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import forge_train_harness_b200 as fth  # noqa: E402
from forge_train_harness_b200.parallel.topology import init_distributed  # noqa: E402


def main():
    mode = sys.argv[1]
    init_distributed()
    par = {"dp_zero": dict(use_distributed_optimizer=True, ddp_bucket_elems=300_000),
           "dp_zero_late": dict(use_distributed_optimizer=True, ddp_bucket_elems=300_000, overlap_grad_reduce=False),
           "dp_plain": dict(use_distributed_optimizer=False),
           "tp_sp": dict(tensor_parallel_size=int(os.environ.get("WORLD_SIZE", "1")), sequence_parallel=True),
           "pp": dict(pipeline_parallel_size=2),
           "tp2dp2": dict(tensor_parallel_size=2, sequence_parallel=True, use_distributed_optimizer=True,
                          ddp_bucket_elems=300_000),
           "pp2dp2": dict(pipeline_parallel_size=2, use_distributed_optimizer=True, ddp_bucket_elems=300_000),
           "tp2pp2": dict(tensor_parallel_size=2, pipeline_parallel_size=2, sequence_parallel=True,
                          use_distributed_optimizer=True),
           "tp2pp2v2": dict(tensor_parallel_size=2, pipeline_parallel_size=2, virtual_pipeline_stages=2,
                            sequence_parallel=True, use_distributed_optimizer=True),
           "single": {}}[mode.split(":")[0]]
    model = dataclasses.replace(fth.preset("tiny"), num_layers=4, seq_length=256, padded_vocab_size=4096, hidden_size=256,
                                ffn_hidden_size=512, num_attention_heads=4, num_query_groups=2, head_dim=64)
    cfg = fth.RunConfig(model=model, optim=fth.OptimConfig(lr=2e-3, lr_schedule="constant"), parallel=fth.ParallelConfig(**par),
                        train=fth.TrainConfig(num_steps=4, micro_batch_size=2, global_batch_size=8, seed=5, dtype="bf16",
                                              cuda_graph=mode.endswith(":graph")),
                        data=fth.DataConfig(prefetch_size=0))
    tr = fth.Trainer(cfg, quiet=True)
    out = []
    for _ in range(4):
        r = tr.train_step()
        out.append([float(r["loss"]), float(r["grad_norm"])])
    torch.cuda.synchronize()
    from forge_train_harness_b200.ops.cuda_ops import check_status
    check_status()
    fused = (tr.opt.fused is not None) or (tr.tpc.fused is not None)
    replays = sum(c.graph_replays for c in tr.chunks)
    tr.close()
    if tr.rank == 0:
        print("RESULT " + json.dumps({"mode": mode, "fused": fused, "steps": out, "graph_replays": replays,
                                      "paths": tr.paths()}), flush=True)
    import torch.distributed as dist
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
