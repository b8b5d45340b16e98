"""Device-timed benchmark of the fused compute+collective kernels against library collectives, with roofline fractions.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 -m forge_train_harness_b200.utils.commbench \
        [--model minicpm4_8b] [--mbs 1] [--json out.json]

For every path the time is CUDA events around ``iters`` back-to-back calls after warm-up, max over ranks.  Roofline of a
fused call = max(FLOPs / measured bf16 peak, bytes that must cross NVLink per GPU / 770 GB/s measured peer-copy bandwidth).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..config.schema import preset
from ..parallel.topology import init_distributed
from .peaks import load_peaks

NVLINK_GBS = 770.0


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    e1.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e-3], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="minicpm4_8b")
    ap.add_argument("--mbs", type=int, default=1)
    ap.add_argument("--json", default="")
    ap.add_argument("--skip-dp", action="store_true", help="time only the tensor-parallel paths")
    ap.add_argument("--n-copy", type=int, default=0, help="copy CTAs of the all-gather kernel (0 = its default)")
    a = ap.parse_args(argv)
    init_distributed()
    rank, tp = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    from ..ops.cuda_ops import Sm100Ops as ops, check_status
    from ..parallel import fused_dp, fused_tp
    from ..parallel.tp import TPComm
    cfg = preset(a.model)
    peaks = load_peaks()
    M, H, F = a.mbs * cfg.seq_length, cfg.hidden_size, cfg.ffn_hidden_size
    Ms = M // tp
    group = dist.group.WORLD
    f = fused_tp.try_create(group, tp, rank, M, H, dev, required=True)
    f.n_copy = a.n_copy
    nccl = TPComm(group, tp, rank, True)
    r = lambda *s: torch.randn(*s, device=dev, dtype=torch.float32).mul_(0.3).to(torch.bfloat16)
    rows = []

    def rec(name, t_fused, t_lib, flops, link_bytes, t_gemm=None):
        roof = max(flops / (peaks["bf16_tflops"] * 1e12), link_bytes / (NVLINK_GBS * 1e9))
        row = {"path": name, "tp": tp, "fused_ms": t_fused * 1e3, "library_ms": t_lib * 1e3, "speedup_vs_library": t_lib / t_fused,
               "gemm_alone_ms": None if t_gemm is None else t_gemm * 1e3,
               "roofline_ms": roof * 1e3, "achieved_fraction_of_roofline": roof / t_fused,
               "bound": "compute" if flops / (peaks["bf16_tflops"] * 1e12) >= link_bytes / (NVLINK_GBS * 1e9) else "nvlink"}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    link = (tp - 1) / tp * M * H * 2.0
    for name, N in (("ag_gemm_qkv", cfg.qkv_dim // tp if tp <= cfg.num_query_groups else (cfg.q_per_kv // (tp // cfg.num_query_groups) + 2) * cfg.head_dim),
                    ("ag_gemm_fc1", 2 * F // tp)):
        x, w = r(Ms, H), r(N, H)
        tf = timed(lambda: f.ag_gemm(x, w, False))
        tl = timed(lambda: ops.linear_fwd(nccl.gather_rows(x), w))
        xf = r(M, H)
        rec(name, tf, tl, 2.0 * M * N * H, link, timed(lambda: ops.linear_fwd(xf, w)))
    for name, K in (("gemm_rs_wo", cfg.q_dim // tp), ("gemm_rs_fc2", F // tp)):
        x, w = r(M, K), r(H, K)
        tf = timed(lambda: f.gemm_rs(x, w, False))
        tl = timed(lambda: nccl.reduce_scatter_rows(ops.linear_fwd(x, w)))
        rec(name, tf, tl, 2.0 * M * H * K, link, timed(lambda: ops.linear_fwd(x, w)))
    if a.skip_dp:
        torch.cuda.synchronize()
        check_status()
        if a.json and rank == 0:
            with open(a.json, "w") as fh:
                json.dump({"peaks": peaks, "nvlink_gbs": NVLINK_GBS, "model": a.model, "mbs": a.mbs, "rows": rows}, fh, indent=1)
        dist.barrier()
        dist.destroy_process_group()
        return
    # DP gradient path on a 1 G-element (fp32) buffer: pull reduce-scatter + sumsq, then AdamW with parameter push
    n = 256 * 1024 * 1024

    from types import SimpleNamespace as NS
    st = NS(numel=n, dtype=torch.bfloat16, device=dev, flat_param=torch.zeros(n, dtype=torch.bfloat16, device=dev), flat_grad=None)

    def _rebind(p, g):
        st.flat_param, st.flat_grad = p, g
    st.rebind = _rebind
    fd = fused_dp.FusedDP(st, NS(dp_group=group, dp=tp, rank=rank))
    st.flat_grad.normal_()
    per = n // tp
    opt = NS(my_ranges=[(rank * per, (rank + 1) * per, 0)], dup_ranges=[], segs=[(0, rank * per, per, 1.0, True)],
             master=torch.zeros(per, device=dev), m=torch.zeros(per, device=dev), v=torch.zeros(per, device=dev), step_count=1,
             oc=NS(adam_beta1=0.9, adam_beta2=0.95, adam_eps=1e-8, weight_decay=0.1), ops=ops)
    one = torch.ones((), device=dev)
    t_rs = timed(lambda: fd.reduce_scatter_sumsq(opt), iters=5)
    shard = torch.empty(per, device=dev)
    t_rs_lib = timed(lambda: (dist.reduce_scatter_tensor(shard, st.flat_grad), ops.sumsq(shard)), iters=5)
    t_ad = timed(lambda: fd.adam_allgather(opt, 1e-3, one), iters=5)
    table = None

    def lib_adam():
        nonlocal table
        table = ops.adamw_segments(opt.master, opt.m, opt.v, st.flat_grad, st.flat_param, opt.segs, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, one, table)
        dist.all_gather_into_tensor(st.flat_param, st.flat_param[rank * per:(rank + 1) * per])
    t_ad_lib = timed(lib_adam, iters=5)
    rec("dp_reduce_scatter_sumsq_1GiB_fp32", t_rs, t_rs_lib, 0.0, (tp - 1) / tp * n * 4.0)
    rec("dp_adamw_param_push_256Mi", t_ad, t_ad_lib, 0.0, (tp - 1) / tp * n * 2.0)
    torch.cuda.synchronize()
    check_status()
    if a.json and rank == 0:
        with open(a.json, "w") as fh:
            json.dump({"peaks": peaks, "nvlink_gbs": NVLINK_GBS, "model": a.model, "mbs": a.mbs, "rows": rows}, fh, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
