"""Run ONE sm_100a op a few times on a small, fixed case — the program that profiler captures are taken of.

    python -m forge_train_harness_b200.utils.profile_case --op flash_bwd [--iters 3]

Cases (a few hundred MB on the device at most, GEMM operands larger than the 126 MB L2):
  gemm_fwd / gemm_dgrad / gemm_wgrad   the FC1 shape of the 0.5B model at 16384 tokens (M 16384, N 8192, K 1024)
  gemm_mxfp8                            the FC1 shape of the 8B model at 4096 tokens (M 4096, N 8192 = one TP-4 shard, K 4096), e4m3 + e8m0
  mxfp8_quant_row / mxfp8_quant_col     quantisation of a 16384 x 4096 bf16 activation
  flash_fwd / flash_bwd                 1 x 4096 tokens, 16 query / 2 KV heads of 64
  rmsnorm_fwd / rmsnorm_bwd / swiglu_fwd / swiglu_bwd / rope / cross_entropy    the 0.5B shapes at 16384 (CE: 4096) tokens
  rmsnorm_plain / embedding_fwd / embedding_bwd / adamw                          the same shapes; AdamW on 64 Mi parameters
  microbatch                            engine steps of the 0.5B shape cut to 2 layers: one micro-batch of 4 x 4096 tokens per
                                        step, no CUDA graph, so that a launch list shows every kernel of a layer and of the head
"""
from __future__ import annotations

import argparse

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args(argv)
    from ..ops.cuda_ops import Sm100Ops as ops, _C, check_status
    from ..ops.torch_ops import rope_table
    dev = "cuda"
    r = lambda *s: torch.randn(*s, device=dev, dtype=torch.float32).mul_(0.5).to(torch.bfloat16)
    M, H, F, V, S, d, nkv, g = 16384, 1024, 4096, 73448, 4096, 64, 2, 8
    if a.op in ("gemm_fwd", "gemm_dgrad", "gemm_wgrad"):
        x, w, dy = r(M, H), r(2 * F, H), r(M, 2 * F)
        mg = torch.zeros(2 * F, H, device=dev)
        fn = {"gemm_fwd": lambda: _C.gemm(x, False, w, False, None, 1.0, 0, 0, 0),
              "gemm_dgrad": lambda: _C.gemm(dy, False, w, True, None, 1.0, 0, 0, 0),
              "gemm_wgrad": lambda: _C.gemm(dy, True, x, True, mg, 1.0, 1, 0, 0)}[a.op]
    elif a.op.startswith("gemm_mxfp8") or a.op.startswith("mxfp8_quant"):
        from ..ops import mxfp8 as mx
        if a.op == "gemm_mxfp8":
            x, w = r(4096, 4096), r(8192, 4096)
            xq, xs = mx.quantize(x)
            wq, ws = mx.quantize(w)
            fn = lambda: mx.gemm(xq, xs, wq, ws, None, 1.0, 0)
        else:
            x = r(M, 4096)
            fn = lambda: mx.quantize(x, a.op.endswith("col"))
    elif a.op in ("flash_fwd", "flash_bwd"):
        qkv = r(S, nkv * (g + 2) * d)
        out, lse = ops.attention_fwd(qkv, S, nkv, g, d)
        do = r(S, nkv * g * d)
        fn = (lambda: ops.attention_fwd(qkv, S, nkv, g, d)) if a.op == "flash_fwd" else \
             (lambda: ops.attention_bwd(do, qkv, out, lse, S, nkv, g, d))
    elif a.op in ("rmsnorm_fwd", "rmsnorm_bwd"):
        x, res, w = r(M, H), r(M, H), r(H)
        _, rstd = ops.rmsnorm_fwd(x, w, 1e-6)
        gw = torch.zeros(H, device=dev)
        fn = (lambda: ops.residual_rmsnorm_fwd(x, res, 0.3, w, 1e-6)) if a.op == "rmsnorm_fwd" else \
             (lambda: ops.rmsnorm_bwd(res, x, w, rstd, gw, res))
    elif a.op == "rmsnorm_plain":
        x, w = r(M, H), r(H)
        fn = lambda: ops.rmsnorm_fwd(x, w, 1e-6)
    elif a.op in ("embedding_fwd", "embedding_bwd"):
        ids = torch.randint(0, V, (M,), device=dev, dtype=torch.int32)
        w, dout = r(V, H), r(M, H)
        mg = torch.zeros(V, H, device=dev)
        fn = (lambda: ops.embedding_fwd(ids, w, 12.0)) if a.op == "embedding_fwd" else \
             (lambda: ops.embedding_bwd(dout, ids, mg, 12.0))
    elif a.op == "adamw":
        n = 64 * 1024 * 1024
        master, m_, v_, grad = (torch.randn(n, device=dev) for _ in range(4))
        v_.abs_()
        param = torch.empty(n, device=dev, dtype=torch.bfloat16)
        one = torch.ones((), device=dev)
        table = ops.build_adam_table([(0, 0, n, 1.0, True)], dev)
        fn = lambda: ops.adamw_segments(master, m_, v_, grad, param, None, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3, one, table)
    elif a.op in ("swiglu_fwd", "swiglu_bwd"):
        gu, di = r(M, 2 * F), r(M, F)
        fn = (lambda: ops.swiglu_fwd(gu)) if a.op == "swiglu_fwd" else (lambda: ops.swiglu_bwd(di, gu))
    elif a.op == "rope":
        qkv, tab = r(M, nkv * (g + 2) * d), rope_table(S, d, 10000.0, dev)
        fn = lambda: ops.rope_fwd_(qkv, tab, S, nkv, g, d)
    elif a.op == "cross_entropy":
        lg = r(4096, V)
        lab = torch.randint(0, V, (4096,), device=dev, dtype=torch.int32)
        mk = torch.ones(4096, device=dev)
        fn = lambda: ops.cross_entropy_fwd_bwd(lg, lab, mk)
    elif a.op == "microbatch":
        import dataclasses
        from .. import OptimConfig, RunConfig, TrainConfig, DataConfig, Trainer, preset
        cfg = RunConfig(model=dataclasses.replace(preset("minicpm4_0.5b"), num_layers=2),
                        optim=OptimConfig(lr=1e-3, lr_schedule="constant"),
                        train=TrainConfig(num_steps=a.iters, micro_batch_size=4, global_batch_size=4, seed=1, dtype="bf16",
                                          cuda_graph=False),
                        data=DataConfig(prefetch_size=0))
        tr = Trainer(cfg, quiet=True)
        fn = tr.train_step
    else:
        raise SystemExit(f"unknown op {a.op}")
    for _ in range(a.iters):
        fn()
    torch.cuda.synchronize()
    check_status()
    print(f"{a.op}: ok")


if __name__ == "__main__":
    main()
