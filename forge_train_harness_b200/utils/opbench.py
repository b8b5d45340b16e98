"""Per-op device timing at production shapes, reported against the measured roofline.

``python -m forge_train_harness_b200.utils.opbench [--model minicpm4_0.5b] [--mbs 4]`` times each sm_100a op with
CUDA events (warm-up, L2 flushed between iterations by writing a buffer larger than L2) and prints achieved
TFLOP/s or GB/s and the fraction of the measured peak.  The counterpart of the reference's per-phase CUDA-event
stub (tools/profile_step.py:113-216), but per kernel.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..config.schema import preset
from ..ops.torch_ops import rope_table
from .peaks import load_peaks


def timeit(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.add_(1.0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2] * 1e-3


def timeit_many(fns: dict, iters=10, warmup=3, flush=None) -> dict:
    """Times several implementations of one op INTERLEAVED (a, b, c, a, b, c, ...), so that all of them see the same
    clocks: on a power-capped part whichever variant ran last in a back-to-back sweep measured the hottest GPU."""
    for _ in range(warmup):
        for fn in fns.values():
            fn()
    torch.cuda.synchronize()
    ts = {k: [] for k in fns}
    for _ in range(iters):
        for k, fn in fns.items():
            if flush is not None:
                flush.add_(1.0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts[k].append(e0.elapsed_time(e1))
    return {k: sorted(v)[len(v) // 2] * 1e-3 for k, v in ts.items()}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="minicpm4_0.5b")
    ap.add_argument("--mbs", type=int, default=4)
    ap.add_argument("--only", default="")
    ap.add_argument("--tp", type=int, default=1, help="time the GEMMs at the shapes one tensor-parallel rank sees")
    ap.add_argument("--json", default="")
    a = ap.parse_args(argv)
    from ..ops.cuda_ops import Sm100Ops as ops, _C, check_status
    cfg = preset(a.model)
    peaks = load_peaks()
    pk_f, pk_b = peaks["bf16_tflops"], peaks["hbm_gbs"]
    M, H, F, V, S = a.mbs * cfg.seq_length, cfg.hidden_size, cfg.ffn_hidden_size, cfg.padded_vocab_size, cfg.seq_length
    d, nkv, g = cfg.head_dim, cfg.num_query_groups, cfg.q_per_kv
    dev = "cuda"
    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)
    r = lambda *s: torch.randn(*s, device=dev, dtype=torch.float32).mul_(0.5).to(torch.bfloat16)
    rows = []

    def rec(name, t, flops=0.0, bytes_=0.0):
        row = {"op": name, "ms": t * 1e3}
        if flops:
            row["tflops"] = flops / t / 1e12
            row["frac_of_measured_bf16_peak"] = row["tflops"] / pk_f
        if bytes_:
            row["gbs"] = bytes_ / t / 1e9
            row["frac_of_measured_hbm"] = row["gbs"] / pk_b
        rows.append(row)
        print(json.dumps(row), flush=True)

    def want(n):
        return not a.only or any(k in n for k in a.only.split(","))

    tp = a.tp
    gemms = [("qkv", cfg.qkv_dim // tp, H), ("wo", H, cfg.q_dim // tp), ("fc1", 2 * F // tp, H), ("fc2", H, F // tp),
             ("lm_head", (V + tp - 1) // tp // 8 * 8, H)]
    for name, N, K in gemms:
        if not want("gemm") and not want(name):
            continue
        x, w, dy = r(M, K), r(N, K), r(M, N)
        mg = torch.zeros(N, K, device=dev)
        fl = 2.0 * M * N * K
        # tile codes: one-CTA tiles (128, 256), CTA-pair tiles (-128, -256), the library's own choice (0); cuBLAS beside them
        fns = {}
        for bn in (128, 256, -128, -256, 0):
            fns[f"gemm_fwd_{name}_bn{bn}"] = lambda bn=bn: _C.gemm(x, False, w, False, None, 1.0, 0, bn, 0)
            fns[f"gemm_dgrad_{name}_bn{bn}"] = lambda bn=bn: _C.gemm(dy, False, w, True, None, 1.0, 0, bn, 0)
            fns[f"gemm_wgrad_{name}_bn{bn}"] = lambda bn=bn: _C.gemm(dy, True, x, True, mg, 1.0, 1, bn, 0)
        fns[f"cublas_fwd_{name}"] = lambda: x @ w.t()
        fns[f"cublas_dgrad_{name}"] = lambda: dy @ w
        fns[f"cublas_wgrad_{name}"] = lambda: dy.t() @ x
        for k, t in timeit_many(fns, flush=flush).items():
            rec(k, t, fl)
        del x, w, dy, mg
    if want("mxfp8"):
        from ..ops import mxfp8 as mx
        for name, N, K in gemms[:4]:
            x, w = r(M, K), r(N, K)
            fl = 2.0 * M * N * K
            rec(f"mxfp8_quant_row_{name}_x", timeit(lambda: mx.quantize(x, False), flush=flush), bytes_=3.0 * M * K)
            rec(f"mxfp8_quant_col_{name}_x", timeit(lambda: mx.quantize(x, True), flush=flush), bytes_=3.0 * M * K)
            xq, xs = mx.quantize(x, False)
            wq, ws = mx.quantize(w, False)
            rec(f"mxfp8_gemm_fwd_{name}", timeit(lambda: mx.gemm(xq, xs, wq, ws, None, 1.0, 0), flush=flush), fl)
            rec(f"bf16_gemm_fwd_{name}", timeit(lambda: _C.gemm(x, False, w, False, None, 1.0, 0, 0, 0), flush=flush), fl)
            del x, w, xq, xs, wq, ws
    if want("norm"):
        x, res, w = r(M, H), r(M, H), r(H)
        rec("rmsnorm_fwd", timeit(lambda: ops.rmsnorm_fwd(x, w, 1e-6), flush=flush), bytes_=2.0 * M * H * 2)
        rec("residual_rmsnorm_fwd", timeit(lambda: ops.residual_rmsnorm_fwd(x, res, 0.3, w, 1e-6), flush=flush), bytes_=4.0 * M * H * 2)
        _, rstd = ops.rmsnorm_fwd(x, w, 1e-6)
        gw = torch.zeros(H, device=dev)
        rec("rmsnorm_bwd", timeit(lambda: ops.rmsnorm_bwd(res, x, w, rstd, gw, res), flush=flush), bytes_=4.0 * M * H * 2)
    if want("swiglu"):
        gu, di = r(M, 2 * F), r(M, F)
        rec("swiglu_fwd", timeit(lambda: ops.swiglu_fwd(gu), flush=flush), bytes_=3.0 * M * F * 2)
        rec("swiglu_bwd", timeit(lambda: ops.swiglu_bwd(di, gu), flush=flush), bytes_=5.0 * M * F * 2)
        del gu, di
    if want("rope"):
        qkv, tab = r(M, cfg.qkv_dim), rope_table(S, d, cfg.rotary_base, dev)
        rec("rope", timeit(lambda: ops.rope_fwd_(qkv, tab, S, nkv, g, d), flush=flush), bytes_=2.0 * M * (cfg.q_dim + cfg.kv_dim) * 2)
    if want("qknorm"):
        # per-head q/k RMSNorm (Qwen3 variant): reads and writes the whole packed QKV forward; backward reads dqkv and the
        # pre-norm copy of the q / k heads and rewrites the q / k heads of dqkv in place
        from ..ops.torch_ops import TorchOps
        qkv, dq = r(M, cfg.qkv_dim), r(M, cfg.qkv_dim)
        wq, wk = r(d), r(d)
        _, rstd = ops.qk_norm_fwd(qkv, wq, wk, 1e-6, nkv, g, d)
        gq, gk = torch.zeros(d, device=dev), torch.zeros(d, device=dev)
        qk_bytes = M * (cfg.q_dim + cfg.kv_dim) * 2
        fns = {"qk_norm_fwd": lambda: ops.qk_norm_fwd(qkv, wq, wk, 1e-6, nkv, g, d),
               "qk_norm_bwd": lambda: ops.qk_norm_bwd(dq, qkv, rstd, wq, wk, gq, gk, nkv, g, d),
               "qk_norm_fwd_pytorch_ops": lambda: TorchOps.qk_norm_fwd(qkv, wq, wk, 1e-6, nkv, g, d),
               "qk_norm_bwd_pytorch_ops": lambda: TorchOps.qk_norm_bwd(dq, qkv, rstd, wq, wk, gq, gk, nkv, g, d)}
        by = {"qk_norm_fwd": 2.0 * M * cfg.qkv_dim * 2, "qk_norm_bwd": 3.0 * qk_bytes}
        for k, t in timeit_many(fns, flush=flush).items():
            rec(k, t, bytes_=by.get(k.replace("_pytorch_ops", ""), 0.0))
        del qkv, dq
    if want("ce"):
        lg = r(M, V)
        lab = torch.randint(0, V, (M,), device=dev, dtype=torch.int32)
        mk = torch.ones(M, device=dev)
        rec("cross_entropy_fwd_bwd", timeit(lambda: ops.cross_entropy_fwd_bwd(lg, lab, mk), iters=5, flush=flush), bytes_=2.0 * M * V * 2)
        del lg
    if want("attn") and hasattr(ops, "attention_fwd"):
        qkv = r(M, cfg.qkv_dim)
        fl = 4.0 * a.mbs * cfg.num_attention_heads * S * S * d / 2  # causal
        out, lse = ops.attention_fwd(qkv, S, nkv, g, d)
        rec("attention_fwd", timeit(lambda: ops.attention_fwd(qkv, S, nkv, g, d), flush=flush), fl)
        if hasattr(ops, "attention_bwd"):
            do = r(M, cfg.q_dim)
            rec("attention_bwd", timeit(lambda: ops.attention_bwd(do, qkv, out, lse, S, nkv, g, d), flush=flush), 2.5 * fl)
        # the library the reference calls (flash-attn 2: forward.py:233, backward.py:510), same shapes, where it is installed:
        # comparison rows only; it needs q / k / v as separate [B, S, heads, d] tensors, so it is given contiguous copies
        try:
            from flash_attn import flash_attn_func
        except Exception:  # noqa: BLE001  (not installed, or built for another architecture)
            flash_attn_func = None
        if flash_attn_func is not None:
            v4 = qkv.view(a.mbs, S, nkv, g + 2, d)
            q = v4[:, :, :, :g].reshape(a.mbs, S, nkv * g, d).contiguous().requires_grad_(True)
            k = v4[:, :, :, g].contiguous().requires_grad_(True)
            vv = v4[:, :, :, g + 1].contiguous().requires_grad_(True)
            try:
                o = flash_attn_func(q, k, vv, causal=True)
                rec("flash_attn2_library_fwd", timeit(lambda: flash_attn_func(q, k, vv, causal=True), flush=flush), fl)
                go = torch.randn_like(o)
                rec("flash_attn2_library_bwd", timeit(lambda: torch.autograd.grad(o, (q, k, vv), go, retain_graph=True), flush=flush), 2.5 * fl)
            except Exception as e:  # noqa: BLE001
                print(json.dumps({"op": "flash_attn2_library", "skipped": f"{type(e).__name__}: {str(e)[:120]}"}), flush=True)
    torch.cuda.synchronize()
    check_status()
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"peaks": peaks, "model": a.model, "mbs": a.mbs, "rows": rows}, f, indent=1)
    return rows


if __name__ == "__main__":
    main()
