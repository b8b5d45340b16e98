"""In-kernel timelines of the flash-attention kernels: where a step of the forward / backward inner loop spends its cycles.

    python -m forge_train_harness_b200.utils.attn_timeline [--seq 4096 --batch 4 --n-kv 2 --g 8 --d 64]

Both kernels can stamp ``clock64()`` at the phase boundaries of their inner loops for ONE chosen CTA (``flash_fwd_set_debug`` /
``flash_bwd_set_debug`` hand them a device buffer; without one the stamps are skipped).  This tool runs one launch with the
buffer set and prints the median cycles per phase: softmax side (wait for S, tensor-memory load, row max + exchange,
exponentials + P store, O correction) for the forward, and per query half of the backward (wait for Q / S^T, first load,
math + stores, fence + arrive) plus the MMA warp's issue segments.  This is how the bottlenecks named in
``profiles/flash_attention_fwd_bwd_d64_s4096.md`` were found (a profiler's counters are per kernel, not per phase).
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

FWD_PHASES = ["wait_s_full", "tmem_ld", "max+xchg", "exp+st", "o_done+fix", "wait_st+arrive", "loop_gap"]
BWD_WG_STAMPS = [0, 6, 1, 2, 3, 4]
BWD_WG_PHASES = ["wait_q", "wait_sdp", "ld0", "math+st", "fence+arrive", "loop"]
BWD_MMA_PHASES = ["wait_pds0", "issue_dkv0+wait_q", "issue_sdp0", "wait_pds1", "issue_dkv1+wait_drained", "issue_dq+sdp1", "loop"]


def _medians(stamps: np.ndarray, order, names) -> dict | None:
    """``stamps[i, step]``: cycles between consecutive stamps of one step (the last phase ends at the next step's first stamp)."""
    n = int((stamps[order[0]] > 0).sum())
    rows = []
    for st in range(2, n - 1):
        t = [int(stamps[i, st]) for i in order] + [int(stamps[order[0], st + 1])]
        rows.append([t[i + 1] - t[i] for i in range(len(order))])
    if not rows:
        return None
    rows = np.array(rows)
    out = dict(zip(names, np.median(rows, 0).astype(int).tolist()))
    out["total"] = int(np.median(rows.sum(1)))
    out["steps"] = n
    return out


def forward_timeline(S=4096, B=4, n_kv=2, g=8, d=64) -> dict:
    from ..ops.cuda_ops import Sm100Ops as ops, _C
    qkv = torch.randn(B * S, n_kv * (g + 2) * d, device="cuda").mul_(0.5).to(torch.bfloat16)
    for _ in range(3):
        ops.attention_fwd(qkv, S, n_kv, g, d)
    dbg = torch.zeros(2 * 8 * 64, dtype=torch.int64, device="cuda")
    _C.flash_fwd_set_debug(dbg.data_ptr())
    try:
        ops.attention_fwd(qkv, S, n_kv, g, d)
        torch.cuda.synchronize()
    finally:
        _C.flash_fwd_set_debug(0)
    t = dbg.view(2, 8, 64).cpu().numpy()
    return {f"query_tile_{i}": _medians(t[i], list(range(7)), FWD_PHASES) for i in range(2)}


def backward_timeline(S=4096, B=4, n_kv=2, g=8, d=64) -> dict:
    from ..ops.cuda_ops import Sm100Ops as ops, _C
    qkv = torch.randn(B * S, n_kv * (g + 2) * d, device="cuda").mul_(0.5).to(torch.bfloat16)
    out, lse = ops.attention_fwd(qkv, S, n_kv, g, d)
    do = torch.randn(B * S, n_kv * g * d, device="cuda").mul_(0.5).to(torch.bfloat16)
    for _ in range(3):
        ops.attention_bwd(do, qkv, out, lse, S, n_kv, g, d)
    dbg = torch.zeros(3 * 8 * 64, dtype=torch.int64, device="cuda")
    _C.flash_bwd_set_debug(dbg.data_ptr())
    try:
        ops.attention_bwd(do, qkv, out, lse, S, n_kv, g, d)
        torch.cuda.synchronize()
    finally:
        _C.flash_bwd_set_debug(0)
    t = dbg.view(3, 8, 64).cpu().numpy()
    res = {f"query_half_{h}": _medians(t[h], BWD_WG_STAMPS, BWD_WG_PHASES) for h in range(2)}
    res["mma_warp"] = _medians(t[2], list(range(7)), BWD_MMA_PHASES)
    return res


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--n-kv", type=int, default=2)
    ap.add_argument("--g", type=int, default=8)
    ap.add_argument("--d", type=int, default=64)
    a = ap.parse_args(argv)
    print(json.dumps({"forward": forward_timeline(a.seq, a.batch, a.n_kv, a.g, a.d),
                      "backward": backward_timeline(a.seq, a.batch, a.n_kv, a.g, a.d) if a.d == 64 else None}, indent=1))


if __name__ == "__main__":
    main()
