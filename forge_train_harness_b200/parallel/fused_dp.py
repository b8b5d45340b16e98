"""Fused data-parallel gradient / parameter path (distributed optimizer over NVLink peer memory).

Replaces ``reduce_scatter -> norm -> AdamW -> bf16 cast -> all_gather`` (three passes over NCCL plus three over local
memory) with two kernels over symmetric memory:

1. ``dp_reduce_scatter``: every rank PULLS its 1/dp slice of each gradient bucket from all peers with plain loads (or one
   ``multimem.ld_reduce`` through the switch), sums in fixed rank order in fp32, writes the slice in place and produces
   the sum of squares for the global-norm clip in the same pass.
2. ``adamw_push``: AdamW on the owned master / moment shard; the rounded bf16 parameter is PUSHED into every rank's
   parameter buffer by the same thread that computed it (or one ``multimem.st``), so the parameter all-gather is not a
   separate collective at all and the next forward's first GEMM simply finds its weights in place.

Ordering between ranks is three flag barriers per step (gradients complete -> pull; pulls done -> buffers reusable;
pushes done -> parameters readable), each a bounded device-side wait.  With gradient accumulation the pulls belong to the
LAST micro-batch of the step, and they overlap its backward bucket by bucket: the flat gradient buffer is laid out in
backward order, so as soon as the backward has passed every parameter of a bucket, ``bucket_ready`` forks a side stream
that waits (flag barrier with a device-numbered epoch, so the fork can live inside a captured CUDA graph) until every rank
has finished that bucket and then pulls this rank's slice of it, while the main stream goes on with the next layers.  Roofline: bytes over NVLink per rank = (dp-1)/dp * 4P (pull) + (dp-1)/dp * 2P (push).
"""
from __future__ import annotations

import sys

import torch

from .symm import PeerBarrier, symm_empty


class FusedDP:
    def __init__(self, store, topo):
        from ..ops.cuda_ops import Sm100Ops
        g = topo.dp_group
        self.store, self.topo = store, topo
        self.grad = symm_empty(store.numel, torch.float32, store.device, g)
        self.param = symm_empty(store.numel, store.dtype, store.device, g)
        self.grad.tensor.zero_()
        self.param.tensor.copy_(store.flat_param)
        store.rebind(self.param.tensor, self.grad.tensor)
        self.barrier = PeerBarrier(store.device, g)
        self.sumsq = torch.zeros((), dtype=torch.float32, device=store.device)
        self._ops = Sm100Ops
        self._table = None
        self.side = torch.cuda.Stream(device=store.device)
        self.buckets_done = 0      # buckets of this step already pulled while the backward was still running
        self.overlapped_total = 0  # over the whole run (reported by tests / the benchmark)

    # -- bucket-by-bucket overlap with the last micro-batch's backward -------------------------------------------------
    def begin_overlap(self) -> None:
        self.sumsq.zero_()
        self.buckets_done = 0

    def bucket_ready(self, opt, idx: int) -> None:
        """Every gradient of bucket ``idx`` is final on THIS rank (main stream order).  On the side stream: wait until that
        holds on every rank, then pull and sum this rank's slice of the bucket (plus its share of the clip norm)."""
        from ..ops.cuda_ops import _C
        self.side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.side):
            self.barrier(3, device_epoch=True)
            r0, r1, _ = opt.my_ranges[idx]
            _C.dp_reduce_scatter(self.grad.ptrs, self.grad.mc_ptr, r0, r1 - r0, self.grad.rank, self.sumsq)
        self.buckets_done += 1
        self.overlapped_total += 1

    def join_overlap(self) -> None:
        torch.cuda.current_stream().wait_stream(self.side)

    def reduce_scatter_sumsq(self, opt) -> torch.Tensor:
        from ..ops.cuda_ops import _C
        rest = list(opt.my_ranges)[self.buckets_done:]
        if self.buckets_done == 0:
            self.sumsq.zero_()
        if rest:
            self.barrier(0)  # every rank's gradients are complete
            for (r0, r1, _) in rest:
                _C.dp_reduce_scatter(self.grad.ptrs, self.grad.mc_ptr, r0, r1 - r0, self.grad.rank, self.sumsq)
        self.buckets_done = 0
        self.barrier(1)  # every pull is done: gradient buffers may be overwritten again
        sq = self.sumsq.clone()
        for (r0, r1, _) in opt.my_ranges:  # gradients that are replicas of another model-parallel rank's count once
            for (d0, d1) in ([] if getattr(opt, "tp_local_norm", False) else opt.dup_ranges):
                lo, hi = max(d0, r0), min(d1, r1)
                if hi > lo:
                    sq = sq - opt.ops.sumsq(self.store.flat_grad[lo:hi])
        return sq

    def adam_allgather(self, opt, lr: float, scale: torch.Tensor) -> None:
        from ..ops.cuda_ops import _C
        oc = opt.oc
        if self._table is None:
            self._table = self._ops.build_adam_table(opt.segs, self.store.device)
        buf, n = self._table
        _C.adamw_push(opt.master, opt.m, opt.v, self.store.flat_grad, self.param.ptrs, self.param.mc_ptr, buf, n, float(lr),
                      oc.adam_beta1, oc.adam_beta2, oc.adam_eps, oc.weight_decay, opt.step_count,
                      scale.reshape(1).to(torch.float32))
        self.barrier(2)  # every push has landed: parameters are readable everywhere


def try_create(store, topo, required: bool = False):
    """Returns a ``FusedDP`` or None (then the NCCL path runs).  Needs bf16 parameters, dp <= 8, and symmetric memory.
    The reason for a fallback is printed by rank 0; with ``required`` (``FORGE_FUSED_DP=require``) it raises instead."""
    if store.dtype != torch.bfloat16 or topo.dp > 8:
        if required:
            raise RuntimeError("fused DP path needs bf16 parameters and dp <= 8")
        return None
    try:
        return FusedDP(store, topo)
    except Exception as e:  # noqa: BLE001
        if required:
            raise
        if topo.rank == 0:
            print(f"[warn] fused DP path unavailable ({type(e).__name__}: {e}); using NCCL collectives", file=sys.stderr, flush=True)
        return None
