"""Distributed optimizer: fp32 master weights + AdamW state, optionally ZeRO-1 sharded over DP.

Semantics: gradients are SUMMED over micro-batches and ranks in fp32, then scaled by
``1 / (global number of loss tokens)`` (train_loop.py:2391-2393); the global L2 norm is clipped
with ``min(1, clip / (norm + 1e-6))`` (``torch.nn.utils.clip_grad_norm_``, used by
ref/reference/train_pure_mup_mtp.py:805); AdamW runs on the fp32 master with four muP x
weight-decay groups — matrix weights get ``lr / width_mult``, tensors with fewer than two
dimensions get no weight decay (train_loop.py:1119-1171) — and the compute-dtype parameters
are re-derived from the master (train_loop.py:1275-1328).

Sharded mode is the Megatron distributed-optimizer layout (``--use-distributed-optimizer``,
ref/reference/train_minicpm4_0.5b_gsm8k.sh:311): every bucket of the flat gradient buffer is
reduce-scattered, each DP rank keeps master / exp_avg / exp_avg_sq only for its 1/dp slice of
every bucket, and the updated low-precision slices are all-gathered back.  Unlike the
reference's param-granular ZeRO-1 (zero_optimizer.py:78-88, known to hang) the partition is
element-granular and equal-sized, so the collectives are plain tensor collectives.

``comm`` selects the collective implementation: ``"nccl"`` (library; also gloo on CPU) or a
fused-kernel backend object exposing ``reduce_scatter_sumsq`` / ``adam_allgather``.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..models.store import ParamStore
from ..models import params as P
from ..parallel.topology import Topology


def _intersect(a0, a1, b0, b1):
    lo, hi = max(a0, b0), min(a1, b1)
    return (lo, hi) if hi > lo else None


def shard_ranges(buckets, dp_world: int, dp_rank: int) -> list[tuple[int, int, int]]:
    """``[(flat_start, flat_end, shard_offset)]``, one per bucket: the slice of the flat buffer DP rank ``dp_rank`` owns and where
    it sits in that rank's shard.  ``buckets`` are ``(start, end)`` pairs (or objects with those attributes)."""
    out = []
    for b in buckets:
        start, end = (b.start, b.end) if hasattr(b, "start") else (int(b[0]), int(b[1]))
        lr_ = (end - start) // dp_world
        s0 = start + dp_rank * lr_
        out.append((s0, s0 + lr_, start // dp_world))
    return out


class DistributedOptimizer:
    def __init__(self, store: ParamStore, topo: Topology, optim_cfg, ops, *, sharded: bool,
                 sequence_parallel: bool = False, fused_backend=None, clip_norm_scope: str = "global"):
        self.store, self.topo, self.oc, self.ops = store, topo, optim_cfg, ops
        self.sharded = bool(sharded and topo.dp > 1)
        self.dpw = topo.dp if self.sharded else 1
        self.dpr = topo.dp_rank if self.sharded else 0
        self.sp = sequence_parallel and topo.tp > 1
        self.fused = fused_backend
        self.tp_local_norm = clip_norm_scope == "tp_local"
        dev = store.device
        n_shard = store.numel // self.dpw
        self.master = torch.zeros(n_shard, dtype=torch.float32, device=dev)
        self.m = torch.zeros(n_shard, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n_shard, dtype=torch.float32, device=dev)
        self.step_count = 0
        cfg = store.cfg
        # my flat ranges, one per bucket: (flat_start, flat_end, shard_off)
        self.my_ranges = shard_ranges(store.buckets, self.dpw, self.dpr)
        # Adam segments: param ∩ my range
        self.segs = []
        for spec in store.specs:
            o, n = store.offsets[spec.name]
            lr_mult = (1.0 / cfg.width_mult) if spec.is_matrix else 1.0
            for (r0, r1, so) in self.my_ranges:
                it = _intersect(o, o + n, r0, r1)
                if it:
                    self.segs.append((so + it[0] - r0, it[0], it[1] - it[0], lr_mult, spec.weight_decay))
        self.segs.sort(key=lambda s: s[0])
        self._table = None  # device-side segment table, built lazily by the CUDA op
        # flat ranges whose gradients are duplicates of another model-parallel rank's
        self.dup_ranges = []
        kv_rows = P.kv_replicated_rows(cfg, topo.tp, topo.tp_rank) if topo.tp > 1 else None
        for spec in store.specs:
            o, n = store.offsets[spec.name]
            if topo.tp > 1 and spec.kind == "replicated" and topo.tp_rank != 0:
                self.dup_ranges.append((o, o + n))
            if spec.kind == "qkv" and kv_rows is not None and topo.tp_rank % P.tp_geometry(cfg, topo.tp, topo.tp_rank).kv_replicas != 0:
                H = store.shapes[spec.name][1]
                self.dup_ranges.append((o + int(kv_rows[0]) * H, o + (int(kv_rows[-1]) + 1) * H))
            if spec.name == "tok_embeddings.weight" and store.tied_copy:
                self.dup_ranges.append((o, o + n))
        self._kv_rows = kv_rows
        self.sync_master_from_params()

    # ------------------------------------------------------------------
    def sync_master_from_params(self) -> None:
        for (r0, r1, so) in self.my_ranges:
            self.master[so:so + (r1 - r0)].copy_(self.store.flat_param[r0:r1])

    def sync_params_from_master(self) -> None:
        for (r0, r1, so) in self.my_ranges:
            self.store.flat_param[r0:r1].copy_(self.master[so:so + (r1 - r0)])
        self._all_gather_params()

    # ------------------------------------------------------------------
    def reduce_model_parallel_grads(self) -> None:
        """Sums that tensor / pipeline parallelism leave to do before the DP reduction:
        sequence-parallel partial sums of replicated (norm) weights over TP, replicated KV-head
        rows over their replica group, and the tied embedding over first + last stage."""
        st, topo = self.store, self.topo
        if topo.tp > 1:
            # With sequence parallelism every replicated weight (the norms) saw only this rank's rows.  Without it the
            # per-head q / k norm weights still saw only this rank's heads: their gradients are partial sums whatever
            # the sequence layout, and left alone the replicas would drift apart.
            bufs = [st.g(s.name) for s in st.specs if s.kind == "replicated" and (self.sp or P.is_head_partial(s))]
            if bufs:
                flat = torch.cat([b.reshape(-1) for b in bufs])
                dist.all_reduce(flat, group=topo.tp_group)
                o = 0
                for b in bufs:
                    b.copy_(flat[o:o + b.numel()].view_as(b))
                    o += b.numel()
        if self._kv_rows is not None and topo.kv_group is not None:
            r0, r1 = int(self._kv_rows[0]), int(self._kv_rows[-1]) + 1
            for s in st.specs:
                if s.kind == "qkv":
                    dist.all_reduce(st.g(s.name)[r0:r1], group=topo.kv_group)
        if (st.cfg.tie_embeddings or st.cfg.mtp_num_layers) and topo.pp > 1 and topo.embed_group is not None and \
                "tok_embeddings.weight" in st.grads and (topo.is_first_stage or topo.is_last_stage):
            dist.all_reduce(st.g("tok_embeddings.weight"), group=topo.embed_group)

    # -- bucket-by-bucket overlap of the DP reduction with the last micro-batch's backward -------------------------
    def overlap_eligible(self) -> bool:
        """Buckets can be reduced while the backward still runs when nothing has to be summed over model-parallel ranks
        first (no TP / PP); both the library path (asynchronous collectives) and the peer-memory path (side-stream pulls
        behind a flag barrier) do it."""
        t = self.topo
        return t.dp > 1 and t.tp == 1 and t.pp == 1

    def begin_overlap(self) -> None:
        self._done_names: set = set()
        self._launched = 0
        self._works: list = []
        self.overlapped_buckets = 0
        if self.fused is not None:
            self.fused.begin_overlap()

    def grads_final(self, prefix: str) -> None:
        """Called by the backward when every parameter whose name starts with ``prefix`` has its final gradient of this
        step.  Launches, in bucket order, the asynchronous reduction of every bucket that is now complete (the flat
        buffer is laid out in backward order, so buckets complete front to back)."""
        st, topo = self.store, self.topo
        self._done_names.update(n for n in st.offsets if n.startswith(prefix))
        while self._launched < len(st.buckets) and all(n in self._done_names for n in st.buckets[self._launched].names):
            b = st.buckets[self._launched]
            buf = st.flat_grad[b.start:b.end]
            if self.fused is not None:
                self.fused.bucket_ready(self, self._launched)
                self._launched += 1
                self.overlapped_buckets += 1
                continue
            if self.sharded and buf.device.type != "cpu":
                r0, r1, _ = self.my_ranges[self._launched]
                w = dist.reduce_scatter_tensor(st.flat_grad[r0:r1], buf, group=topo.dp_group, async_op=True)
            else:
                w = dist.all_reduce(buf, group=topo.dp_group, async_op=True)
            self._works.append(w)
            self._launched += 1
            self.overlapped_buckets += 1

    def _reduce_grads(self) -> None:
        topo, st = self.topo, self.store
        if topo.dp == 1:
            return
        launched = getattr(self, "_launched", 0)
        for w in getattr(self, "_works", []):
            w.wait()
        self._works, self._launched = [], 0
        if not self.sharded:
            if launched == 0:
                dist.all_reduce(st.flat_grad, group=topo.dp_group)
            elif launched < len(st.buckets):
                dist.all_reduce(st.flat_grad[st.buckets[launched].start:], group=topo.dp_group)
            return
        for b, (r0, r1, _) in list(zip(st.buckets, self.my_ranges))[launched:]:
            buf = st.flat_grad[b.start:b.end]
            if buf.device.type == "cpu":
                dist.all_reduce(buf, group=topo.dp_group)
            else:
                dist.reduce_scatter_tensor(st.flat_grad[r0:r1], buf, group=topo.dp_group)

    def _all_gather_params(self) -> None:
        topo, st = self.topo, self.store
        if not self.sharded:
            return
        for b, (r0, r1, _) in zip(st.buckets, self.my_ranges):
            buf = st.flat_param[b.start:b.end]
            if buf.device.type == "cpu":
                parts = list(buf.chunk(self.dpw))
                dist.all_gather(parts, st.flat_param[r0:r1].clone(), group=topo.dp_group)
            else:
                dist.all_gather_into_tensor(buf, st.flat_param[r0:r1], group=topo.dp_group)

    def _local_sumsq(self) -> torch.Tensor:
        st = self.store
        tot = torch.zeros((), dtype=torch.float32, device=st.device)
        for (r0, r1, _) in self.my_ranges:
            tot = tot + self.ops.sumsq(st.flat_grad[r0:r1])
            for (d0, d1) in ([] if self.tp_local_norm else self.dup_ranges):
                it = _intersect(d0, d1, r0, r1)
                if it:
                    tot = tot - self.ops.sumsq(st.flat_grad[it[0]:it[1]])
        return tot

    # ------------------------------------------------------------------
    def step(self, lr: float, inv_tokens: torch.Tensor) -> torch.Tensor:
        """One optimizer step.  ``inv_tokens`` is a 0-dim fp32 tensor.  Returns the global grad norm
        (of the token-normalised gradient) as a 0-dim tensor; nothing here synchronises the host."""
        st, topo, oc = self.store, self.topo, self.oc
        self.step_count += 1
        self.reduce_model_parallel_grads()
        if self.fused is not None:
            self._works, self._launched = [], 0
            sq = self.fused.reduce_scatter_sumsq(self)
        else:
            self._reduce_grads()
            sq = self._local_sumsq()
        if self.tp_local_norm:
            # this TP rank's own shards only (replicated weights included): sum the DP slices of a ZeRO-1 shard, nothing else
            if self.sharded:
                sq = sq.reshape(1).clone()
                dist.all_reduce(sq, group=topo.dp_group)
                sq = sq[0]
        elif topo.world_size > 1:
            sq = sq.reshape(1).clone()
            dist.all_reduce(sq)
            sq = sq[0]
            if not self.sharded and topo.dp > 1:
                sq = sq / topo.dp
        norm = torch.sqrt(torch.clamp(sq, min=0.0)) * inv_tokens
        if oc.clip_grad > 0:
            coef = torch.clamp(oc.clip_grad / (norm + 1e-6), max=1.0)
        else:
            coef = torch.ones_like(norm)
        scale = (coef * inv_tokens).to(torch.float32)
        if self.fused is not None:
            self.fused.adam_allgather(self, lr, scale)
        else:
            self._table = self.ops.adamw_segments(
                self.master, self.m, self.v, st.flat_grad, st.flat_param, self.segs, lr, oc.adam_beta1,
                oc.adam_beta2, oc.adam_eps, oc.weight_decay, self.step_count, scale, self._table)
            self._all_gather_params()
        return norm

    # ------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"master": self.master, "exp_avg": self.m, "exp_avg_sq": self.v, "step": self.step_count,
                "dp_world": self.dpw, "dp_rank": self.dpr}

    def load_state_dict(self, sd: dict, weights_only: bool = False) -> None:
        self.master.copy_(sd["master"])
        if not weights_only:
            self.m.copy_(sd["exp_avg"])
            self.v.copy_(sd["exp_avg_sq"])
            self.step_count = int(sd["step"])
        self.sync_params_from_master()

    def set_flat_range(self, key: str, flat_start: int, values: torch.Tensor) -> None:
        """Write ``values`` (fp32, 1-D) as elements ``[flat_start, flat_start + len)`` of the FLAT state ``key``
        (``master`` | ``exp_avg`` | ``exp_avg_sq``); only the part this rank's shard owns is kept."""
        t = {"master": self.master, "exp_avg": self.m, "exp_avg_sq": self.v}[key]
        n = values.numel()
        for (r0, r1, so) in self.my_ranges:
            it = _intersect(flat_start, flat_start + n, r0, r1)
            if it:
                t[so + it[0] - r0: so + it[1] - r0].copy_(values[it[0] - flat_start: it[1] - flat_start])

    # full (unsharded) views for layout-independent checkpoints ---------------
    def gather_full_state(self) -> dict[str, torch.Tensor]:
        """``{"master"|"exp_avg"|"exp_avg_sq": flat fp32 [numel]}`` assembled over the DP shards."""
        out = {}
        for key, t in (("master", self.master), ("exp_avg", self.m), ("exp_avg_sq", self.v)):
            full = torch.zeros(self.store.numel, dtype=torch.float32, device=t.device)
            if self.dpw == 1:
                for (r0, r1, so) in self.my_ranges:
                    full[r0:r1] = t[so:so + r1 - r0]
            else:
                parts = [torch.empty_like(t) for _ in range(self.dpw)]
                dist.all_gather(parts, t, group=self.topo.dp_group)
                for b in self.store.buckets:
                    lr_ = (b.end - b.start) // self.dpw
                    for r in range(self.dpw):
                        so = b.start // self.dpw
                        full[b.start + r * lr_: b.start + (r + 1) * lr_] = parts[r][so:so + lr_]
            out[key] = full
        return out

    def scatter_full_state(self, full: dict[str, torch.Tensor], step: int, weights_only: bool = False) -> None:
        pairs = [("master", self.master)]
        if not weights_only:
            pairs += [("exp_avg", self.m), ("exp_avg_sq", self.v)]
            self.step_count = int(step)
        for key, t in pairs:
            for (r0, r1, so) in self.my_ranges:
                t[so:so + r1 - r0].copy_(full[key][r0:r1])
        self.sync_params_from_master()
