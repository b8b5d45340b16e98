"""Training engine: one process per GPU, static forward / manual backward, distributed optimizer.

Public contract (the counterpart of ``TrainLoopConfig`` / ``run_training_loop`` in
workload/src/training_engine_tensor/train_loop.py:120-167, 1508-2557): build a ``RunConfig``, call
``run_training_loop(cfg)``; rank 0 prints one ``[LOSS] step= global_loss= grad_norm= time_s=
mfu_e2e_standard=`` line per step and a ``[PHASE]`` banner.  Per step: zero the flat fp32 gradient,
run ``grad_accum`` micro-batches (one pinned H2D copy each, CUDA-graph replay of forward + loss +
backward when enabled), all-reduce the fp64 loss statistics, run the distributed optimizer (gradient
reduce-scatter / all-reduce, 1/tokens scale, global-norm clip, AdamW on fp32 master, low-precision
parameter all-gather), log, checkpoint.

Differences from the reference, on purpose: step time is device-timed and the reported MFU divides by
the MEASURED B200 bf16 peak and uses the max over ranks (the reference uses rank 0 and a hard-coded H100
peak, train_loop.py:89, 2496-2504); nothing but the once-per-step log read synchronises the host (the
reference's ``if total_norm > clip`` does, train_loop.py:2444); resume restores the data cursor instead
of replaying batches (train_loop.py:1489-1505).
"""
from __future__ import annotations

import os
import random
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

from .config.schema import RunConfig
from .data.sources import BatchStager, Prefetcher, build_source, build_mtp_tensors
from .models import params as P
from .models.minicpm4 import ModelChunk
from .models.store import ParamStore, pipeline_chunks
from .ops import get_ops, rope_table
from .optim.distributed import DistributedOptimizer
from .optim.schedule import compute_lr
from .parallel.pipeline import PipeLinks, build_schedule
from .parallel.topology import Topology, build_topology, init_distributed, spans_nodes
from .parallel.tp import TPComm
from .utils import wire
from .utils.peaks import load_peaks, mfu_percent


def _dtype_of(name: str):
    return {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}[name]


class Trainer:
    def __init__(self, cfg: RunConfig, *, device=None, ops=None, topo: Topology | None = None,
                 init_mode: str = "reference", capture=None, quiet: bool = False):
        self.cfg = cfg
        t, m, par = cfg.train, cfg.model, cfg.parallel
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.quiet = quiet
        geo0 = P.tp_geometry(m, par.tensor_parallel_size, 0)
        self.topo = topo or build_topology(par.tensor_parallel_size, par.pipeline_parallel_size, geo0.kv_replicas)
        topo = self.topo
        self.rank, self.world = topo.rank, topo.world_size
        self.dtype = _dtype_of(t.dtype)
        self._seed_all(t.seed)
        if t.deterministic:
            os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
            torch.use_deterministic_algorithms(True, warn_only=True)
        self.ops = ops or get_ops(self.device)
        if hasattr(self.ops, "set_deterministic"):
            self.ops.set_deterministic(bool(t.deterministic))
        if par.fp8 == "mxfp8" and self.dtype == torch.bfloat16:
            # block-scaled fp8 for every linear product whose dimensions are multiples of 32 (the ragged vocabulary
            # products stay bf16); the one-kernel TP paths are bf16 kernels, so this option uses the library collectives
            from .ops.mxfp8 import Mxfp8Ops
            self.ops = Mxfp8Ops(self.ops)
        self.tpc = TPComm(topo.tp_group, topo.tp, topo.tp_rank, par.sequence_parallel)
        want_tp = os.environ.get("FORGE_FUSED_TP", "1")  # "0" = NCCL collectives, "require" = fail instead of falling back
        if self.tpc.sp and self.device.type == "cuda" and par.fused_comm and self.dtype == torch.bfloat16 and par.fp8 == "off" \
                and want_tp != "0" and not spans_nodes(topo.tp_ranks):
            from .parallel import fused_tp
            self.tpc.fused = fused_tp.try_create(topo.tp_group, topo.tp, topo.tp_rank, t.micro_batch_size * m.seq_length,
                                                 m.hidden_size, self.device, required=want_tp == "require")
        chunks = pipeline_chunks(m, topo.pp, par.virtual_pipeline_stages, topo.pp_rank, par.pipeline_layer_split)
        self.store = ParamStore(m, chunks, tp=topo.tp, tp_rank=topo.tp_rank, dp=topo.dp, dtype=self.dtype,
                                device=self.device, bucket_elems=par.ddp_bucket_elems, pp=topo.pp)
        self._init_weights(init_mode)
        self.rope = rope_table(m.max_position_embeddings, m.head_dim, m.rotary_base, self.device)
        self.capture = capture
        self.chunks = [ModelChunk(m, self.store, c, self.ops, self.tpc, self.rope,
                                  capture.module_hook if capture is not None and capture.level >= 2 else None)
                       for c in chunks]
        for c in self.chunks:
            c.recompute = t.recompute
            c.recompute_num_layers = t.recompute_num_layers
            c.debug_checks = t.debug_checks or os.environ.get("FORGE_DEBUG_CHECKS", "0") == "1"
        fused = None
        want_dp = os.environ.get("FORGE_FUSED_DP", "1")
        if self.device.type == "cuda" and par.fused_comm and par.use_distributed_optimizer and topo.dp > 1 and want_dp != "0" \
                and not spans_nodes(topo.dp_ranks):     # a DP group that crosses nodes keeps NCCL
            from .parallel import fused_dp
            fused = fused_dp.try_create(self.store, topo, required=want_dp == "require")
        self.opt = DistributedOptimizer(self.store, topo, cfg.optim, self.ops, sharded=par.use_distributed_optimizer,
                                        sequence_parallel=par.sequence_parallel, fused_backend=fused,
                                        clip_norm_scope=par.clip_norm_scope)
        self.links = PipeLinks(topo)
        self.grad_accum = cfg.grad_accum(topo.dp)
        self.source = build_source(cfg.data, m, t.micro_batch_size, topo.dp_rank, topo.dp, t.seed)
        self.prefetch = None
        self.with_mtp = bool(m.mtp_num_layers)   # under PP the branch lives on the last stage (with its own copy of the embedding)
        self.stager = BatchStager(t.micro_batch_size, m.seq_length, self.device, self.with_mtp,
                                  dev_slots=self.grad_accum if topo.pp > 1 else 1)
        self.step = t.start_step  # completed steps (absolute)
        self.peaks = load_peaks()
        self.flops_per_token = m.flops_per_token(self.with_mtp)
        self._graph = None
        self._graph_last = None       # the last micro-batch of a step, with the DP bucket pulls forked off its backward
        self._graph_last_stats = None
        self._graph_last_buckets = 0
        self._graph_stats = None
        self._graph_failed = False
        self.graph_launches = 0  # sm_100a kernels recorded in the captured micro-batch graph
        self.graph_replays = 0
        self._layer_graphs = False  # TP / PP runs: the chunks' layer loops are replayed from CUDA graphs (after one eager step)
        self._layer_graph_steps = 0  # steps run since the layer graphs were enabled (the first of them captures)
        self.stats = torch.zeros(4, dtype=torch.float64, device=self.device)
        self.launch_count = 0
        self.last = {}
        # Reader of the device status word the sm_100a kernels write when a bounded wait gives up (an mbarrier that never
        # completed, a peer flag that never arrived).  None when no such kernel can run (CPU, oracle ops).
        self._read_status = None
        if self.device.type == "cuda" and self.ops.name.startswith("sm100"):
            from .ops.cuda_ops import _C
            self._read_status = lambda: int(_C.read_status(True))

    # ------------------------------------------------------------------
    def _seed_all(self, seed: int):
        random.seed(seed)
        np.random.seed(seed % (2 ** 32))
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)

    def _init_weights(self, init_mode: str):
        t = self.cfg.train
        root = self.cfg.ckpt.checkpoint_root
        canon = os.path.join(root, "canonical_state_fp32.pt") if root else ""
        if canon and os.path.isfile(canon):
            self.store.load_canonical_state(torch.load(canon, map_location="cpu", weights_only=True))
        elif init_mode == "device":
            self.store.init_device(t.seed, t.forge_init_ones)
        elif init_mode == "reference":
            self.store.init_reference(t.seed, t.forge_init_ones)
        else:
            raise ValueError(f"init_mode must be 'reference' or 'device', not {init_mode!r}")

    def start_data(self):
        if self.prefetch is None:
            self.prefetch = Prefetcher(self.source, self.cfg.data.prefetch_size,
                                       enabled=self.cfg.data.prefetch_size > 0)

    # ------------------------------------------------------------------
    def _mb_stats(self, out: dict, batch: dict):
        nll = out["nll"]
        s = torch.zeros(4, dtype=torch.float64, device=self.device)
        s[0] = nll.sum(dtype=torch.float64)
        s[1] = batch["mask"].sum(dtype=torch.float64)
        if "mtp_nll" in out:
            s[2] = out["mtp_nll"].sum(dtype=torch.float64)
            s[3] = batch["mtp_mask"].sum(dtype=torch.float64)
        return s

    def _fwd_bwd(self, batch: dict):
        """One micro-batch through the single local chunk (no pipeline).  Returns fp64[4] stats."""
        ch = self.chunks[0]
        out, cache = ch.forward(batch)
        if self.capture is not None:
            self.capture.per_token_loss(out["nll"], self.cfg.train.micro_batch_size)
        stats = self._mb_stats(out, batch)
        ch.run_backward(batch, cache)
        return stats

    def verify_kernels(self, sync: bool = True) -> None:
        """Raise if any kernel of the work enqueued so far gave up on a bounded wait.  A kernel that gives up returns
        early, so whatever consumed its output (a gradient sum, a parameter push, a gathered shard) is wrong: the step
        must not be logged, checkpointed or followed by another one.  Synchronises the host with the device."""
        if self._read_status is None:
            return
        if sync and self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        code = self._read_status()
        if code:
            from .ops.status import STATUS_NAMES
            where = ""
            if code == 7:
                from .ops.cuda_ops import Sm100Ops
                where = f" [first bad position in its tensor: {Sm100Ops.bad_index_position()}]"
            raise RuntimeError(f"step {self.step}: sm_100a kernel reported status {code} "
                               f"({STATUS_NAMES.get(code, 'unknown')}){where}; the step's results are not valid")

    def _fwd_bwd_overlapped(self, batch: dict):
        """The last micro-batch of a step: every gradient bucket goes to the DP reduction as soon as the backward has passed
        its parameters, so the collective (library path) or the peer-memory pulls (fused path) run under the rest of it."""
        self.opt.begin_overlap()
        self.chunks[0].on_grads_final = self.opt.grads_final
        try:
            stats = self._fwd_bwd(batch)
        finally:
            self.chunks[0].on_grads_final = None
        if self.opt.fused is not None:
            self.opt.fused.join_overlap()
        return stats

    def _capture_last_graph(self, batch: dict):
        """Second graph, sharing the first one's memory pool (they never run at the same time).  The gradient buffer is
        restored afterwards: the capture itself launches nothing, but the first replay must see this step's sums."""
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=self._graph.pool()):
                self._graph_last_stats = self._fwd_bwd_overlapped(batch)
            self._graph_last_buckets = self.opt.fused.buckets_done
            self.opt.fused.overlapped_total -= self._graph_last_buckets   # counted at replay
            self.opt.fused.buckets_done = 0
            self._graph_last = g
        except Exception as e:  # keep training with the plain graph and the pulls after the backward
            self._graph_last = None
            self.cfg = self.cfg.replace(parallel={"overlap_grad_reduce": False})
            if not self.quiet and self.rank == 0:
                print(f"[warn] capture of the overlapped last micro-batch failed, pulling after the backward: {e}", file=sys.stderr, flush=True)
            torch.cuda.synchronize()

    def _try_capture_graph(self, batch: dict):
        """Capture forward + loss + backward of ONE micro-batch (train_loop.py:1926-2125)."""
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._fwd_bwd(batch)  # warm-up: allocator, lazy handles
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.verify_kernels(sync=False)
            self.store.zero_grad()
            g = torch.cuda.CUDAGraph()
            n0 = self._launch_count()
            with torch.cuda.graph(g):
                self._graph_stats = self._fwd_bwd(batch)
            self.graph_launches = self._launch_count() - n0
            self._graph = g
        except RuntimeError as e:
            if "kernel reported status" in str(e):
                raise
            self._graph, self._graph_failed = None, True
            if not self.quiet and self.rank == 0:
                print(f"[debug] CUDA graph capture failed, running eager: {e}", file=sys.stderr, flush=True)
            torch.cuda.synchronize()
            self.store.zero_grad()
        except Exception as e:  # fall back to eager, as the reference does
            self._graph, self._graph_failed = None, True
            if not self.quiet and self.rank == 0:
                print(f"[debug] CUDA graph capture failed, running eager: {e}", file=sys.stderr, flush=True)
            torch.cuda.synchronize()
            self.store.zero_grad()

    def _launch_count(self) -> int:
        if self.device.type != "cuda" or not self.ops.name.startswith("sm100"):
            return 0
        from .ops.cuda_ops import _C
        return int(_C.launch_count())

    def _maybe_enable_layer_graphs(self) -> None:
        """Tensor / pipeline-parallel runs cannot capture a whole micro-batch (pipeline send / recv and the library
        collectives of the embedding and the head sit between the chunks), but the layer loops between them can be: after
        the first step has run eagerly (lazy allocations, symmetric-memory rendezvous of every call site), each chunk
        captures its forward and backward layer loop once per in-flight slot and replays them from then on.  The decision
        depends only on the configuration, so every rank of the job takes it at the same step."""
        t, topo = self.cfg.train, self.topo
        if self._layer_graphs or not t.cuda_graph or self.device.type != "cuda" or self.capture is not None:
            return
        if topo.tp == 1 and topo.pp == 1:
            return                       # the whole micro-batch is captured instead (_try_capture_graph)
        if self.ops.name != "sm100" or os.environ.get("FORGE_LAYER_GRAPHS", "1") == "0":
            return
        if topo.tp > 1 and self.tpc.fused is None:
            return                       # library collectives inside the layer loop: left eager
        if self.with_mtp or self.cfg.model.qk_norm or t.recompute_num_layers:
            return
        for c in self.chunks:
            c.enable_graphs()
        self._layer_graphs = True

    def _use_graph(self) -> bool:
        t = self.cfg.train
        return (t.cuda_graph and self.device.type == "cuda" and self.topo.pp == 1 and self.topo.tp == 1
                and self.capture is None and not self._graph_failed)

    # ------------------------------------------------------------------
    def _run_microbatches_nopp(self):
        for mb in range(self.grad_accum):
            if self.capture is not None:
                self.capture.begin_microbatch(mb)
            batch = self.stager.stage(self.prefetch.get())
            last = mb == self.grad_accum - 1
            overlap = last and self.cfg.parallel.overlap_grad_reduce and self.opt.overlap_eligible()
            if self._use_graph():
                if self._graph is None:
                    self._try_capture_graph(batch)
                if self._graph is not None:
                    if overlap and self.opt.fused is not None:
                        # the last micro-batch has its own graph: same kernels, plus the bucket pulls on a forked stream
                        if self._graph_last is None:
                            self._capture_last_graph(batch)
                        if self._graph_last is not None:
                            self.opt.begin_overlap()
                            self._graph_last.replay()
                            self.graph_replays += 1
                            self.stats += self._graph_last_stats
                            self.opt.fused.buckets_done = self._graph_last_buckets
                            self.opt.fused.overlapped_total += self._graph_last_buckets
                            continue
                    self._graph.replay()
                    self.graph_replays += 1
                    self.stats += self._graph_stats
                    continue
            if overlap:
                # eager last micro-batch: each gradient bucket is handed to the DP reduction as soon as the backward has
                # passed its parameters, so the collective runs under the rest of the backward
                self.stats += self._fwd_bwd_overlapped(batch)
                continue
            self.stats += self._fwd_bwd(batch)

    def _run_microbatches_pp(self):
        topo, t, m = self.topo, self.cfg.train, self.cfg.model
        n_mb = self.grad_accum
        # one pinned-buffer H2D copy per micro-batch, each into its own device copy (all are alive until their backward)
        batches = [self.stager.stage(self.prefetch.get(), slot=i) for i in range(n_mb)]
        vpp = self.cfg.parallel.virtual_pipeline_stages
        sched = build_schedule(topo.pp, topo.pp_rank, vpp, n_mb)
        rows = t.micro_batch_size * m.seq_length
        if self.tpc.sp:
            rows //= topo.tp
        shape = (rows, m.hidden_size)
        caches = {}

        def needs_recv(kind, v):
            ch = self.chunks[v]
            return (kind == "F" and not ch.spec.has_embedding) or (kind == "B" and not ch.spec.has_head)

        def post(k):
            kind, v, _ = sched[k]
            if needs_recv(kind, v):
                return (self.links.post_recv_act if kind == "F" else self.links.post_recv_grad)(shape, self.dtype, self.device)
            return None
        # Receives may be posted one action ahead, so that the transfer runs under the current action's kernels.  Never
        # while CUDA graphs are still being captured: a capture begins with a device-wide synchronize, which would wait
        # for the posted receive, whose sender is a peer waiting in its own synchronize for THIS rank's next send.  The
        # look-ahead is the default on the CPU / gloo path; on NCCL it is opt-in (FORGE_PP_PREFETCH=1) and starts with the
        # first step after the one that captured the layer graphs.
        ahead = (self.device.type != "cuda") or (os.environ.get("FORGE_PP_PREFETCH", "0") == "1"
                                                 and (not self._layer_graphs or self._layer_graph_steps >= 1))
        posted = post(0) if sched else None
        for k, (kind, v, i) in enumerate(sched):
            nxt = post(k + 1) if (ahead and k + 1 < len(sched)) else None
            ch = self.chunks[v]
            if kind == "F":
                x_in = self.links.wait_recv(posted) if posted is not None else None
                out, cache = ch.forward(batches[i], x_in)
                caches[(v, i)] = cache
                if ch.spec.has_head:
                    self.stats += self._mb_stats(out, batches[i])
                else:
                    self.links.send_act(out)
            else:
                g_out = self.links.wait_recv(posted) if posted is not None else None
                g_in = ch.run_backward(batches[i], caches.pop((v, i)), g_out)
                if g_in is not None:
                    self.links.send_grad(g_in)
            posted = nxt if ahead else (post(k + 1) if k + 1 < len(sched) else None)
        self.links.drain()

    # ------------------------------------------------------------------
    def train_step(self, verify: bool = False) -> dict:
        """Runs one optimizer step.  Returns device tensors (no host sync): loss, grad_norm, tokens.  With ``verify`` the
        host waits for the step and raises if a kernel reported a wait that ran out (``verify_kernels``); callers that
        pipeline steps without a sync (the benchmark) call ``verify_kernels`` themselves at their own sync points."""
        topo = self.topo
        self.start_data()
        step_abs = self.step + 1
        if self.capture is not None:
            self.capture.begin_step(self.step)
        self.store.zero_grad()
        self.stats.zero_()
        if topo.pp == 1:
            self._run_microbatches_nopp()
        else:
            self._run_microbatches_pp()
        stats = self.stats
        if topo.world_size > 1:
            if not (topo.is_last_stage and topo.tp_rank == 0):
                stats = torch.zeros_like(stats)
            else:
                stats = stats.clone()
            if self.capture is not None:
                self.capture.loss_scalar("pre", stats)
            dist.all_reduce(stats)
        elif self.capture is not None:
            self.capture.loss_scalar("pre", stats)
        n_main = torch.clamp(stats[1], min=1.0)
        inv_tokens = (1.0 / n_main).to(torch.float32)
        loss = stats[0] / n_main
        if self.with_mtp:
            loss = loss + self.cfg.model.mtp_loss_weight * stats[2] / torch.clamp(stats[3], min=1.0)
        if self.capture is not None:
            self.capture.grads("pre", self.store)
        lr = compute_lr(step_abs, self.cfg.optim)
        norm = self.opt.step(lr, inv_tokens)
        self.weights_changed()
        if self.capture is not None:
            self.capture.grads("post", self.store, scale=inv_tokens)
            self.capture.loss_scalar("post", stats)
        self.step = step_abs
        if self._layer_graphs:
            self._layer_graph_steps += 1
        self._maybe_enable_layer_graphs()
        self.last = {"loss": loss, "grad_norm": norm, "tokens": stats[1], "lr": lr}
        if verify:
            self.verify_kernels()
        return self.last

    def paths(self) -> dict:
        """Which implementation of each communication / launch path this trainer runs (reported by the benchmark and the
        training log, so that a fallback to the library collectives is never silent)."""
        return {"ops": self.ops.name, "fused_dp": self.opt.fused is not None, "fused_tp": self.tpc.fused is not None,
                "cuda_graph": self._graph is not None or self._layer_graphs, "tp": self.topo.tp, "pp": self.topo.pp, "dp": self.topo.dp,
                "dp_buckets_overlapped_with_backward": getattr(self.opt.fused, "overlapped_total", 0) if self.opt.fused is not None
                else getattr(self.opt, "overlapped_buckets", 0), "dp_buckets": len(self.store.buckets)}

    def weights_changed(self):
        """Tell op tables that keep derived copies of the weights (the MXFP8 quantised ones) that the bf16 parameters moved."""
        hook = getattr(self.ops, "after_optimizer_step", None)
        if hook is not None:
            hook()

    # ------------------------------------------------------------------
    def data_state(self) -> dict:
        return self.prefetch.state_dict() if self.prefetch is not None else self.source.state_dict()

    def rng_state(self) -> dict:
        d = {"torch": torch.get_rng_state(), "numpy": np.random.get_state(), "python": random.getstate()}
        if self.device.type == "cuda":
            d["cuda"] = torch.cuda.get_rng_state(self.device)
        return d

    def set_rng_state(self, d: dict):
        torch.set_rng_state(d["torch"])
        np.random.set_state(d["numpy"])
        random.setstate(d["python"])
        if self.device.type == "cuda" and "cuda" in d:
            torch.cuda.set_rng_state(d["cuda"], self.device)

    def close(self):
        if self.prefetch is not None:
            self.prefetch.stop()
            self.prefetch = None


# ---------------------------------------------------------------------------

def _max_over_ranks(x: float, device) -> float:
    if dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])
    return x


def run_training_loop(cfg: RunConfig, *, trainer: Trainer | None = None, loss_tag: str | None = None,
                      teardown: bool = False, out=None) -> list[wire.LossRecord]:
    """Train ``cfg.train.num_steps`` steps.  Returns the per-step records rank 0 printed."""
    from .ckpt import manager as ckpt
    out = out or sys.stdout
    t0_wall = time.time()
    created = init_distributed()
    sess = None
    if trainer is None and cfg.train.hash_capture_level > 0 and cfg.train.hash_output:
        # hash capture asked for by the configuration (a gate product's hash_capture_level / hash_output): per-rank dumps
        # ``<hash_output>.rank<r>`` of the loss / gradient families (level 1) and of every module's output (level 2)
        from .gates.capture import CaptureSession
        sess = CaptureSession(cfg.train.hash_output, level=cfg.train.hash_capture_level, rank=dist.get_rank() if dist.is_initialized() else 0)
    tr = trainer or Trainer(cfg, init_mode=cfg.train.init_mode, capture=sess)
    t, oc, m = cfg.train, cfg.optim, cfg.model
    tag = loss_tag or t.loss_tag
    rank0 = tr.rank == 0
    if t.resume_from:
        ckpt.load(tr, t.resume_from, weights_only=t.init_weights_only)
        tr.weights_changed()
        if rank0:
            print(wire.format_resume_startup(time.time() - t0_wall), file=out, flush=True)
    if rank0:
        print(wire.format_phase_line(t.phase_name or "train", tr.step, oc.lr, oc.min_lr, oc.lr_warmup_iters,
                                     oc.lr_decay_iters, oc.lr_wsd_decay_iters, t.init_weights_only,
                                     cfg.data.data_path or cfg.data.data_loader), file=out, flush=True)
    cuda = tr.device.type == "cuda"
    peak = tr.peaks.get("bf16_tflops_sustained", tr.peaks["bf16_tflops"])
    tokens_per_step = t.micro_batch_size * m.seq_length * tr.grad_accum * tr.topo.dp
    records = []
    sink = open(t.metrics_jsonl, "a") if (t.metrics_jsonl and rank0) else None
    end_step = tr.step + t.num_steps
    from .utils.step_profile import StepProfiler
    prof = StepProfiler(tr.rank)   # FORGE_PROFILE_STEP=<n>: that step of one rank runs under the profiler
    while tr.step < end_step:
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        tw = time.perf_counter()
        with prof.maybe(tr.step + 1):
            res = tr.train_step()
        if cuda:
            e1.record()
            e1.synchronize()
            dt = e0.elapsed_time(e1) / 1e3
        else:
            dt = time.perf_counter() - tw
        # before the loss line is printed and before any checkpoint is written: a kernel whose wait ran out left wrong data
        tr.verify_kernels(sync=False)
        dt_max = _max_over_ranks(dt, tr.device)
        loss, gn = float(res["loss"]), float(res["grad_norm"])
        mfu = mfu_percent(tr.flops_per_token, tokens_per_step, dt_max, tr.world, peak)
        rec = wire.LossRecord(tag, tr.step, loss, gn, dt_max, mfu)
        records.append(rec)
        if rank0:
            print(wire.format_loss_line(tr.step, loss, gn, dt_max, mfu, tag,
                                        tokens_per_sec_per_gpu=tokens_per_step / dt_max / tr.world,
                                        step_time_max_ranks_s=dt_max), file=out, flush=True)
            if sink:
                import json
                sink.write(json.dumps({"step": tr.step, "loss": loss, "grad_norm": gn, "time_s": dt_max,
                                       "mfu": mfu, "lr": res["lr"]}) + "\n")
                sink.flush()
        if t.save_path and (tr.step == end_step or (t.save_interval and tr.step % t.save_interval == 0)):
            ckpt.save(tr, t.save_path)
    if sink:
        sink.close()
    if tr.capture is not None:
        tr.capture.dump()
    if trainer is None:
        tr.close()
    if teardown:
        ordered_teardown(created)
    return records


def ordered_teardown(destroy_pg: bool = True):
    """Drain the GPU, barrier, destroy the process group, free cached memory (train_loop.py:2689-2726)."""
    import gc
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    for _ in range(3):
        gc.collect()
    if dist.is_initialized():
        try:
            dist.barrier()
        finally:
            if destroy_pg:
                dist.destroy_process_group()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    print("ALL DONE", flush=True)
