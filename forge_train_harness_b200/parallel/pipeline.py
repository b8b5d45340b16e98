"""Pipeline schedules (1F1B and interleaved 1F1B) as static action lists, plus the p2p plumbing.

The reference has no pipeline parallelism (``--pipeline-model-parallel-size 1`` in
ref/reference/train_minicpm4_0.5b_gsm8k.sh:310); the semantics here are Megatron's: model chunk
``v*pp + p`` lives on stage ``p``; the k-th forward "virtual micro-batch" of a rank maps to chunk
``(k // pp) % vpp`` and micro-batch ``(k // (pp*vpp))*pp + k % pp``; backward walks chunks in reverse;
a rank runs ``(pp - p - 1)*2 + (vpp - 1)*pp`` warm-up forwards (``pp - p - 1`` when ``vpp == 1``),
then one-forward-one-backward, then the remaining backwards.

Because the backward is hand-derived, a schedule is just a list of ``("F"|"B", chunk, microbatch)``.

Transport: activations and gradients travel by ``isend`` / ``irecv`` over NCCL (gloo on CPU) and are waited for on the stream
(the host does not block on NCCL).  A receive can be posted one schedule action ahead of its consumer, so that the transfer
overlaps the current action's compute (default on gloo, ``FORGE_PP_PREFETCH=1`` on NCCL; never during a CUDA-graph capture
step: see ``engine.py``).  Every
directed edge of the pipeline ring — activations p -> p+1 and gradients p+1 -> p — gets its OWN
two-rank process group, hence its own communicator and stream: a send that waits for its receiver
blocks only that edge, never the opposite direction, so the schedule needs no hand-paired
send/recv batching to stay deadlock-free, and transfers overlap with compute.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def build_schedule(pp: int, pp_rank: int, vpp: int, n_mb: int) -> list[tuple[str, int, int]]:
    if pp == 1 and vpp == 1:
        out = []
        for i in range(n_mb):
            out += [("F", 0, i), ("B", 0, i)]
        return out
    if vpp > 1 and n_mb % pp:
        raise ValueError("interleaved pipelining needs the number of micro-batches to be a multiple of pp")
    total = n_mb * vpp

    def fwd_of(k):
        return ((k // pp) % vpp, (k // (pp * vpp)) * pp + k % pp) if vpp > 1 else (0, k)

    def bwd_of(k):
        return (vpp - 1 - (k // pp) % vpp, (k // (pp * vpp)) * pp + k % pp) if vpp > 1 else (0, k)

    if vpp == 1:
        warm = min(pp - pp_rank - 1, total)
    elif n_mb == pp:
        warm = total
    else:
        warm = min((pp - pp_rank - 1) * 2 + (vpp - 1) * pp, total)
    acts = [("F",) + fwd_of(k) for k in range(warm)]
    for i in range(total - warm):
        acts.append(("F",) + fwd_of(warm + i))
        acts.append(("B",) + bwd_of(i))
    for i in range(total - warm, total):
        acts.append(("B",) + bwd_of(i))
    return acts


class PipeLinks:
    """The four directed p2p edges of one rank: activations from prev / to next, grads from next / to prev."""

    def __init__(self, topo):
        self.topo = topo
        self.fwd_to_next = self.fwd_from_prev = self.bwd_to_prev = self.bwd_from_next = None
        self._pending = []
        if topo.pp == 1:
            return
        # every rank creates every edge group, in the same order
        for d in range(topo.dp):
            for x in range(topo.tp):
                for p in range(topo.pp):
                    a, b = topo.rank_of(p, d, x), topo.rank_of((p + 1) % topo.pp, d, x)
                    if a == b:
                        continue
                    g_act = dist.new_group(sorted({a, b}))
                    g_grad = dist.new_group(sorted({a, b}))
                    if topo.rank == a:
                        self.fwd_to_next, self.bwd_from_next = g_act, g_grad
                    if topo.rank == b:
                        self.fwd_from_prev, self.bwd_to_prev = g_act, g_grad

    def send_act(self, t):
        self._pending.append((dist.isend(t, self.topo.next_stage_rank, group=self.fwd_to_next), t))

    def post_recv_act(self, shape, dtype, device):
        """Post the receive now, wait later (``wait_recv``): posting it one schedule action ahead lets the transfer run
        under the current action's kernels instead of starting when its consumer is about to be enqueued."""
        t = torch.empty(shape, dtype=dtype, device=device)
        return dist.irecv(t, self.topo.prev_stage_rank, group=self.fwd_from_prev), t

    def post_recv_grad(self, shape, dtype, device):
        t = torch.empty(shape, dtype=dtype, device=device)
        return dist.irecv(t, self.topo.next_stage_rank, group=self.bwd_from_next), t

    @staticmethod
    def wait_recv(posted):
        """With NCCL this makes the CURRENT STREAM wait for the transfer (the host does not block); with gloo it blocks."""
        work, t = posted
        work.wait()
        return t

    def recv_act(self, shape, dtype, device):
        return self.wait_recv(self.post_recv_act(shape, dtype, device))

    def send_grad(self, t):
        self._pending.append((dist.isend(t, self.topo.prev_stage_rank, group=self.bwd_to_prev), t))

    def recv_grad(self, shape, dtype, device):
        return self.wait_recv(self.post_recv_grad(shape, dtype, device))

    def drain(self):
        for w, _ in self._pending:
            w.wait()
        self._pending.clear()
