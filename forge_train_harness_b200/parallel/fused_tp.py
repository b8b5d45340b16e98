"""Fused sequence-parallel TP paths: all-gather -> GEMM and GEMM -> reduce-scatter as single kernels over peer memory.

Buffers (symmetric over the TP group):
  gather     [M, H] bf16   a rank's own row shard is written into ITS buffer (by the producing kernel directly, or by a copy);
                           ``ag_gemm``'s copy CTAs pull the other shards from the peers' buffers into the local one while the
                           GEMM CTAs already consume the local shard.  Two kinds:
                             * one DEDICATED buffer per call site (``key``) for activations the backward pass keeps (the
                               gathered normed inputs of QKV / FC1): the gathered buffer IS the cached tensor, nothing is
                               cloned, and the buffer is not touched again before the same site's next micro-batch;
                             * a PAIR of transient buffers, alternating, for gathers consumed at once (backward-time
                               gathers of the output gradients).
  shard[2]   [M/tp, H] bf16   row-parallel output shards; every rank TMA-reduce-adds its partial tiles into the owners'.
                              The returned shard is valid until the next ``gemm_rs`` call but one (it is then zeroed for
                              reuse); the layer code consumes it in the very next kernel.

Ordering between ranks.  ``ag_gemm`` is self-sequenced: a device counter numbers the calls, each kernel announces "my shard
for call n is in place" to the peers with a release store, and a copy CTA waits (bounded) for a peer's announcement before it
pulls from that peer, so no barrier launch precedes the kernel and the local tiles start immediately.  A buffer is safe to
rewrite because a rank starts call n + 1 only after its own call n finished, and call n finishes only after every peer
announced call n, i.e. after every peer finished call n - 1: with two alternating buffers (or a dedicated one, reused a whole
micro-batch later) no peer can still be reading what is being overwritten.  ``gemm_rs`` zeroes the NEXT shard copy, runs the
kernel, then one flag barrier (all adds landed; peers may now add into the next copy, already zero).
Roofline per call: max(FLOPs / measured GEMM peak, (tp-1)/tp * M*H*2 bytes / NVLink bandwidth).

Usable when the activation has H columns, M % (128 * tp) == 0 and tp <= 8; otherwise ``TPComm`` keeps the NCCL collectives.
"""
from __future__ import annotations

import sys

import torch

from .symm import PeerBarrier, symm_empty


class FusedTP:
    def __init__(self, group, tp: int, rank: int, M: int, H: int, device, n_copy_ctas: int = 0):
        self.group, self.device = group, device
        self.tp, self.rank, self.M, self.H, self.Ms = tp, rank, M, H, M // tp
        self.transient = [symm_empty(M * H, torch.bfloat16, device, group) for _ in range(2)]
        self.sites: dict = {}
        self.shard = [symm_empty(self.Ms * H, torch.bfloat16, device, group) for _ in range(2)]
        for b in self.shard:
            b.tensor.zero_()
        self.flags = torch.zeros(M // 128, dtype=torch.int32, device=device)
        self.ctr = torch.zeros(2, dtype=torch.int32, device=device)       # {calls completed, CTAs done}: device-sequenced
        self.ready = symm_empty(8, torch.int32, device, group)            # ready[q]: last call rank q's shard is in place for
        self.ready.tensor.zero_()
        self.barrier = PeerBarrier(device, group)                          # also orders the zeroing above before any use
        self.barrier.device_epochs = True   # the barrier numbers its own calls: the layer code can be replayed from CUDA graphs
        self.g_turn = self.s_turn = 0
        self.n_copy = n_copy_ctas
        self.calls = {"ag_gemm": 0, "gemm_rs": 0, "copy_in": 0}

    def supports(self, rows: int, cols: int) -> bool:
        return cols == self.H and rows in (self.M, self.Ms)

    # -- gather buffers --------------------------------------------------------------------------------------------------
    def _site(self, key):
        buf = self.sites.get(key)
        if buf is None:
            # collective over the TP group: every rank reaches the same call sites in the same order
            buf = symm_empty(self.M * self.H, torch.bfloat16, self.device, self.group)
            self.sites[key] = buf
        return buf

    def _own_rows(self, buf):
        return buf.tensor.view(self.M, self.H)[self.rank * self.Ms:(self.rank + 1) * self.Ms]

    def slot(self, key) -> torch.Tensor:
        """This rank's rows ``[M/tp, H]`` of the dedicated gather buffer of call site ``key``: a producing kernel that
        writes its output here saves the copy-in of the following ``ag_gemm(..., key=key)``."""
        return self._own_rows(self._site(key))

    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, w_mn: bool, alpha: float = 1.0, key=None):
        """Returns ``(y [M, N_local], x_full [M, H])``; ``x_full`` is the gather buffer itself (see the module docstring
        for how long it stays valid)."""
        from ..ops.cuda_ops import _C
        if key is None:
            buf = self.transient[self.g_turn]
            self.g_turn ^= 1
        else:
            buf = self._site(key)
        own = self._own_rows(buf)
        if x_shard.data_ptr() != own.data_ptr():
            own.copy_(x_shard)
            self.calls["copy_in"] += 1
        self.calls["ag_gemm"] += 1
        y = _C.ag_gemm(buf.ptrs, self.M, self.H, w, w_mn, self.rank, self.n_copy, self.flags, 0, float(alpha), self.ctr,
                       self.ready.ptrs)
        return y, buf.tensor.view(self.M, self.H)

    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, w_mn: bool, alpha: float = 1.0) -> torch.Tensor:
        """``x [M, K_local]`` times the local weight slice, summed over ranks, rows scattered: returns ``[M/tp, H]``."""
        from ..ops.cuda_ops import _C
        cur = self.shard[self.s_turn]
        self.s_turn ^= 1
        self.shard[self.s_turn].tensor.zero_()  # the copy the NEXT call adds into
        self.calls["gemm_rs"] += 1
        _C.gemm_rs(x, w, w_mn, cur.ptrs, self.H, self.rank, float(alpha))
        self.barrier(1)
        return cur.tensor.view(self.Ms, self.H)


def try_create(group, tp, rank, M, H, device, required: bool = False):
    """A ``FusedTP`` or None (then ``TPComm`` keeps the NCCL collectives).  The reason is always printed by rank 0; with
    ``required`` (``FORGE_FUSED_TP=require``) a failure raises instead."""
    if tp < 2 or tp > 8 or M % (128 * tp) or H % 8:
        if required:
            raise RuntimeError(f"fused TP path needs 2 <= tp <= 8, M % (128 tp) == 0, H % 8 == 0 (tp={tp}, M={M}, H={H})")
        return None
    try:
        return FusedTP(group, tp, rank, M, H, device)
    except Exception as e:  # noqa: BLE001
        if required:
            raise
        if rank == 0:
            print(f"[warn] fused TP path unavailable ({type(e).__name__}: {e}); using NCCL collectives", file=sys.stderr, flush=True)
        return None
