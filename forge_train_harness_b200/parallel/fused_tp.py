"""Fused sequence-parallel TP paths: all-gather -> GEMM and GEMM -> reduce-scatter as single kernels over peer memory.

Buffers (symmetric over the TP group, allocated once):
  gather[2]   [M, H] bf16   a rank writes its own row shard into ITS buffer; ``ag_gemm``'s copy CTAs pull the other shards
                            from the peers' buffers into the local one while the GEMM CTAs already consume the local shard.
  shard[2]    [M/tp, H] bf16   row-parallel output shards; every rank TMA-reduce-adds its partial tiles into the owners'.
The two copies of each buffer alternate between consecutive calls, so ONE flag barrier per call is enough:
  ag_gemm:  write own shard -> barrier (all shards written; everyone finished the call before last that used this copy) -> kernel
  gemm_rs:  zero the NEXT copy -> kernel -> barrier (all adds landed; peers may now add into the next copy, already zero)
Roofline per call: max(FLOPs / measured GEMM peak, (tp-1)/tp * M*H*2 bytes / NVLink bandwidth).

Usable when the activation has H columns, M % (128 * tp) == 0 and tp <= 8; otherwise ``TPComm`` keeps the NCCL collectives.
"""
from __future__ import annotations

import sys

import torch

from .symm import PeerBarrier, symm_empty


class FusedTP:
    def __init__(self, group, tp: int, rank: int, M: int, H: int, device, n_copy_ctas: int = 0):
        self.tp, self.rank, self.M, self.H, self.Ms = tp, rank, M, H, M // tp
        self.gather = [symm_empty(M * H, torch.bfloat16, device, group) for _ in range(2)]
        self.shard = [symm_empty(self.Ms * H, torch.bfloat16, device, group) for _ in range(2)]
        for b in self.shard:
            b.tensor.zero_()
        self.flags = torch.zeros(M // 128, dtype=torch.int32, device=device)
        self.barrier = PeerBarrier(device, group)
        self.g_turn = self.s_turn = 0
        self.epoch = 0
        self.n_copy = n_copy_ctas

    def supports(self, rows: int, cols: int) -> bool:
        return cols == self.H and rows in (self.M, self.Ms)

    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, w_mn: bool, alpha: float = 1.0):
        """Returns ``(y [M, N_local], x_full [M, H])``."""
        from ..ops.cuda_ops import _C
        buf = self.gather[self.g_turn]
        self.g_turn ^= 1
        full = buf.tensor.view(self.M, self.H)
        full[self.rank * self.Ms:(self.rank + 1) * self.Ms].copy_(x_shard)
        self.barrier(0)
        self.epoch += 1
        y = _C.ag_gemm(buf.ptrs, self.M, self.H, w, w_mn, self.rank, self.n_copy, self.flags, self.epoch, float(alpha))
        return y, full.clone()

    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, w_mn: bool, alpha: float = 1.0) -> torch.Tensor:
        """``x [M, K_local]`` times the local weight slice, summed over ranks, rows scattered: returns ``[M/tp, H]``."""
        from ..ops.cuda_ops import _C
        cur = self.shard[self.s_turn]
        self.s_turn ^= 1
        self.shard[self.s_turn].tensor.zero_()  # the copy the NEXT call adds into
        _C.gemm_rs(x, w, w_mn, cur.ptrs, self.H, self.rank, float(alpha))
        self.barrier(1)
        return cur.tensor.view(self.Ms, self.H).clone()


def try_create(group, tp, rank, M, H, device):
    if tp < 2 or tp > 8 or M % (128 * tp) or H % 8:
        return None
    try:
        return FusedTP(group, tp, rank, M, H, device)
    except Exception as e:  # noqa: BLE001
        if rank == 0:
            print(f"[debug] fused TP path unavailable ({type(e).__name__}: {e}); using NCCL collectives", file=sys.stderr, flush=True)
        return None
