"""Tensor / sequence-parallel communication around column- and row-parallel linears.

Without sequence parallelism these are the conjugate pair of the hand-written TP reference:
identity forward / all-reduce backward on a column-parallel input (``_CopyToTP``,
ref/reference/model_minicpm4_8b_tp.py:188-206) and all-reduce forward / identity backward on
a row-parallel output (``_ReduceFromTP``, :209-227).  With sequence parallelism (Megatron
semantics; the reference has no code for it) the residual stream is sharded by rows:
all-gather before a column-parallel GEMM, reduce-scatter after a row-parallel GEMM, and the
transposed collectives in backward.

This class is the library-collective implementation (NCCL on GPU, gloo on CPU).  The fused
sm_100a kernels that overlap the same transfers with the GEMM tiles plug in through
``ops.ag_linear_fwd`` / ``ops.linear_rs_fwd`` and are selected by the engine when available.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class TPComm:
    def __init__(self, group=None, size: int = 1, rank: int = 0, sequence_parallel: bool = False):
        self.group, self.size, self.rank = group, size, rank
        self.sp = bool(sequence_parallel and size > 1)
        self.fused = None  # a parallel.fused_tp.FusedTP when the one-kernel paths are available

    # -- linear + collective pairs (the places the fused kernels plug in) -----------------------
    def _fusable(self, x, w):
        f = self.fused
        return f is not None and self.sp and x.dtype == torch.bfloat16 and x.is_cuda

    def col_slot(self, key, rows: int, cols: int, dtype):
        """Where the producer of a column-parallel linear's input may write its ``[rows, cols]`` output directly (this
        rank's rows of the call site's all-gather buffer), or None when the one-kernel path is not in use."""
        f = self.fused
        if f is None or not self.sp or key is None or dtype != torch.bfloat16 or not f.supports(rows * self.size, cols):
            return None
        return f.slot(key)

    def col_linear_fwd(self, ops, x, w, alpha=1.0, key=None):
        """Column-parallel forward: ``(y, x_full)`` with ``y = gather(x) @ w^T``.  ``key`` names the call site (layer,
        linear, in-flight micro-batch slot) whose gathered input the backward pass keeps."""
        if self._fusable(x, w) and self.fused.supports(x.shape[0] * self.size, x.shape[1]):
            return self.fused.ag_gemm(x, w, False, alpha, key=key)
        xf = self.col_input_fwd(x)
        return ops.linear_fwd(xf, w, alpha), xf

    def row_linear_fwd(self, ops, x, w, alpha=1.0):
        """Row-parallel forward: ``reduce_scatter(x @ w^T)`` (all-reduce without sequence parallelism)."""
        if self._fusable(x, w) and self.fused.supports(x.shape[0], w.shape[0]):
            return self.fused.gemm_rs(x, w, False, alpha)
        return self.row_output_fwd(ops.linear_fwd(x, w, alpha))

    def row_linear_dgrad(self, ops, dy, w, alpha=1.0):
        """Backward of a row-parallel linear w.r.t. its input: ``(dx, dy_full)`` with ``dx = gather(dy) @ w``."""
        if self._fusable(dy, w) and self.fused.supports(dy.shape[0] * self.size, dy.shape[1]):
            return self.fused.ag_gemm(dy, w, True, alpha)
        dyf = self.row_output_bwd(dy)
        return ops.linear_dgrad(dyf, w, alpha), dyf

    def col_linear_dgrad(self, ops, dy, w, alpha=1.0):
        """Backward of a column-parallel linear w.r.t. its input: ``reduce_scatter(dy @ w)``."""
        if self._fusable(dy, w) and self.fused.supports(dy.shape[0], w.shape[1]):
            return self.fused.gemm_rs(dy, w, True, alpha)
        return self.col_input_bwd(ops.linear_dgrad(dy, w, alpha))

    # -- primitives ------------------------------------------------------------
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            dist.all_reduce(x, group=self.group)
        return x

    def gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        out = torch.empty((x.shape[0] * self.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        out = torch.empty((x.shape[0] // self.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        if x.device.type == "cpu":  # gloo has no reduce_scatter_tensor
            tmp = x.clone()
            dist.all_reduce(tmp, group=self.group)
            n = out.shape[0]
            out.copy_(tmp[self.rank * n:(self.rank + 1) * n])
        else:
            dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
        return out

    # -- composed: what a layer calls --------------------------------------------
    def col_input_fwd(self, x):
        return self.gather_rows(x) if self.sp else x

    def col_input_bwd(self, dx):
        if self.size == 1:
            return dx
        return self.reduce_scatter_rows(dx) if self.sp else self.all_reduce(dx)

    def row_output_fwd(self, y):
        if self.size == 1:
            return y
        return self.reduce_scatter_rows(y) if self.sp else self.all_reduce(y)

    def row_output_bwd(self, dy):
        return self.gather_rows(dy) if self.sp else dy

    def shard_rows_of(self, x):
        """The rows of a replicated ``[M, ...]`` tensor this rank owns under sequence parallelism."""
        if not self.sp:
            return x
        n = x.shape[0] // self.size
        return x[self.rank * n:(self.rank + 1) * n]
