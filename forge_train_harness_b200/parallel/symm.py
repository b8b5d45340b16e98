"""Symmetric memory over NVLink: buffers every rank of a group maps at the same offsets.

Allocation and the handle exchange use ``torch.distributed._symmetric_memory`` (CUDA VMM allocations exported to the peers
of an NCCL group, optionally also bound to an NVSwitch multicast object).  Everything that touches the memory afterwards is
this package's own kernels (``csrc/comm_sm100.cu``): plain peer loads / stores, or ``multimem`` on the multicast mapping.
"""
from __future__ import annotations

import os

import torch


class SymmBuffer:
    def __init__(self, tensor, handle):
        self.tensor, self.handle = tensor, handle
        self.ptrs = [int(p) for p in handle.buffer_ptrs]
        mc = int(getattr(handle, "multicast_ptr", 0) or 0)
        self.mc_ptr = mc if os.environ.get("FORGE_MULTIMEM", "0") == "1" else 0
        self.rank, self.world = handle.rank, handle.world_size


def symm_empty(numel: int, dtype, device, group) -> SymmBuffer:
    import torch.distributed._symmetric_memory as sm
    t = sm.empty(numel, dtype=dtype, device=device)
    h = sm.rendezvous(t, group)
    return SymmBuffer(t, h)


class PeerBarrier:
    """Device-side flag barrier over a group (bounded wait; a timeout lands in the kernel status word)."""

    def __init__(self, device, group, lanes: int = 4, limit_s: float | None = None):
        # A training rank can legitimately be late by tens of seconds (first-step graph capture, a lazy build, a data
        # stall), so the training-path limit is long (host-side collective timeouts are 30 minutes); when it does run
        # out, the status word makes the step raise (``Trainer.verify_kernels``).  Tests pass short limits.
        if limit_s is None:
            limit_s = float(os.environ.get("FORGE_PEER_WAIT_S", "120"))
        self.buf = symm_empty(8 * lanes, torch.int32, device, group)
        self.buf.tensor.zero_()
        torch.cuda.synchronize()
        import torch.distributed as dist
        dist.barrier(group=group)  # every pad is zero before the first epoch is written
        self.epoch = [0] * lanes
        self.limit_s = limit_s
        # device-side epoch counters: with ``device_epochs`` the kernel numbers its own calls, so a captured CUDA graph
        # that contains barriers can be replayed (a host-side epoch would be frozen into the graph)
        self.epoch_dev = torch.zeros(lanes, dtype=torch.int32, device=device)
        self.device_epochs = False

    def __call__(self, lane: int = 0, device_epoch: bool | None = None):
        """``device_epoch`` overrides the object's default for this call; a lane must stick to one numbering."""
        from ..ops.cuda_ops import _C
        if self.device_epochs if device_epoch is None else device_epoch:
            _C.peer_barrier(self.buf.ptrs, self.buf.rank, 0, lane, self.limit_s, self.epoch_dev)
            return
        self.epoch[lane] += 1
        _C.peer_barrier(self.buf.ptrs, self.buf.rank, self.epoch[lane], lane, self.limit_s, None)
