"""Op registry with a per-op version router.

Every engine op exists in two versions: ``baseline`` (plain PyTorch, ``torch_ops.TorchOps``; the
oracle and the CPU path) and ``sm100`` (hand-written sm_100a CUDA, ``cuda_ops.Sm100Ops``).  The
environment variable ``OP_<NAME>`` (upper-cased op name, e.g. ``OP_ATTENTION_FWD=baseline``) picks a
version per op; the default on a CUDA device is ``sm100`` for every op the extension provides.  This
mirrors the reference's per-operator router, which resolves ``OP_<NAME>`` -> registry default ->
``"baseline"`` so exactly one op can be swapped for an A/B run (tools/stage2_op_router.py:57-101).

On a CUDA device the extension is REQUIRED: if it cannot be loaded the import error propagates instead
of silently training on library kernels (set ``FORGE_ALLOW_BASELINE=1`` to opt in to the PyTorch path).
"""
from __future__ import annotations

import os

from .torch_ops import TorchOps, rope_table

OP_NAMES = [
    "embedding_fwd", "embedding_bwd", "rmsnorm_fwd", "residual_rmsnorm_fwd", "residual_add", "rmsnorm_bwd",
    "linear_fwd", "linear_dgrad", "linear_wgrad", "rope_fwd_", "rope_bwd_", "qk_norm_fwd", "qk_norm_bwd",
    "attention_fwd", "attention_bwd", "attention_rope_bwd", "swiglu_fwd", "swiglu_bwd", "cross_entropy_fwd_bwd", "adamw_segments", "sumsq",
]


def op_version(name: str, default: str) -> str:
    return os.environ.get("OP_" + name.upper().rstrip("_"), default)


class RoutedOps:
    """Binds each op name to the chosen implementation once, at construction."""

    def __init__(self, impls: dict, default: str):
        self.versions = {}
        for n in OP_NAMES:
            ver = op_version(n, default)
            impl = impls.get(ver)
            if impl is None or not hasattr(impl, n):
                if ver != "baseline" and default == ver and hasattr(impls["baseline"], n):
                    ver, impl = "baseline", impls["baseline"]  # op not provided by the extension
                else:
                    raise KeyError(f"op {n!r} has no version {ver!r}")
            setattr(self, n, getattr(impl, n))
            self.versions[n] = ver
        self.name = default
        self._impls = impls
        # not a versioned op: the debug input check of whichever implementation runs the model
        self.check_ids = getattr(impls.get(default), "check_ids", TorchOps.check_ids)

    def set_deterministic(self, on: bool) -> None:
        """Forwarded to every implementation that has a deterministic mode (fixed summation orders instead of atomics)."""
        for impl in self._impls.values():
            f = getattr(impl, "set_deterministic", None)
            if f is not None:
                f(on)


def get_ops(device="cpu"):
    import torch
    dev = torch.device(device)
    impls = {"baseline": TorchOps}
    if dev.type != "cuda":
        return RoutedOps(impls, "baseline")
    if os.environ.get("FORGE_ALLOW_BASELINE") == "1" and os.environ.get("FORGE_FORCE_BASELINE") == "1":
        return RoutedOps(impls, "baseline")
    from . import cuda_ops  # raises if the sm_100a extension is missing
    impls["sm100"] = cuda_ops.Sm100Ops
    return RoutedOps(impls, "sm100")


__all__ = ["TorchOps", "RoutedOps", "get_ops", "rope_table", "OP_NAMES", "op_version"]
