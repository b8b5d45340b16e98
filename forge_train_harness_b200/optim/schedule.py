"""Learning-rate schedules, evaluated at the 1-indexed step (train_loop.py:2450-2453)."""
from __future__ import annotations

import math


def wsd_lr(step: int, max_lr: float, min_lr: float, warmup: int, decay: int, wsd_decay: int) -> float:
    """Warmup -> stable plateau -> exponential-style anneal ``min + (2 * 0.5**r - 1) * (max - min)``
    over the last ``wsd_decay`` steps before ``decay`` -> ``min_lr`` (train_loop.py:173-186)."""
    if step < warmup:
        return max_lr * step / warmup
    if step > decay:
        return min_lr
    start = decay - wsd_decay
    if step <= start:
        return max_lr
    ratio = float(step - start) / float(wsd_decay)
    return min_lr + (2.0 * math.pow(0.5, ratio) - 1.0) * (max_lr - min_lr)


def cosine_lr(step: int, max_lr: float, min_lr: float, warmup: int, decay: int) -> float:
    if warmup and step < warmup:
        return max_lr * step / warmup
    if decay <= warmup or step >= decay:
        return min_lr if decay > 0 else max_lr
    t = (step - warmup) / float(decay - warmup)
    return min_lr + 0.5 * (1.0 + math.cos(math.pi * t)) * (max_lr - min_lr)


def compute_lr(step: int, oc) -> float:
    """``oc`` is an ``OptimConfig``.  ``lr_decay_iters == 0`` with the WSD schedule means "never decay"."""
    if oc.lr_schedule == "constant":
        return oc.lr
    if oc.lr_schedule == "cosine":
        return cosine_lr(step, oc.lr, oc.min_lr, oc.lr_warmup_iters, oc.lr_decay_iters)
    decay = oc.lr_decay_iters if oc.lr_decay_iters > 0 else 1 << 62
    return wsd_lr(step, oc.lr, oc.min_lr, oc.lr_warmup_iters, decay, oc.lr_wsd_decay_iters)
