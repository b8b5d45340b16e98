"""Roofline denominators: measured on the deployment pool when a ``MEASURED_PEAKS.json`` is present.

The reference hard-codes the H100 figure 989.4e12 FLOP/s per GPU as its MFU denominator
(train_loop.py:89).  Here the denominator is the measured cuBLAS bf16 throughput of the B200 in use
(``bf16_tflops_sustained`` for a number timed inside a long training step), falling back to an
earlier measurement of the same part when the file is absent.
"""
from __future__ import annotations

import json
import os

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
NOMINAL_BF16_TFLOPS = 2250.0
H100_BF16_PEAK_FLOPS = 989.4e12


def load_peaks(path: str | None = None) -> dict:
    cands = [path] if path else []
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    cands += [os.environ.get("FORGE_MEASURED_PEAKS", ""), os.path.join(here, "MEASURED_PEAKS.json")]
    for c in cands:
        if c and os.path.isfile(c):
            with open(c) as f:
                d = json.load(f)
            d["source"] = "measured"
            return d
    return dict(FALLBACK)


def mfu_percent(flops_per_token: float, tokens: float, seconds: float, n_gpus: int, peak_tflops: float) -> float:
    """MFU on the reference's 0-100 scale."""
    if seconds <= 0:
        return 0.0
    return 100.0 * flops_per_token * tokens / (seconds * n_gpus * peak_tflops * 1e12)
