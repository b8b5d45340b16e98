"""Error statistics for kernel tests: not only the worst element but the distribution and its SIGN.

A max-norm bound hides a kernel that is slightly wrong everywhere in the same direction (a dropped rounding term, a biased
accumulation), which is what compounds over a long training run.  ``err_stats`` reports, against an fp64 (or fp32) oracle,
the mean, 95th percentile and maximum of |error| and the signed mean, all relative to the oracle's RMS so that entries near
zero do not blow the ratio up; ``assert_close_stats`` bounds all four.  This is the per-op contract of the reference's
operator workflow (prompt/develop_prompt/_shared/stage2-subagent-playbook.md:63-93: signed mean, +/- ratio, p95).
"""
import torch


def err_stats(got: torch.Tensor, ref: torch.Tensor) -> dict:
    g, r = got.detach().double().reshape(-1), ref.detach().double().reshape(-1)
    rms = float(r.pow(2).mean().sqrt()) or 1.0
    e = (g - r) / rms
    a = e.abs()
    n = a.numel()
    if n > 4_000_000:  # quantile on a strided sample; mean / max / sign on everything
        samp = a[:: n // 2_000_000]
    else:
        samp = a
    pos, neg = int((e > 0).sum()), int((e < 0).sum())
    return {"mean": float(a.mean()), "p95": float(torch.quantile(samp.float(), 0.95)), "max": float(a.max()),
            "signed_mean": float(e.mean()), "pos_neg_ratio": pos / max(neg, 1), "rms_ref": rms, "n": n}


def assert_close_stats(got, ref, *, mean, p95, mx, bias=None, what=""):
    """Bounds are relative to the oracle's RMS.  ``bias`` bounds |signed mean| (default: a quarter of ``mean``, i.e. the
    errors must mostly cancel)."""
    s = err_stats(got, ref)
    bias = mean * 0.25 if bias is None else bias
    msg = f"{what} error stats {s}"
    assert s["mean"] <= mean, msg
    assert s["p95"] <= p95, msg
    assert s["max"] <= mx, msg
    assert abs(s["signed_mean"]) <= bias, msg
    return s


def padded(shape, dtype, pad_rows=3, pad_cols=8, sentinel=-777.0):
    """A tensor of ``shape`` that is a VIEW into a larger buffer filled with a sentinel: a kernel that writes outside its
    output (a tile that is not clipped at a ragged edge) changes the sentinel.  Returns ``(view, check)``."""
    R, C = shape
    big = torch.full((R + 2 * pad_rows, C + 2 * pad_cols), sentinel, device="cuda", dtype=dtype)
    view = big[pad_rows:pad_rows + R, pad_cols:pad_cols + C]

    def check():
        b = big.clone()
        b[pad_rows:pad_rows + R, pad_cols:pad_cols + C] = sentinel
        assert bool((b == sentinel).all()), "a kernel wrote outside its output tensor"
    return view, check
