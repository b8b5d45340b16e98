"""Stdout wire protocol: ``[LOSS]`` / ``[LOSS_REF]`` / ``[LOSS_RES]`` / ``[PHASE]`` / ``[RESUME_STARTUP]`` lines.

Grammar and float format (``.9e``, an fp32 round trip) follow harness/wire_format.py:94-131 and the
emitters at train_loop.py:2507-2515, 1818-1829, evals/resume_startup_gate.py:119-135.  Extra
``key=value`` fields may follow the parsed prefix; parsers ignore them (wire_format.py:107-111).
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass

LOSS_FLOAT_FORMAT = ".9e"
_FLOAT = r"[-+]?(?:\d+\.?\d*(?:[eE][-+]?\d+)?|nan|inf)"
_LOSS_RE = re.compile(
    r"^\[(?P<tag>LOSS|LOSS_REF|LOSS_RES)\]\s+step=(?P<step>\d+)\s+global_loss=(?P<loss>" + _FLOAT +
    r")\s+grad_norm=(?P<gn>" + _FLOAT + r")(?:\s+time_s=(?P<t>" + _FLOAT + r"))?(?:\s+mfu_e2e_standard=(?P<mfu>" +
    _FLOAT + r"))?(?P<rest>.*)$", re.IGNORECASE)
_MEGATRON_RE = re.compile(r"iteration\s+(\d+)\s*/.*?lm loss:\s*(" + _FLOAT + r").*?grad norm:\s*(" + _FLOAT + ")", re.I)
_PHASE_RE = re.compile(r"^\[PHASE\]\s+(?P<body>.*)$")
_KV_RE = re.compile(r"(\w+)=(\S+)")


@dataclass(frozen=True)
class LossRecord:
    tag: str
    step: int
    loss: float
    grad_norm: float
    time_s: float | None = None
    mfu: float | None = None
    extra: dict | None = None


def format_loss_line(step: int, loss: float, grad_norm: float, time_s: float, mfu: float, tag: str = "LOSS",
                     **extra) -> str:
    line = (f"[{tag}] step={step} global_loss={loss:{LOSS_FLOAT_FORMAT}} grad_norm={grad_norm:{LOSS_FLOAT_FORMAT}} "
            f"time_s={time_s:.6f} mfu_e2e_standard={mfu:.6f}")
    for k, v in extra.items():
        line += f" {k}={v:.6f}" if isinstance(v, float) else f" {k}={v}"
    return line


def parse_loss_line(line: str, strict: bool = True) -> LossRecord | None:
    m = _LOSS_RE.match(line.strip())
    if not m:
        return None
    loss, gn = float(m["loss"]), float(m["gn"])
    if strict and not (math.isfinite(loss) and math.isfinite(gn)):
        raise ValueError(f"non-finite value in wire line: {line.strip()}")
    extra = {k: v for k, v in _KV_RE.findall(m["rest"] or "")}
    return LossRecord(m["tag"].upper(), int(m["step"]), loss, gn, float(m["t"]) if m["t"] else None,
                      float(m["mfu"]) if m["mfu"] else None, extra)


def parse_loss_lines(text: str, tag: str = "LOSS", strict: bool = True, megatron_fallback: bool = False) -> list[LossRecord]:
    out = []
    for ln in text.splitlines():
        r = parse_loss_line(ln, strict) if ln.lstrip().startswith("[") else None
        if r is not None and r.tag == tag:
            out.append(r)
    if not out and megatron_fallback:
        for ln in text.splitlines():
            m = _MEGATRON_RE.search(ln)
            if m:
                out.append(LossRecord(tag, int(m[1]), float(m[2]), float(m[3])))
    return out


def format_phase_line(name, start_step, lr, min_lr, warmup, decay, wsd_decay, init_weights_only, data_path) -> str:
    return (f"[PHASE] name={name} start_step={start_step} lr={lr} min_lr={min_lr} warmup={warmup} decay={decay} "
            f"wsd_decay={wsd_decay} init_weights_only={int(bool(init_weights_only))} data_path={data_path}")


def parse_phase_line(line: str) -> dict | None:
    m = _PHASE_RE.match(line.strip())
    return dict(_KV_RE.findall(m["body"])) if m else None


def format_resume_startup(seconds: float) -> str:
    return f"[RESUME_STARTUP] seconds={seconds:.3f}"
