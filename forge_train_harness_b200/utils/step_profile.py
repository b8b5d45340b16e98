"""Profile ONE training step of one rank behind a single environment variable, and render a per-kernel summary.

    FORGE_PROFILE_STEP=5 [FORGE_PROFILE_RANK=0[,2,...]] [FORGE_PROFILE_DIR=profile_out] python -m forge_train_harness_b200.train ...
    python -m forge_train_harness_b200.utils.step_profile profile_out/step_5_rank0.json [--previous older.json] [--md out.md]

The reference wraps rank 0 of its launcher in ``nsys profile`` when ``HARNESS_NSYS`` is set (evals/scripts/launch_dp.py:35-56)
and renders ``nsys stats`` into a ``summary.md`` with a delta-vs-previous column (tools/profile_render.py:144-221, 381-404).
nsys is not part of this image; the same contract is kept with ``torch.profiler`` (CUPTI activity records): the chosen step
of the chosen rank runs under the profiler, every kernel's device time is summed by name, and the summary states how much
of the step the GPU was busy and how much it sat idle between kernels, which is the launch-bound signal.  A step that runs
under the profiler is slower than a plain one: its time is never a benchmark number.
"""
from __future__ import annotations

import argparse
import collections
import json
import os
import re
import sys


class StepProfiler:
    """Context manager factory used by the training loop: ``with prof.maybe(step):`` around ``train_step``."""

    def __init__(self, rank: int):
        self.step = int(os.environ.get("FORGE_PROFILE_STEP", "-1"))
        self.ranks_wanted = {int(r) for r in os.environ.get("FORGE_PROFILE_RANK", "0").split(",") if r.strip()}
        self.dir = os.environ.get("FORGE_PROFILE_DIR", "profile_out")
        self.rank = rank
        self.enabled = self.step >= 0 and rank in self.ranks_wanted

    def maybe(self, step_abs: int):
        if not self.enabled or step_abs != self.step:
            import contextlib
            return contextlib.nullcontext()
        return _Capture(self, step_abs)


class _Capture:
    def __init__(self, owner: StepProfiler, step: int):
        self.o, self.step = owner, step

    def __enter__(self):
        import torch
        from torch.profiler import ProfilerActivity, profile
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        self.p = profile(activities=acts)
        self.p.__enter__()
        return self

    def __exit__(self, *exc):
        import torch
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.p.__exit__(*exc)
        os.makedirs(self.o.dir, exist_ok=True)
        summary = summarise_events(self.p.events())
        summary["step"], summary["rank"] = self.step, self.o.rank
        path = os.path.join(self.o.dir, f"step_{self.step}_rank{self.o.rank}.json")
        with open(path, "w") as f:
            json.dump(summary, f, indent=1)
        with open(path[:-5] + ".md", "w") as f:
            f.write(render_md(summary, None))
        print(f"[profile] step {self.step} rank {self.o.rank}: {path}", file=sys.stderr, flush=True)
        return False


def _short(name: str) -> str:
    name = re.sub(r"\(.*", "", name).strip()
    return re.sub(r"^void\s+", "", name)


def summarise_events(events) -> dict:
    """Device kernels / copies only: ``{kernels: {name: {launches, us}}, busy_us, span_us, idle_us, n_launches}``.
    ``busy`` is the union of the device intervals (overlapping streams counted once), ``span`` first start to last end."""
    agg: dict = collections.OrderedDict()
    ivals = []
    for e in events:
        dt = getattr(e, "device_type", None)
        if dt is None or "CUDA" not in str(dt).upper():
            continue
        tr = getattr(e, "time_range", None)
        if tr is None:
            continue
        us = float(tr.end - tr.start)
        if us <= 0:
            continue
        a = agg.setdefault(_short(e.name), {"launches": 0, "us": 0.0})
        a["launches"] += 1
        a["us"] += us
        ivals.append((float(tr.start), float(tr.end)))
    return _finish(agg, ivals)


def _finish(agg, ivals) -> dict:
    ivals.sort()
    busy, cur_s, cur_e = 0.0, None, None
    for s, e in ivals:
        if cur_e is None or s > cur_e:
            if cur_e is not None:
                busy += cur_e - cur_s
            cur_s, cur_e = s, e
        else:
            cur_e = max(cur_e, e)
    if cur_e is not None:
        busy += cur_e - cur_s
    span = (max(e for _, e in ivals) - ivals[0][0]) if ivals else 0.0
    kernels = collections.OrderedDict(sorted(agg.items(), key=lambda kv: -kv[1]["us"]))
    return {"kernels": kernels, "busy_us": busy, "span_us": span, "idle_us": max(span - busy, 0.0),
            "n_launches": sum(a["launches"] for a in agg.values())}


def render_md(cur: dict, prev: dict | None, top: int = 40) -> str:
    total = sum(a["us"] for a in cur["kernels"].values()) or 1.0
    lines = [f"# Step profile (step {cur.get('step')}, rank {cur.get('rank')})", "",
             f"device span {cur['span_us'] / 1e3:.2f} ms, busy {cur['busy_us'] / 1e3:.2f} ms "
             f"({100.0 * cur['busy_us'] / max(cur['span_us'], 1e-9):.1f} %), idle between kernels {cur['idle_us'] / 1e3:.2f} ms, "
             f"{cur['n_launches']} device activities", ""]
    if prev is not None:
        lines.append(f"previous: span {prev['span_us'] / 1e3:.2f} ms, busy {prev['busy_us'] / 1e3:.2f} ms, "
                     f"idle {prev['idle_us'] / 1e3:.2f} ms")
        lines.append("")
    hdr = "| kernel | launches | total us | share |" + (" delta us |" if prev is not None else "")
    lines += [hdr, "|---|---|---|---|" + ("---|" if prev is not None else "")]
    for name, a in list(cur["kernels"].items())[:top]:
        row = f"| `{name[:110]}` | {a['launches']} | {a['us']:.0f} | {100.0 * a['us'] / total:.1f} % |"
        if prev is not None:
            p = prev["kernels"].get(name)
            row += f" {a['us'] - p['us']:+.0f} |" if p else " new |"
        lines.append(row)
    if prev is not None:
        gone = [n for n in prev["kernels"] if n not in cur["kernels"]]
        if gone:
            lines += ["", "no longer launched: " + ", ".join(f"`{n[:60]}`" for n in gone[:20])]
    return "\n".join(lines) + "\n"


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("summary")
    ap.add_argument("--previous", default="")
    ap.add_argument("--md", default="")
    ap.add_argument("--top", type=int, default=40)
    a = ap.parse_args(argv)
    cur = json.load(open(a.summary), object_pairs_hook=collections.OrderedDict)
    prev = json.load(open(a.previous), object_pairs_hook=collections.OrderedDict) if a.previous else None
    md = render_md(cur, prev, a.top)
    if a.md:
        with open(a.md, "w") as f:
            f.write(md)
    print(md)


if __name__ == "__main__":
    main()
