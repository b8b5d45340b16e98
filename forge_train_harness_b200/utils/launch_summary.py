"""Turn a profiler launch list into a per-kernel summary with the change against a previous capture.

    python -m forge_train_harness_b200.utils.launch_summary launches.csv [--previous summary.json] [--skip-first-half]
        [--json summary.json] [--md summary.md]

The input is the CSV that ``ncu --metrics gpu__time_duration.sum --csv --log-file launches.csv <cmd>`` writes: one row per
launch with the kernel name and its device time.  The output groups launches by kernel (template arguments kept, call
arguments dropped), sorts by total time and, when ``--previous`` names the JSON of an earlier summary, adds the delta per
kernel, which is what one looks at after changing a kernel.  The reference does the same job from ``nsys stats`` output
(tools/profile_render.py: ``summary.md`` / ``profile.json`` with a delta-vs-previous column); this tree captures with ncu
because nsys is not part of the image.
"""
from __future__ import annotations

import argparse
import collections
import csv
import json
import re
import sys


def parse_launches(lines) -> list[tuple[str, float]]:
    """``[(kernel name, microseconds)]`` in launch order from ncu's CSV (profiler banner lines start with ``==``)."""
    rows = [ln for ln in lines if not ln.startswith("==")]
    out = []
    for r in csv.DictReader(rows):
        if r.get("Metric Name") != "gpu__time_duration.sum":
            continue
        v = float(r["Metric Value"].replace(",", ""))
        unit = (r.get("Metric Unit") or "").lower()
        us = v / 1e3 if unit in ("ns", "nsecond") else v * 1e3 if unit in ("ms", "msecond") else v * 1e6 if unit in ("s", "second") else v
        out.append((re.sub(r"\(.*", "", r["Kernel Name"]).strip(), us))
    return out


def summarise(launches: list[tuple[str, float]]) -> dict:
    agg: dict = collections.OrderedDict()
    for name, us in launches:
        a = agg.setdefault(name, {"launches": 0, "us": 0.0})
        a["launches"] += 1
        a["us"] += us
    total = sum(a["us"] for a in agg.values())
    kernels = [{"kernel": k, "launches": a["launches"], "us": round(a["us"], 2),
                "share": round(a["us"] / total, 4) if total else 0.0}
               for k, a in sorted(agg.items(), key=lambda kv: -kv[1]["us"])]
    return {"total_us": round(total, 2), "launches": len(launches), "kernels": kernels}


def with_delta(cur: dict, prev: dict | None) -> dict:
    if not prev:
        return cur
    old = {k["kernel"]: k for k in prev.get("kernels", [])}
    for k in cur["kernels"]:
        o = old.get(k["kernel"])
        k["delta_us"] = round(k["us"] - o["us"], 2) if o else None
    cur["delta_total_us"] = round(cur["total_us"] - prev.get("total_us", 0.0), 2)
    cur["gone"] = sorted(set(old) - {k["kernel"] for k in cur["kernels"]})
    return cur


def to_markdown(s: dict, top: int = 25) -> str:
    has_delta = any("delta_us" in k for k in s["kernels"])
    head = "| kernel | launches | us | share |" + (" delta us |" if has_delta else "")
    lines = [f"{s['launches']} launches, {s['total_us']:.1f} us"
             + (f" ({s['delta_total_us']:+.1f} us against the previous capture)" if "delta_total_us" in s else ""), "",
             head, "|---|---|---|---|" + ("---|" if has_delta else "")]
    for k in s["kernels"][:top]:
        row = f"| `{k['kernel'][:90]}` | {k['launches']} | {k['us']:.1f} | {100 * k['share']:.1f} % |"
        if has_delta:
            d = k.get("delta_us")
            row += (" new |" if d is None else f" {d:+.1f} |")
        lines.append(row)
    if s.get("gone"):
        lines += ["", "no longer launched: " + ", ".join(f"`{g[:60]}`" for g in s["gone"])]
    return "\n".join(lines) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("csv")
    ap.add_argument("--previous", default="")
    ap.add_argument("--skip-first-half", action="store_true", help="keep the second half of the launches (e.g. the second of two steps)")
    ap.add_argument("--json", default="")
    ap.add_argument("--md", default="")
    a = ap.parse_args(argv)
    with open(a.csv) as f:
        launches = parse_launches(f.readlines())
    if a.skip_first_half:
        launches = launches[len(launches) // 2:]
    prev = None
    if a.previous:
        with open(a.previous) as f:
            prev = json.load(f)
    s = with_delta(summarise(launches), prev)
    md = to_markdown(s)
    if a.json:
        with open(a.json, "w") as f:
            json.dump(s, f, indent=1)
    if a.md:
        with open(a.md, "w") as f:
            f.write(md)
    sys.stdout.write(md)
    return 0


if __name__ == "__main__":
    sys.exit(main())
