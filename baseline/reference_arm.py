"""Reference arm of ``bench.py``: the UNMODIFIED reference engine from ``baseline/_ref`` on the same shape."""
from __future__ import annotations

import json


def run_reference(a) -> None:
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired yet"}), flush=True)
