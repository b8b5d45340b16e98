"""Render a per-gate single-source TOML into the two self-contained products (reference side / this engine's side).

Rules of the reference's renderer (tools/render_gate_configs.py:1-33, 68-81): seed a flat dict from the model and optim
axis tables plus the registry's global ``[env]``; overlay ``[shared]``, ``[shared.gate]``, ``[optim]``, ``[model]`` and then
the side table (``[ref]`` or ``[ours]``) low -> high, a ``_override`` suffix being only an authoring marker for "this
overwrites a lower layer"; drop every key whose value is the tombstone ``"@unset"``; derive ``grad_accum_steps =
global_batch_size // (micro_batch_size * world_size)`` and ``NUM_PROCS = world_size``; strip review-only keys; split by
transport — a bare name listed (upper-cased) in the registry's global ``[env]`` travels as ``[env]`` UPPERCASE, everything
else as ``[cli]``.  ``product_env`` turns a product into ``export KEY=value`` lines (tools/product_env.py).
"""
from __future__ import annotations

import tomllib

REVIEW_ONLY_KEYS = {"review_mfu_target", "mfu_elastic_tolerance", "mfu_elastic_rounds", "mfu_elastic_eps", "mfu_full_every_smokes"}
UNSET = "@unset"


def _overlay(dst: dict, table: dict) -> None:
    for k, v in table.items():
        if isinstance(v, dict):
            continue
        dst[k[:-9] if k.endswith("_override") else k] = v


def render_gate(gate_doc: dict, model: dict, optim: dict, global_env: dict, seed: int = 1234) -> dict:
    """Returns ``{"ref": {"cli": {...}, "env": {...}}, "ours": {...}}``."""
    env_names = {k.lower() for k in global_env}
    out = {}
    for side in ("ref", "ours"):
        flat: dict = {}
        flat.update(model)
        flat.update(optim)
        flat["seed"] = seed
        flat.update({k.lower(): v for k, v in global_env.items()})
        shared = gate_doc.get("shared", {})
        _overlay(flat, shared)
        _overlay(flat, shared.get("gate", {}))
        _overlay(flat, gate_doc.get("optim", {}))
        _overlay(flat, gate_doc.get("model", {}))
        _overlay(flat, gate_doc.get(side, {}))
        flat = {k: v for k, v in flat.items() if v != UNSET and k not in REVIEW_ONLY_KEYS}
        ws = int(flat.get("world_size", 1))
        if "global_batch_size" in flat and "micro_batch_size" in flat:
            denom = int(flat["micro_batch_size"]) * ws
            if int(flat["global_batch_size"]) % denom:
                raise ValueError("global_batch_size must be a multiple of micro_batch_size * world_size")
            flat["grad_accum_steps"] = int(flat["global_batch_size"]) // denom
        flat["num_procs"] = ws
        env_names_side = env_names | {"num_procs"}
        out[side] = {"cli": {k: v for k, v in flat.items() if k not in env_names_side},
                     "env": {k.upper(): v for k, v in flat.items() if k in env_names_side}}
    return out


def dumps_product(prod: dict) -> str:
    def val(v):
        if isinstance(v, bool):
            return "true" if v else "false"
        if isinstance(v, (int, float)):
            return repr(v)
        if isinstance(v, list):
            return "[" + ", ".join(val(x) for x in v) + "]"
        return '"' + str(v).replace("\\", "\\\\").replace('"', '\\"') + '"'
    lines = []
    for table in ("cli", "env"):
        lines.append(f"[{table}]")
        lines += [f"{k} = {val(v)}" for k, v in prod[table].items()]
        lines.append("")
    return "\n".join(lines)


def product_env(prod: dict, port_allocator=None) -> list[str]:
    """``export`` lines: bool -> 1/0, list -> space-joined, ``<runtime>`` skipped, ``<auto-port>`` allocated."""
    lines = []
    for table in ("cli", "env"):
        for k, v in prod.get(table, {}).items():
            if v == "<runtime>":
                continue
            if v == "<auto-port>":
                v = port_allocator() if port_allocator else 29500
            if isinstance(v, bool):
                v = int(v)
            if isinstance(v, list):
                v = " ".join(str(x) for x in v)
            lines.append(f"export {k.upper()}='{v}'")
    return lines


def load_toml(path: str) -> dict:
    with open(path, "rb") as f:
        return tomllib.load(f)
