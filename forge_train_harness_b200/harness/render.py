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


def load_axes(root: str) -> dict:
    """``{"model": {name: table}, "optim": {...}, "data": {...}}`` from ``<root>/{model,optim,data}/<name>.toml`` — the axis
    directories a gate picks one file of each from (harness/config_runtime.py:191-234 validates the same three axes)."""
    import os
    out = {}
    for axis in ("model", "optim", "data"):
        d = os.path.join(root, axis)
        out[axis] = {}
        if not os.path.isdir(d):
            continue
        for fn in sorted(os.listdir(d)):
            if fn.endswith(".toml"):
                doc = load_toml(os.path.join(d, fn))
                if axis not in doc:
                    raise ValueError(f"{os.path.join(d, fn)} has no [{axis}] table")
                out[axis][fn[:-5]] = doc[axis]
    return out


RUNTIME = "<runtime>"


def resolve_deploy(product: dict, runtime_values: dict) -> dict:
    """Freeze-time fill of the ``<runtime>`` sentinels of a rendered product (tools/resolve_deploy.py): values only the
    execution host knows (data paths, checkpoint roots, ports).  Every sentinel must get a value; an unknown key in
    ``runtime_values`` is an error too, so a typo cannot silently leave a sentinel behind."""
    out = {t: dict(product.get(t, {})) for t in ("cli", "env")}
    used = set()
    for t in out:
        for k, v in out[t].items():
            if v == RUNTIME:
                key = k if k in runtime_values else k.lower() if k.lower() in runtime_values else k.upper()
                if key not in runtime_values:
                    raise KeyError(f"product key {k!r} is <runtime> and no value was given for it")
                out[t][k] = runtime_values[key]
                used.add(key)
    extra = set(runtime_values) - used
    if extra:
        raise KeyError(f"runtime values {sorted(extra)} match no <runtime> sentinel of the product")
    return out


def load_toml(path: str) -> dict:
    with open(path, "rb") as f:
        return tomllib.load(f)
