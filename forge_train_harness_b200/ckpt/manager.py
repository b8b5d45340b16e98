"""Checkpoint save / load / reshard.

Two on-disk formats:

* ``megatron_dist`` (default) — Megatron-style directory layout with a DISTRIBUTED payload:

      <root>/latest_checkpointed_iteration.txt
      <root>/iter_<N:07d>/metadata.json
      <root>/iter_<N:07d>/mp_rank_<tp:02d>[_<pp:03d>]/model_optim_rng.pt      written by DP rank 0 of the model-parallel rank
      <root>/iter_<N:07d>/mp_rank_<tp:02d>[_<pp:03d>]/distrib_optim_dp<d:03d>.pt   written by EVERY DP rank (ZeRO-1 shard)
      <root>/iter_<N:07d>/mp_rank_<tp:02d>[_<pp:03d>]/layout.json

  ``model_optim_rng.pt`` holds the local TP shard of every weight under its FQN (compute dtype), the step, the optimizer step
  counter and the data cursor.  ``distrib_optim_dp<d>.pt`` holds that DP rank's OWN slice of the fp32 master / exp_avg /
  exp_avg_sq (nothing is gathered: a rank writes what it has), its slice table, its RNG states and its data cursor.
  ``metadata.json`` records the parallel layout and, per model-parallel rank, the flat offset / size / local shape of every
  tensor and the bucket table, so a loader at ANY other TP x PP x DP layout can work out which slices of which files hold the
  rows it needs and read only those (files are opened memory-mapped).  Loading at the same layout reads one shard file per
  rank.  Publishing is atomic: write into ``iter_<N>.tmp``, fsync, rename, then replace the tracker file.  The reference
  stores no data position and replays batches on resume (train_loop.py:1489-1505, 1776-1783).
  ``ckpt/export_megatron.py`` rewrites such a checkpoint under Megatron-LM state-dict names.
* ``legacy`` — the reference engine's ``<root>/step_<N>/training_state.pt``: rank 0 ``torch.save`` of lists in
  parameter order ``{fp32_master, exp_avgs, exp_avg_sqs, state_steps, step, rng_*}`` (train_loop.py:1354-1406);
  load picks the newest ``*training_state.pt`` by mtime (train_loop.py:1409-1486).  TP = PP = 1 only.

``init_weights_only`` loads the weights but neither optimizer state, step nor RNG (the SFT phase hand-off).
"""
from __future__ import annotations

import dataclasses
import glob
import json
import os
import shutil

import torch
import torch.distributed as dist

from ..models import params as P
from ..optim.distributed import shard_ranges

TRACKER = "latest_checkpointed_iteration.txt"
STATE_KEYS = ("master", "exp_avg", "exp_avg_sq")


def _barrier():
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def _mp_dir(tp_rank: int, pp_rank: int, pp: int) -> str:
    return f"mp_rank_{tp_rank:02d}" if pp == 1 else f"mp_rank_{tp_rank:02d}_{pp_rank:03d}"


def _fsync_write(path: str, obj) -> None:
    with open(path, "wb") as f:
        torch.save(obj, f)
        f.flush()
        os.fsync(f.fileno())


def _per_param_optimizer_state(tr) -> dict:
    """Full per-parameter optimizer state on every rank (gathers over DP): used by the legacy single-file codec only."""
    full = tr.opt.gather_full_state()
    out = {}
    for name, (o, n) in tr.store.offsets.items():
        shp = tr.store.shapes[name]
        out[name] = {k: full[k][o:o + n].view(shp).cpu().clone() for k in STATE_KEYS}
    return out


def save(tr, root: str) -> str:
    fmt = tr.cfg.ckpt.format
    if fmt == "legacy":
        return _save_legacy(tr, root)
    topo, step, opt, store = tr.topo, tr.step, tr.opt, tr.store
    final = os.path.join(root, f"iter_{step:07d}")
    tmp = final + ".tmp"
    if tr.rank == 0:
        os.makedirs(root, exist_ok=True)
        if os.path.isdir(tmp):
            shutil.rmtree(tmp)
        os.makedirs(tmp)
    _barrier()
    d = os.path.join(tmp, _mp_dir(topo.tp_rank, topo.pp_rank, topo.pp))
    os.makedirs(d, exist_ok=True)
    # every rank that owns optimizer state writes exactly that (a ZeRO-1 shard, or the whole state on DP rank 0 otherwise)
    if opt.sharded or topo.dp_rank == 0:
        _fsync_write(os.path.join(d, f"distrib_optim_dp{opt.dpr:03d}.pt"), {
            "master": opt.master.detach().cpu(), "exp_avg": opt.m.detach().cpu(), "exp_avg_sq": opt.v.detach().cpu(),
            "ranges": [list(r) for r in opt.my_ranges], "dp_rank": opt.dpr, "dp_world": opt.dpw,
            "rng_state": tr.rng_state(), "data_state": tr.data_state(), "optimizer_step": opt.step_count})
    if topo.dp_rank == 0:
        _fsync_write(os.path.join(d, "model_optim_rng.pt"), {
            "model": {k: v.detach().cpu().clone() for k, v in store.params.items()},
            "optimizer_step": opt.step_count,
            "iteration": step,
            "data_state": tr.data_state(),
            "checkpoint_version": 3.0,
            "args": {k: dataclasses.asdict(getattr(tr.cfg, k)) for k in ("model", "optim", "parallel")},
        })
        with open(os.path.join(d, "layout.json"), "w") as f:
            json.dump({"tp_rank": topo.tp_rank, "pp_rank": topo.pp_rank, "numel": store.numel,
                       "buckets": [[b.start, b.end] for b in store.buckets], "dp_shards": opt.dpw,
                       "params": {n: [o, c, list(store.shapes[n])] for n, (o, c) in store.offsets.items()}}, f)
            f.flush()
            os.fsync(f.fileno())
    _barrier()
    if tr.rank == 0:
        mp = {}
        for ld in sorted(glob.glob(os.path.join(tmp, "mp_rank_*", "layout.json"))):
            mp[os.path.basename(os.path.dirname(ld))] = json.load(open(ld))
        meta = {"format": "megatron_dist", "version": 2, "iteration": step, "tp": topo.tp, "pp": topo.pp, "dp": topo.dp,
                "vpp": tr.cfg.parallel.virtual_pipeline_stages, "layer_split": list(tr.cfg.parallel.pipeline_layer_split),
                "sharded_optimizer": opt.sharded, "model": dataclasses.asdict(tr.cfg.model), "dtype": tr.cfg.train.dtype, "mp": mp}
        with open(os.path.join(tmp, "metadata.json"), "w") as f:
            json.dump(meta, f, indent=1)
            f.flush()
            os.fsync(f.fileno())
        if os.path.isdir(final):
            shutil.rmtree(final)
        os.rename(tmp, final)
        tpath = os.path.join(root, TRACKER)
        with open(tpath + ".tmp", "w") as f:
            f.write(str(step))
            f.flush()
            os.fsync(f.fileno())
        os.replace(tpath + ".tmp", tpath)
    _barrier()
    return final


def latest_iteration(root: str) -> int | None:
    """Highest COMPLETE checkpoint: the tracker if its directory is complete, else the newest complete dir."""
    def complete(it):
        return os.path.isfile(os.path.join(root, f"iter_{it:07d}", "metadata.json"))
    tpath = os.path.join(root, TRACKER)
    if os.path.isfile(tpath):
        try:
            it = int(open(tpath).read().strip())
            if complete(it):
                return it
        except ValueError:
            pass
    its = []
    for d in glob.glob(os.path.join(root, "iter_*")):
        b = os.path.basename(d)
        if b.endswith(".tmp"):
            continue
        try:
            it = int(b[5:])
        except ValueError:
            continue
        if complete(it):
            its.append(it)
    return max(its) if its else None


def _resolve(path: str) -> tuple[str, str]:
    """Returns ``(format, concrete path)`` for a root or a specific checkpoint directory."""
    if os.path.isfile(os.path.join(path, "metadata.json")):
        return "megatron_dist", path
    it = latest_iteration(path)
    if it is not None:
        return "megatron_dist", os.path.join(path, f"iter_{it:07d}")
    cands = glob.glob(os.path.join(path, "**", "*training_state.pt"), recursive=True)
    if cands:
        return "legacy", max(cands, key=os.path.getmtime)
    raise FileNotFoundError(f"no checkpoint under {path}")


class ShardReader:
    """Random access to the optimizer state of a ``megatron_dist`` checkpoint by (model-parallel rank, flat range).
    Shard files are opened memory-mapped and kept open, so only the pages a caller touches are read."""

    def __init__(self, concrete: str, meta: dict):
        self.dir, self.meta, self._files = concrete, meta, {}
        self.bytes_requested = 0

    def _shard(self, mp_name: str, d: int) -> dict:
        key = (mp_name, d)
        if key not in self._files:
            path = os.path.join(self.dir, mp_name, f"distrib_optim_dp{d:03d}.pt")
            try:
                self._files[key] = torch.load(path, map_location="cpu", weights_only=False, mmap=True)
            except (RuntimeError, ValueError):   # a file not written in the zip format cannot be mapped
                self._files[key] = torch.load(path, map_location="cpu", weights_only=False)
        return self._files[key]

    def flat_range(self, mp_name: str, key: str, start: int, count: int) -> torch.Tensor:
        """Elements ``[start, start + count)`` of the flat state ``key`` of one model-parallel rank, assembled from the DP
        shards that own them."""
        lay = self.meta["mp"][mp_name]
        out = torch.empty(count, dtype=torch.float32)
        dpw = int(lay["dp_shards"])
        for d in range(dpw):
            for (r0, r1, so) in shard_ranges(lay["buckets"], dpw, d):
                lo, hi = max(r0, start), min(r1, start + count)
                if hi > lo:
                    out[lo - start: hi - start] = self._shard(mp_name, d)[key][so + lo - r0: so + hi - r0]
                    self.bytes_requested += (hi - lo) * 4
        return out

    def mp_ranks(self):
        return {name: (int(l["tp_rank"]), int(l["pp_rank"])) for name, l in self.meta["mp"].items()}


def full_param_state(reader: ShardReader, cfg, name: str, spec, keys=STATE_KEYS) -> dict:
    """``{key: FULL logical fp32 tensor}`` of one parameter, assembled from every old TP shard that holds part of it."""
    old_tp = reader.meta["tp"]
    full = {k: torch.zeros(spec.full_shape, dtype=torch.float32) for k in keys}
    found = False
    for mp_name, (tp_r, _pp_r) in reader.mp_ranks().items():
        ent = reader.meta["mp"][mp_name]["params"].get(name)
        if ent is None:
            continue
        found = True
        o, n, shp = ent
        dim, idx = P.shard_rows(spec, cfg, old_tp, tp_r)
        for k in keys:
            src = reader.flat_range(mp_name, k, o, n).view(shp)
            if idx is None:
                full[k].copy_(src)
            else:
                full[k].index_copy_(dim, idx, src)
    if not found:
        raise KeyError(f"{name} not found in checkpoint {reader.dir}")
    return full


def local_param_state(reader: ShardReader, cfg, name: str, spec, new_tp: int, new_rank: int, keys=STATE_KEYS) -> dict:
    """``{key: fp32 tensor}`` of the rows (or columns) of one parameter that TP rank ``new_rank`` of a ``new_tp``-way layout
    holds, read from whichever old shards have them: old ranks without any needed row are not opened for this tensor, and
    for tensors sharded along dim 0 only the needed row runs are read (each row is one contiguous run of the flat shard)."""
    old_tp = reader.meta["tp"]
    dim_n, idx_n = P.shard_rows(spec, cfg, new_tp, new_rank)
    shape = list(spec.full_shape)
    if idx_n is not None:
        shape[dim_n] = idx_n.numel()
    out = {k: torch.zeros(shape, dtype=torch.float32) for k in keys}
    found = False
    filled = None
    for mp_name, (tp_r, _pp_r) in sorted(reader.mp_ranks().items()):
        ent = reader.meta["mp"][mp_name]["params"].get(name)
        if ent is None:
            continue
        found = True
        o, n, shp = ent
        dim_o, idx_o = P.shard_rows(spec, cfg, old_tp, tp_r)
        if idx_o is None and idx_n is None:           # replicated on both sides: any one copy
            for k in keys:
                out[k].copy_(reader.flat_range(mp_name, k, o, n).view(shp))
            break
        dim = dim_o if idx_o is not None else dim_n
        extent = spec.full_shape[dim]
        full_o = idx_o if idx_o is not None else torch.arange(extent)
        full_n = idx_n if idx_n is not None else torch.arange(extent)
        inv = torch.full((extent,), -1, dtype=torch.long)
        inv[full_n] = torch.arange(full_n.numel())
        pos = inv[full_o]                               # new local position of every old local row (-1: not needed)
        if filled is None:
            filled = torch.zeros(full_n.numel(), dtype=torch.bool)
        need = (pos >= 0)
        need[need.clone()] &= ~filled[pos[need]]
        if not bool(need.any()):
            continue
        old_rows = torch.nonzero(need).reshape(-1)
        new_rows = pos[old_rows]
        filled[new_rows] = True
        if dim == 0:
            row_elems = n // shp[0]
            runs, start = [], 0
            rows = old_rows.tolist()
            for i in range(1, len(rows) + 1):
                if i == len(rows) or rows[i] != rows[i - 1] + 1:
                    runs.append((rows[start], rows[i - 1] + 1, start))
                    start = i
            for k in keys:
                flat_out = out[k].view(shape[0], -1)
                for a, b, at in runs:
                    src = reader.flat_range(mp_name, k, o + a * row_elems, (b - a) * row_elems).view(b - a, -1)
                    flat_out.index_copy_(0, new_rows[at:at + (b - a)], src)
        else:
            for k in keys:
                src = reader.flat_range(mp_name, k, o, n).view(shp)
                out[k].index_copy_(dim, new_rows, src.index_select(dim, old_rows))
    if not found:
        raise KeyError(f"{name} not found in checkpoint {reader.dir}")
    if filled is not None and not bool(filled.all()):
        raise KeyError(f"{name}: the checkpoint's shards do not cover every row this layout needs")
    return out


def load(tr, path: str, weights_only: bool = False) -> int:
    fmt, concrete = _resolve(path)
    if fmt == "legacy":
        return _load_legacy(tr, concrete, weights_only)
    meta = json.load(open(os.path.join(concrete, "metadata.json")))
    if meta.get("version", 1) < 2:
        raise ValueError(f"{concrete} was written by an older layout of this format (no per-rank optimizer shards)")
    topo, store, cfg, opt = tr.topo, tr.store, tr.cfg.model, tr.opt
    n_mp = len(meta["mp"])
    if n_mp != meta["tp"] * meta["pp"]:
        raise FileNotFoundError(f"checkpoint {concrete} has {n_mp} model-parallel shards, expected {meta['tp'] * meta['pp']}")
    same = (meta["tp"] == topo.tp and meta["pp"] == topo.pp and meta.get("vpp", 1) == tr.cfg.parallel.virtual_pipeline_stages
            and list(meta.get("layer_split", [])) == list(tr.cfg.parallel.pipeline_layer_split)
            and int(meta["dp"] if meta["sharded_optimizer"] else 1) == opt.dpw and bool(meta["sharded_optimizer"]) == bool(opt.sharded))
    my_mp = _mp_dir(topo.tp_rank, topo.pp_rank, topo.pp)
    keys = ("master",) if weights_only else STATE_KEYS
    own = None
    if same:
        # one file per rank: this rank's own shard, exactly as it was written
        own = torch.load(os.path.join(concrete, my_mp, f"distrib_optim_dp{opt.dpr:03d}.pt"), map_location="cpu", weights_only=False)
        opt.master.copy_(own["master"])
        if not weights_only:
            opt.m.copy_(own["exp_avg"])
            opt.v.copy_(own["exp_avg_sq"])
            opt.step_count = int(own["optimizer_step"])
        opt.sync_params_from_master()
        common = {"iteration": meta["iteration"], "optimizer_step": own["optimizer_step"], "data_state": own.get("data_state")}
    else:
        reader = ShardReader(concrete, meta)
        for name in store.params:
            spec = store.spec_by_name[name]
            local = local_param_state(reader, cfg, name, spec, topo.tp, topo.tp_rank, keys)
            o, n = store.offsets[name]
            for k in keys:
                opt.set_flat_range(k, o, local[k].reshape(-1).to(opt.master.device))
        any_mp = sorted(meta["mp"])[0]
        first = reader._shard(any_mp, 0)
        common = {"iteration": meta["iteration"], "optimizer_step": first["optimizer_step"], "data_state": first.get("data_state")}
        if not weights_only:
            opt.step_count = int(common["optimizer_step"])
        opt.sync_params_from_master()
        tr.last_load_bytes = reader.bytes_requested
    if not weights_only:
        tr.step = int(common["iteration"])
        if own is not None and own.get("rng_state"):
            tr.set_rng_state(own["rng_state"])
        ds = common.get("data_state")
        if ds is not None:
            tr.source.load_state_dict(ds)
    return tr.step


# ---------------------------------------------------------------------------
# legacy codec
# ---------------------------------------------------------------------------

def _ordered_names(tr):
    return [s.name for s in tr.store.specs]


def _save_legacy(tr, root: str) -> str:
    """Writes exactly what the reference's ``save_checkpoint`` writes (train_loop.py:1354-1406), so that its own
    ``load_checkpoint`` (train_loop.py:1409-1486) reads the file: tensors in lists in parameter order, the numpy and python
    RNG states as ``pickle.dumps`` BYTES, the torch CPU and CUDA generator states as uint8 tensors.  ``data_cursor`` is an
    extra key the reference ignores."""
    if tr.topo.tp != 1 or tr.topo.pp != 1:
        raise ValueError("the legacy step_<N>/training_state.pt format supports TP = PP = 1 only")
    state = _per_param_optimizer_state(tr)
    d = os.path.join(root, f"step_{tr.step}")
    if tr.rank == 0:
        os.makedirs(d, exist_ok=True)
        names = _ordered_names(tr)
        rng = tr.rng_state()
        import pickle
        cuda_rng = rng.get("cuda")
        if cuda_rng is None:  # written on a CPU run: a well-formed (seed 0, offset 0) CUDA generator state
            cuda_rng = torch.zeros(16, dtype=torch.uint8)
        obj = {"fp32_master": [state[n]["master"] for n in names],
               "exp_avgs": [state[n]["exp_avg"] for n in names],
               "exp_avg_sqs": [state[n]["exp_avg_sq"] for n in names],
               "state_steps": [torch.tensor(float(tr.opt.step_count)) for _ in names],
               "step": torch.tensor(tr.step, dtype=torch.int32),
               "rng_torch": rng["torch"], "rng_cuda": cuda_rng.cpu(),
               "rng_numpy": pickle.dumps(rng["numpy"]),
               "rng_random": pickle.dumps(rng["python"]),
               "data_cursor": torch.tensor(tr.data_state().get("cursor", -1), dtype=torch.int64)}
        tmp = os.path.join(d, "training_state.pt.tmp")
        _fsync_write(tmp, obj)
        os.replace(tmp, os.path.join(d, "training_state.pt"))
    _barrier()
    return d


def _unpickle_rng(blob):
    """RNG states arrive as ``pickle.dumps`` bytes (the reference's files and this module's) or as the uint8 tensor of
    those bytes (files written by earlier versions of this module)."""
    import pickle
    if isinstance(blob, torch.Tensor):
        blob = blob.cpu().numpy().tobytes()
    return pickle.loads(blob)


def _load_legacy(tr, file: str, weights_only: bool) -> int:
    sd = torch.load(file, map_location="cpu", weights_only=True)
    names = _ordered_names(tr)
    if len(sd["fp32_master"]) != len(names):
        raise ValueError("legacy checkpoint parameter count does not match the model")
    flat = {k: torch.zeros(tr.store.numel, dtype=torch.float32, device=tr.store.device) for k in ("master", "exp_avg", "exp_avg_sq")}
    for i, n in enumerate(names):
        o, cnt = tr.store.offsets[n]
        flat["master"][o:o + cnt].copy_(sd["fp32_master"][i].reshape(-1))
        if not weights_only:
            flat["exp_avg"][o:o + cnt].copy_(sd["exp_avgs"][i].reshape(-1))
            flat["exp_avg_sq"][o:o + cnt].copy_(sd["exp_avg_sqs"][i].reshape(-1))
    opt_step = int(sd["state_steps"][0]) if sd["state_steps"] else 0
    tr.opt.scatter_full_state(flat, opt_step, weights_only=weights_only)
    if not weights_only:
        tr.step = int(sd["step"])
        # all four generators, as the reference restores them (train_loop.py:1476-1483)
        import random

        import numpy as np
        torch.set_rng_state(sd["rng_torch"].cpu())
        if tr.device.type == "cuda" and sd.get("rng_cuda") is not None:
            torch.cuda.set_rng_state(sd["rng_cuda"].cpu(), tr.device)
        if sd.get("rng_numpy") is not None:
            np.random.set_state(_unpickle_rng(sd["rng_numpy"]))
        if sd.get("rng_random") is not None:
            random.setstate(_unpickle_rng(sd["rng_random"]))
        cur = int(sd.get("data_cursor", torch.tensor(-1)))
        if cur >= 0:
            tr.source.load_state_dict({"cursor": cur})
        else:
            tr.source.seek_microbatches(tr.step * tr.grad_accum)
    return tr.step
