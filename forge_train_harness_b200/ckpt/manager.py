"""Checkpoint save / load / reshard.

Two on-disk formats:

* ``megatron_dist`` (default) — Megatron-style directory layout: ``<root>/latest_checkpointed_iteration.txt``
  and ``<root>/iter_<N:07d>/mp_rank_<tp:02d>[_<pp:03d>]/model_optim_rng.pt`` written by DP rank 0 of every
  model-parallel rank, plus ``metadata.json`` with the parallel layout.  Tensors are stored per FQN as the
  local TP shard (model weights in the compute dtype; optimizer ``master`` / ``exp_avg`` / ``exp_avg_sq`` in
  fp32, assembled over the ZeRO-1 DP shards), and the shard <-> full index map is a pure function of
  (model config, tp, rank), so a checkpoint saved at one TP x PP x DP layout loads at any other.  The file
  also carries the step, RNG states, the LR-relevant step counter and the DATA CURSOR (the reference stores
  no data position and replays batches on resume, train_loop.py:1489-1505, 1776-1783).  Publishing is atomic:
  write into ``iter_<N>.tmp``, fsync, rename, then replace the tracker file.
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

TRACKER = "latest_checkpointed_iteration.txt"


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
    full = tr.opt.gather_full_state()
    out = {}
    for name, (o, n) in tr.store.offsets.items():
        shp = tr.store.shapes[name]
        out[name] = {k: full[k][o:o + n].view(shp).cpu().clone() for k in ("master", "exp_avg", "exp_avg_sq")}
    return out


def save(tr, root: str) -> str:
    fmt = tr.cfg.ckpt.format
    if fmt == "legacy":
        return _save_legacy(tr, root)
    topo, step = tr.topo, tr.step
    final = os.path.join(root, f"iter_{step:07d}")
    tmp = final + ".tmp"
    if tr.rank == 0:
        os.makedirs(root, exist_ok=True)
        if os.path.isdir(tmp):
            shutil.rmtree(tmp)
        os.makedirs(tmp)
    _barrier()
    opt_state = _per_param_optimizer_state(tr)  # collective over the DP group
    if topo.dp_rank == 0:
        d = os.path.join(tmp, _mp_dir(topo.tp_rank, topo.pp_rank, topo.pp))
        os.makedirs(d, exist_ok=True)
        _fsync_write(os.path.join(d, "model_optim_rng.pt"), {
            "model": {k: v.detach().cpu().clone() for k, v in tr.store.params.items()},
            "optimizer": opt_state,
            "optimizer_step": tr.opt.step_count,
            "iteration": step,
            "rng_state": [tr.rng_state()],
            "data_state": tr.data_state(),
            "checkpoint_version": 3.0,
            "args": {k: dataclasses.asdict(getattr(tr.cfg, k)) for k in ("model", "optim", "parallel")},
        })
    _barrier()
    if tr.rank == 0:
        meta = {"format": "megatron_dist", "iteration": step, "tp": topo.tp, "pp": topo.pp, "dp": topo.dp,
                "vpp": tr.cfg.parallel.virtual_pipeline_stages, "sharded_optimizer": tr.opt.sharded,
                "model": dataclasses.asdict(tr.cfg.model), "dtype": tr.cfg.train.dtype}
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


def load(tr, path: str, weights_only: bool = False) -> int:
    fmt, concrete = _resolve(path)
    if fmt == "legacy":
        return _load_legacy(tr, concrete, weights_only)
    meta = json.load(open(os.path.join(concrete, "metadata.json")))
    old_tp, old_pp = meta["tp"], meta["pp"]
    files = {}
    for d in sorted(glob.glob(os.path.join(concrete, "mp_rank_*"))):
        parts = os.path.basename(d).split("_")
        tp_r = int(parts[2])
        pp_r = int(parts[3]) if len(parts) > 3 else 0
        files[(tp_r, pp_r)] = os.path.join(d, "model_optim_rng.pt")
    if len(files) != old_tp * old_pp:
        raise FileNotFoundError(f"checkpoint {concrete} has {len(files)} model-parallel shards, expected {old_tp * old_pp}")
    topo, store, cfg = tr.topo, tr.store, tr.cfg.model
    same = (old_tp == topo.tp and old_pp == topo.pp and meta.get("vpp", 1) == tr.cfg.parallel.virtual_pipeline_stages)
    common = None
    if same:
        sd = torch.load(files[(topo.tp_rank, topo.pp_rank)], map_location="cpu", weights_only=False)
        common = sd
        shards = {name: {k: sd["optimizer"][name][k] for k in ("master", "exp_avg", "exp_avg_sq")} for name in store.params}
    else:
        loaded = {k: torch.load(f, map_location="cpu", weights_only=False) for k, f in files.items()}
        common = loaded[(0, 0)] if (0, 0) in loaded else next(iter(loaded.values()))
        shards = {}
        for name in store.params:
            spec = store.spec_by_name[name]
            full = {k: torch.zeros(spec.full_shape, dtype=torch.float32) for k in ("master", "exp_avg", "exp_avg_sq")}
            found = False
            for (tp_r, pp_r), sd in loaded.items():
                if name not in sd["optimizer"]:
                    continue
                found = True
                dim, idx = P.shard_rows(spec, cfg, old_tp, tp_r)
                for k in full:
                    src = sd["optimizer"][name][k]
                    if idx is None:
                        full[k].copy_(src)
                    else:
                        full[k].index_copy_(dim, idx, src)
            if not found:
                raise KeyError(f"{name} not found in checkpoint {concrete}")
            dim, idx = P.shard_rows(spec, cfg, topo.tp, topo.tp_rank)
            shards[name] = {k: (v if idx is None else v.index_select(dim, idx)) for k, v in full.items()}
    flat = {k: torch.zeros(store.numel, dtype=torch.float32, device=store.device) for k in ("master", "exp_avg", "exp_avg_sq")}
    for name, (o, n) in store.offsets.items():
        for k in flat:
            flat[k][o:o + n].copy_(shards[name][k].reshape(-1))
    tr.opt.scatter_full_state(flat, common["optimizer_step"], weights_only=weights_only)
    if not weights_only:
        tr.step = int(common["iteration"])
        if same and common.get("rng_state"):
            tr.set_rng_state(common["rng_state"][0])
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
