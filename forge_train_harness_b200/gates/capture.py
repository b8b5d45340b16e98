"""Tensor-hash capture layer: blake2b-128 records of activations, gradients and losses for the alignment gates.

Record format and key families follow the reference's contract (evals/harness_hook/_dump.py:89-123,
evals/harness_hook/recipes/README.md:10-40, 64-80; emitter on the candidate side train_loop.py:95-114, 2563-2669):

    {"hash": <blake2b-128 hex of the raw bytes>, "shape": [...], "dtype": "torch.bfloat16"}

    step_<N>.rank<r>.mb<m>.fwd.<fqn>#<call>          level 2   module outputs
    step_<N>.rank<r>.mb<m>.bwd.<fqn>#<call>          level 2   gradient w.r.t. the module output
    step_<N>.rank<r>.mb<m>.loss.per_token.preallreduce   level 1   [MBS, S] fp32 NLL
    step_<N>.rank<r>.loss.scalar.{pre,post}allreduce     level 1
    step_<N>.rank<r>.grad.<fqn>.{pre,post}allreduce      level 1   fp32 main-grad per parameter

``mb<m>.`` prefixes only fwd / bwd / per-token keys.  Level 0 makes every method a no-op.  Dumps are one JSON file
per rank, ``<output>.rank<r>``, written atomically.  Hashing is blake2b on the HOST (the gates compare digests of raw
bytes, so a device-side hash of another kind would not be comparable); tensors are staged device -> pinned host on a
dedicated copy stream through a fixed ring so capture never allocates in the hot loop (evals/capture_offload.py:147-369).
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

CHUNK = 8_000_000  # elements per blake2b update, as the reference streams


def hash_tensor(t: torch.Tensor) -> dict:
    h = hashlib.blake2b(digest_size=16)
    shape, dtype = list(t.shape), str(t.dtype)
    if t.numel():
        flat = t.detach().reshape(-1)
        for chunk in flat.split(CHUNK):
            c = chunk.cpu().contiguous()
            h.update((c if c.dtype == torch.uint8 else c.view(torch.uint8)).numpy())
    return {"hash": h.hexdigest(), "shape": shape, "dtype": dtype}


class StagingRing:
    """Fixed pinned-memory ring + copy stream.  ``stage(t)`` returns a CPU view valid until the slot is reused (it waits for
    the copy).  ``submit(key, t, sink)`` is the asynchronous form the capture session uses: the device -> host copy is
    enqueued on the copy stream and a WORKER THREAD waits for it, hashes the bytes and stores the record, so the training
    thread never blocks on a hash (blake2b runs at ~1 GB/s per core, which is what made level-2 capture cost most of a
    step when it ran inline); the training thread only waits when every slot of the ring is still being hashed."""

    def __init__(self, nbytes: int = 256 << 20, slots: int = 4, device=None):
        self.cuda = torch.cuda.is_available() and device is not None and torch.device(device).type == "cuda"
        self.slots = slots
        self.bufs = [torch.empty(nbytes, dtype=torch.uint8, pin_memory=self.cuda) for _ in range(slots)] if self.cuda else []
        self.events = [None] * slots
        self.turn = 0
        self.stream = torch.cuda.Stream() if self.cuda else None
        import queue
        import threading
        self._free = threading.Semaphore(slots)
        self._q: "queue.Queue" = queue.Queue()
        self._err = None
        self._worker = threading.Thread(target=self._run, daemon=True)
        self._worker.start()

    def _run(self):
        while True:
            item = self._q.get()
            if item is None:
                self._q.task_done()
                return
            key, view, ev, sink, slot_held = item
            try:
                if ev is not None:
                    ev.synchronize()
                sink[key] = hash_tensor(view)
            except BaseException as e:  # surfaced by flush()
                self._err = e
            finally:
                if slot_held:
                    self._free.release()
                self._q.task_done()

    def submit(self, key: str, t: torch.Tensor, sink: dict) -> None:
        """Record ``hash_tensor(t)`` under ``key`` in ``sink`` without blocking on the copy or the hash."""
        nb = t.numel() * t.element_size()
        if not self.cuda or t.device.type != "cuda" or nb > self.bufs[0].numel():
            host = t.detach().to("cpu", copy=True)   # CPU tensors (and oversized ones) are snapshotted, then hashed off-thread
            self._q.put((key, host, None, sink, False))
            return
        self._free.acquire()                          # a slot whose previous content has been hashed
        k = self.turn
        self.turn = (self.turn + 1) % self.slots
        dst = self.bufs[k][:nb].view(t.dtype).view(t.shape)
        # a device-side snapshot first (an HBM copy on the training stream): several captured tensors are later updated in
        # place (logits become their gradient, RoPE rotates QKV), and the PCIe copy below runs behind the training stream
        snap = t.detach().clone()
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            dst.copy_(snap, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        snap.record_stream(self.stream)
        self._q.put((key, dst, ev, sink, True))

    def flush(self) -> None:
        """Wait until every submitted tensor has been hashed; re-raises a worker failure."""
        self._q.join()
        if self._err is not None:
            err, self._err = self._err, None
            raise err

    def stage(self, t: torch.Tensor) -> torch.Tensor:
        if not self.cuda or t.device.type != "cuda":
            return t.detach().cpu()
        nb = t.numel() * t.element_size()
        k = self.turn
        self.turn = (self.turn + 1) % self.slots
        if nb > self.bufs[k].numel():
            return t.detach().cpu()
        if self.events[k] is not None:
            self.events[k].synchronize()
        dst = self.bufs[k][:nb].view(t.dtype).view(t.shape)
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            dst.copy_(t.detach(), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        t.record_stream(self.stream)
        self.events[k] = ev
        ev.synchronize()
        return dst


class CaptureSession:
    """``mode="hash"`` keeps a digest per tensor (the bitwise gates); ``mode="tensor"`` keeps the tensors themselves on the
    host and ``dump`` writes one ``torch.save`` file per rank, for the tolerance-mode alignment against a reference whose
    kernels differ (``verdicts.align_tolerance``)."""

    def __init__(self, output_file: str | None, level: int = 1, rank: int = 0, fqn_alias=None, device=None, mode: str = "hash"):
        if mode not in ("hash", "tensor"):
            raise ValueError("capture mode must be 'hash' or 'tensor'")
        self.out, self.level, self.rank, self.mode = output_file, int(level), rank, mode
        self.records: dict[str, dict] = {}
        self.step, self.mb = 0, 0
        self.calls: dict[tuple, int] = {}
        self.alias = fqn_alias or (lambda n: n)
        self.ring = StagingRing(device=device) if self.level > 0 else None

    # -- positioning ---------------------------------------------------------
    def begin_step(self, step: int):
        self.step, self.mb = step, 0
        self.calls.clear()

    def begin_microbatch(self, mb: int):
        self.mb = mb
        self.calls.clear()

    def _put(self, key: str, t: torch.Tensor):
        if self.mode == "tensor":
            self.records[key] = t.detach().to("cpu", copy=True)
            return
        if self.ring is not None:
            self.ring.submit(key, t, self.records)   # hashed by the ring's worker thread; dump() waits for it
        else:
            self.records[key] = hash_tensor(t)

    # -- capture points ---------------------------------------------------------
    def module_hook(self, kind: str, fqn: str, t: torch.Tensor):
        if self.level < 2:
            return
        k = (kind, fqn)
        idx = self.calls.get(k, 0)
        self.calls[k] = idx + 1
        self._put(f"step_{self.step}.rank{self.rank}.mb{self.mb}.{kind}.{self.alias(fqn)}#{idx}", t)

    def per_token_loss(self, nll: torch.Tensor, micro_batch: int):
        if self.level < 1:
            return
        self._put(f"step_{self.step}.rank{self.rank}.mb{self.mb}.loss.per_token.preallreduce",
                  nll.float().view(micro_batch, -1))

    def loss_scalar(self, which: str, stats: torch.Tensor):
        if self.level < 1:
            return
        self._put(f"step_{self.step}.rank{self.rank}.loss.scalar.{which}allreduce", stats[:2].double())

    def grads(self, which: str, store, scale=None):
        if self.level < 1:
            return
        for name, g in store.grads.items():
            t = g if scale is None else g * scale
            self._put(f"step_{self.step}.rank{self.rank}.grad.{self.alias(name)}.{which}allreduce", t)

    # -- output -----------------------------------------------------------------
    def dump(self):
        if self.ring is not None:
            self.ring.flush()
        if self.level < 1 or not self.out:
            return
        path = f"{self.out}.rank{self.rank}"
        tmp = path + ".tmp"
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        if self.mode == "tensor":
            torch.save(self.records, tmp)
            os.replace(tmp, path)
            return
        with open(tmp, "w") as f:
            json.dump(self.records, f)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)


def load_merged(output_file: str) -> dict:
    """Union of every ``<output>.rank<r>`` file (harness/capture_artifacts.py:63-138)."""
    import glob
    out: dict = {}
    files = sorted(glob.glob(output_file + ".rank*"))
    if os.path.isfile(output_file):
        files.append(output_file)
    for fn in files:
        if fn.endswith(".tmp"):
            continue
        with open(fn) as f:
            out.update(json.load(f))
    return out


_POS = __import__("re").compile(r"^step_\d+\.rank\d+\.(mb\d+\.)?")


def family_key(key: str) -> str:
    """``step_3.rank0.mb1.fwd.layers.0.wqkv#0`` -> ``fwd.layers.0.wqkv``; ``...grad.<fqn>.preallreduce`` -> ``grad.<fqn>``
    (post-all-reduce records keep their suffix, so they never stand in for the local gradient)."""
    k = _POS.sub("", key).split("#", 1)[0]
    if k.endswith(".preallreduce"):
        k = k[: -len(".preallreduce")]
    return k


def diff_tensors(baseline: dict, candidate: dict, *, family: str, rel_tol: float, fit_scale: bool = False,
                 max_tol: float | None = None, scales: dict | None = None) -> dict:
    """Tolerance-mode alignment of two tensor captures.  Keys are reduced to ``<family>.<fqn>`` (the first occurrence of a
    key wins: step, rank, micro-batch and call index are dropped) and tensors are flattened.  For every key both sides have,
    the relative L2 error ``||a - b|| / ||b||`` must stay below ``rel_tol`` and the largest element error, relative to the
    reference's RMS, below ``max_tol`` (default ``25 x rel_tol``: a bf16 rounding of an entry several times the RMS is a
    few percent of the RMS by itself, so the L2 figure is the tight one).  ``scales`` multiplies named candidate keys by a
    known factor (a capture point that sits on the other side of a constant scale); ``fit_scale`` removes the best common
    scalar per key instead (gradients w.r.t. a module output depend on where a stack applies its residual scale) and
    reports it.  No overlap, or a size mismatch, fails."""
    max_tol = 25.0 * rel_tol if max_tol is None else max_tol

    def reduce(d):
        out = {}
        for k, v in d.items():
            fk = family_key(k)
            if fk.startswith(family + ".") and isinstance(v, torch.Tensor) and fk not in out:
                out[fk] = v
        return out
    b, c = reduce(baseline), reduce(candidate)
    common = sorted(set(b) & set(c))
    rows, worst, bad = {}, 0.0, []
    for k in common:
        x, y = c[k].double().reshape(-1), b[k].double().reshape(-1)
        if x.numel() != y.numel():
            bad.append(k)
            rows[k] = {"error": f"sizes {tuple(c[k].shape)} vs {tuple(b[k].shape)}"}
            continue
        scale = float((scales or {}).get(k, 1.0))
        if fit_scale:
            den = float((x * x).sum())
            scale = float((x * y).sum()) / den if den > 0 else 1.0
        norm = float(y.pow(2).sum().sqrt()) or 1.0
        rms = norm / max(y.numel(), 1) ** 0.5
        d = x * scale - y
        l2, mx = float(d.pow(2).sum().sqrt()) / norm, float(d.abs().max()) / (rms or 1.0)
        rows[k] = {"rel_l2": l2, "max_rel_err": mx, "scale": scale}
        worst = max(worst, l2)
        if not (l2 <= rel_tol and mx <= max_tol):
            bad.append(k)
    return {"passed": bool(common) and not bad, "overlap": len(common), "mismatched": bad, "worst_rel_err": worst,
            "rel_tol": rel_tol, "max_tol": max_tol, "missing_in_candidate": sorted(set(b) - set(c)), "per_key": rows}


def diff_captures(baseline: dict, candidate: dict, *, prefix: str = "", require_baseline_complete: bool = False) -> dict:
    """Intersect-and-diff of two hash dicts (evals/_capture_diff.py:73-248).

    Zero overlap is a FAIL; with ``require_baseline_complete`` every baseline key must exist in the candidate."""
    bk = {k for k in baseline if prefix in k}
    ck = {k for k in candidate if prefix in k}
    common = sorted(bk & ck)
    mism = [k for k in common if baseline[k]["hash"] != candidate[k]["hash"]
            or baseline[k].get("shape") != candidate[k].get("shape")]
    missing = sorted(bk - ck)
    ok = bool(common) and not mism and not (require_baseline_complete and missing)
    return {"passed": ok, "overlap": len(common), "mismatched": mism, "missing_in_candidate": missing,
            "extra_in_candidate": sorted(ck - bk)}
