"""Token sources with an O(1) resumable cursor, a background prefetcher and one-copy H2D staging.

* ``SyntheticTokens`` — seeded uniform token ids, labels = inputs shifted by one.  Sample ``i`` is a
  pure function of ``(seed, i)``, so seeking is free and the data is independent of the DP layout.
* ``MegatronBinary`` — reader (and a writer for tests / synthetic corpora) of the Megatron indexed
  ``.bin/.idx`` format with the reference reader's windowing and sharding rules
  (ref/reference/train_pure_mup_mtp.py:132-230): concatenate documents, cut into non-overlapping
  ``seq+1`` windows, shared seeded shuffle, round-robin split over DP ranks, per-epoch reshuffle.
  Unlike the reference (which resumes by replaying and discarding batches, train_loop.py:1489-1505)
  the position is ``(epoch, pos)`` and is restored directly.
* ``Prefetcher`` — daemon producer thread with bounded queue (train_loop.py:294-394); skips
  micro-batches whose loss mask is all zero, as both reference stacks do.
* ``BatchStager`` — one pinned host buffer and one device buffer holding ids / labels / mask (+ MTP
  tensors); a micro-batch is ONE ``cudaMemcpyAsync`` and the device views keep stable addresses for
  CUDA-graph replay (train_loop.py:1641-1665).  Token ids travel as int32.
"""
from __future__ import annotations

import queue
import struct
import threading

import numpy as np
import torch

_IDX_MAGIC = b"MMIDIDX\x00\x00"
_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32, 8: np.uint16}
_DTYPE_CODES = {np.dtype(v): k for k, v in _DTYPES.items()}


def build_mtp_tensors(ids: torch.Tensor, labels: torch.Tensor, mask: torch.Tensor):
    """Next-next-token targets: input = labels, label[t] = labels[t+1], mask[t] = mask[t]*mask[t+1],
    last position masked (ref/reference/train_pure_mup_mtp.py:456-471).  All ``[B, S]``."""
    mtp_ids = labels.clone()
    mtp_labels = torch.zeros_like(labels)
    mtp_labels[:, :-1] = labels[:, 1:]
    mtp_mask = torch.zeros_like(mask)
    mtp_mask[:, :-1] = mask[:, :-1] * mask[:, 1:]
    return mtp_ids, mtp_labels, mtp_mask


class SyntheticTokens:
    def __init__(self, vocab: int, seq_len: int, micro_batch: int, dp_rank: int, dp_size: int, seed: int = 0):
        self.vocab, self.seq_len, self.mbs, self.dp_rank, self.dp_size, self.seed = \
            vocab, seq_len, micro_batch, dp_rank, dp_size, seed
        self.cursor = 0  # globally consumed samples (same on every DP rank, independent of the DP degree)

    def state_dict(self):
        return {"kind": "synthetic", "cursor": self.cursor, "seed": self.seed}

    def load_state_dict(self, sd):
        self.cursor = int(sd["cursor"])

    def seek_microbatches(self, n: int):
        self.cursor = int(n) * self.mbs * self.dp_size

    def _sample(self, idx: int) -> torch.Tensor:
        g = torch.Generator().manual_seed((self.seed * 1_000_003 + idx) & 0x7FFFFFFFFFFFFFFF)
        return torch.randint(0, self.vocab, (self.seq_len + 1,), generator=g, dtype=torch.int64)

    def __iter__(self):
        return self

    def __next__(self):
        base = self.cursor + self.dp_rank * self.mbs
        w = torch.stack([self._sample(base + b) for b in range(self.mbs)])
        self.cursor += self.mbs * self.dp_size
        return {"tokens": w[:, :-1].contiguous(), "labels": w[:, 1:].contiguous(),
                "loss_mask": torch.ones(self.mbs, self.seq_len, dtype=torch.float32)}


def write_megatron_binary(prefix: str, documents: list[np.ndarray], dtype=np.int32) -> None:
    """Write ``<prefix>.bin`` / ``<prefix>.idx`` (one sequence per document)."""
    dt = np.dtype(dtype)
    sizes = np.array([len(d) for d in documents], dtype=np.int32)
    pointers = np.zeros(len(documents), dtype=np.int64)
    if len(documents) > 1:
        pointers[1:] = np.cumsum(sizes[:-1].astype(np.int64) * dt.itemsize)
    with open(prefix + ".bin", "wb") as f:
        for d in documents:
            f.write(np.asarray(d, dtype=dt).tobytes())
    with open(prefix + ".idx", "wb") as f:
        f.write(_IDX_MAGIC)
        f.write(struct.pack("<q", 1))
        f.write(struct.pack("<B", _DTYPE_CODES[dt]))
        f.write(struct.pack("<q", len(documents)))
        f.write(struct.pack("<q", len(documents) + 1))
        f.write(sizes.tobytes())
        f.write(pointers.tobytes())
        f.write(np.arange(len(documents) + 1, dtype=np.int64).tobytes())


class MegatronBinary:
    def __init__(self, prefix: str, seq_len: int, micro_batch: int, dp_rank: int, dp_size: int, seed: int):
        with open(prefix + ".idx", "rb") as f:
            if f.read(9) != _IDX_MAGIC:
                raise ValueError("not a Megatron .idx file")
            struct.unpack("<q", f.read(8))
            code = struct.unpack("<B", f.read(1))[0]
            n_seq = struct.unpack("<q", f.read(8))[0]
            struct.unpack("<q", f.read(8))
            sizes = np.frombuffer(f.read(n_seq * 4), dtype=np.int32)
            pointers = np.frombuffer(f.read(n_seq * 8), dtype=np.int64)
        dt = np.dtype(_DTYPES[code])
        data = np.memmap(prefix + ".bin", dtype=dt, mode="r")
        contiguous = bool(np.all(pointers == np.concatenate([[0], np.cumsum(sizes[:-1].astype(np.int64))]) * dt.itemsize))
        if contiguous:
            flat = data[: int(sizes.astype(np.int64).sum())]
        else:
            flat = np.concatenate([data[p // dt.itemsize: p // dt.itemsize + s] for p, s in zip(pointers, sizes)])
        w = seq_len + 1
        n_win = len(flat) // w
        self.windows = flat[: n_win * w].reshape(n_win, w)
        order = np.arange(n_win)
        np.random.RandomState(seed).shuffle(order)
        self.base_order = order[dp_rank::dp_size]
        self.n_local = len(self.base_order)
        self.seq_len, self.mbs, self.dp_rank, self.dp_size, self.seed = seq_len, micro_batch, dp_rank, dp_size, seed
        self.epoch, self.pos = 0, 0
        self._order = self.base_order

    def _order_for_epoch(self, epoch: int):
        order = self.base_order
        for e in range(1, epoch + 1):  # the reference permutes the previous epoch's order
            rng = np.random.RandomState(self.seed + self.dp_rank + self.dp_size + e * 1000)
            order = order[rng.permutation(self.n_local)]
        return order

    def state_dict(self):
        """``pos`` counts samples of THIS rank's round-robin share, so the state also records the DP degree it belongs to
        and the layout-independent number of samples the whole DP group has consumed in the epoch."""
        return {"kind": "megatron_binary", "epoch": self.epoch, "pos": self.pos, "dp_size": self.dp_size,
                "consumed_in_epoch": self.pos * self.dp_size}

    def load_state_dict(self, sd):
        epoch, pos = int(sd["epoch"]), int(sd["pos"])
        old_dp = int(sd.get("dp_size", self.dp_size))
        if old_dp != self.dp_size:
            # Another DP degree: in epoch 0 every rank reads ``order[rank::dp]`` of ONE shared shuffle, so "the group has
            # consumed the first n samples" carries over.  Later epochs permute each rank's share with a seed that depends
            # on the layout (the reference's rule), so a position inside them has no counterpart in another layout.
            if epoch != 0:
                raise ValueError(f"data position was saved at dp={old_dp} in epoch {epoch}; only an epoch-0 position can be "
                                 f"moved to dp={self.dp_size} (later epochs are shuffled per DP rank)")
            consumed = int(sd.get("consumed_in_epoch", pos * old_dp))
            if consumed % self.dp_size:
                raise ValueError(f"{consumed} samples consumed at dp={old_dp} do not split evenly over dp={self.dp_size}")
            pos = consumed // self.dp_size
        self.epoch, self.pos = epoch, pos
        self._order = self._order_for_epoch(self.epoch)

    def seek_microbatches(self, n: int):
        total = n * self.mbs
        self.epoch, self.pos = divmod(total, self.n_local) if self.n_local else (0, 0)
        self._order = self._order_for_epoch(self.epoch)

    def __iter__(self):
        return self

    def __next__(self):
        if self.n_local == 0:
            raise StopIteration
        rows = []
        for _ in range(self.mbs):
            if self.pos >= self.n_local:
                self.epoch += 1
                self._order = self._order_for_epoch(self.epoch)
                self.pos = 0
            rows.append(self.windows[self._order[self.pos]])
            self.pos += 1
        b = torch.from_numpy(np.stack(rows).astype(np.int64))
        return {"tokens": b[:, :-1].contiguous(), "labels": b[:, 1:].contiguous(),
                "loss_mask": torch.ones(self.mbs, self.seq_len, dtype=torch.float32)}


def build_source(data_cfg, model_cfg, micro_batch: int, dp_rank: int, dp_size: int, seed: int):
    if data_cfg.data_loader == "synthetic":
        return SyntheticTokens(model_cfg.padded_vocab_size, model_cfg.seq_length, micro_batch, dp_rank, dp_size,
                               data_cfg.synthetic_seed)
    if data_cfg.data_loader == "megatron_binary":
        return MegatronBinary(data_cfg.data_path, model_cfg.seq_length, micro_batch, dp_rank, dp_size, seed)
    if data_cfg.data_loader == "hf":
        from .hf_stream import HFStream, parse_data_path
        return HFStream(parse_data_path(data_cfg.data_path), model_cfg.seq_length, micro_batch, dp_rank, dp_size, seed)
    if data_cfg.data_loader == "modelbest":
        from .hf_stream import build_modelbest
        return build_modelbest(data_cfg.data_path)
    raise ValueError(f"unknown data_loader {data_cfg.data_loader!r}")


class Prefetcher:
    """Runs ``next(source)`` on a daemon thread.  ``state_dict`` is the cursor of the NEXT batch the
    consumer will receive (not of the producer), so a checkpoint resumes exactly."""

    def __init__(self, source, depth: int = 8, enabled: bool = True):
        self.source, self.enabled = source, enabled and depth > 0
        self._q: queue.Queue = queue.Queue(maxsize=max(depth, 1))
        self._stop = threading.Event()
        self._consumer_state = source.state_dict()
        self._thread = None
        if self.enabled:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def _produce(self):
        while True:
            b = next(self.source)
            if float(b["loss_mask"].sum()) > 0:
                return b, self.source.state_dict()

    def _run(self):
        try:
            while not self._stop.is_set():
                item = self._produce()
                while not self._stop.is_set():
                    try:
                        self._q.put(item, timeout=0.1)
                        break
                    except queue.Full:
                        continue
        except StopIteration:
            self._q.put(None)
        except BaseException as e:  # surface producer failures to the consumer
            self._q.put(e)

    def get(self):
        if not self.enabled:
            b, st = self._produce()
        else:
            item = self._q.get()
            if item is None:
                raise StopIteration
            if isinstance(item, BaseException):
                raise item
            b, st = item
        self._consumer_state = st
        return b

    def state_dict(self):
        return dict(self._consumer_state)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)


class BatchStager:
    """Packs a micro-batch into one pinned buffer and moves it with one async copy."""

    def __init__(self, micro_batch: int, seq_len: int, device, with_mtp: bool, dev_slots: int = 1):
        """``dev_slots`` device-side copies are kept (a pipeline schedule holds every micro-batch of a step until its
        backward pass has run); ``stage(b, slot)`` picks which one the copy lands in."""
        self.B, self.S, self.device = micro_batch, seq_len, torch.device(device)
        n = micro_batch * seq_len
        self.fields = ["ids", "labels", "mask"] + (["mtp_ids", "mtp_labels", "mtp_mask"] if with_mtp else [])
        self.nbytes = 4 * n * len(self.fields)
        pin = self.device.type == "cuda"
        self.hosts = [torch.empty(self.nbytes, dtype=torch.uint8, pin_memory=pin) for _ in range(2 if pin else 1)]
        self.events = [None] * len(self.hosts)
        self.turn = 0
        self._n = n
        self._pin = pin
        self.devs, self.dviews_all = [], []
        for _ in range(max(1, dev_slots)):
            dev = torch.empty(self.nbytes, dtype=torch.uint8, device=self.device) if pin else \
                torch.empty(self.nbytes, dtype=torch.uint8)
            views = {}
            for i, f in enumerate(self.fields):
                dt = torch.float32 if f.endswith("mask") else torch.int32
                views[f] = dev[4 * n * i: 4 * n * (i + 1)].view(dt)
            self.devs.append(dev)
            self.dviews_all.append(views)
        self.dev, self.dviews = self.devs[0], self.dviews_all[0]

    def _hviews(self, host):
        n, out = self._n, {}
        for i, f in enumerate(self.fields):
            dt = torch.float32 if f.endswith("mask") else torch.int32
            out[f] = host[4 * n * i: 4 * n * (i + 1)].view(dt)
        return out

    def stage(self, b: dict, slot: int = 0) -> dict:
        """``b`` holds CPU ``tokens``/``labels``/``loss_mask`` ``[B, S]``.  Fills one of two pinned
        buffers (waiting only for that buffer's previous copy) and enqueues one async H2D copy on
        the current stream into device copy ``slot``.  Returns device views."""
        k = self.turn
        self.turn = (self.turn + 1) % len(self.hosts)
        if self.events[k] is not None:
            self.events[k].synchronize()
        hv = self._hviews(self.hosts[k])
        hv["ids"].copy_(b["tokens"].reshape(-1))
        hv["labels"].copy_(b["labels"].reshape(-1))
        hv["mask"].copy_(b["loss_mask"].reshape(-1))
        if "mtp_ids" in hv:
            mi, ml, mm = build_mtp_tensors(b["tokens"], b["labels"], b["loss_mask"])
            hv["mtp_ids"].copy_(mi.reshape(-1))
            hv["mtp_labels"].copy_(ml.reshape(-1))
            hv["mtp_mask"].copy_(mm.reshape(-1))
        dev = self.devs[slot]
        if self._pin:
            dev.copy_(self.hosts[k], non_blocking=True)
            if self.events[k] is None:
                self.events[k] = torch.cuda.Event()
            self.events[k].record()
        else:
            dev.copy_(self.hosts[k])
        out = dict(self.dviews_all[slot])
        out["seq_len"] = self.S
        return out
