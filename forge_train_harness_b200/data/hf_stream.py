"""Streaming tokenize + mix + pack data source over local parquet / JSON-lines files (``data_loader = "hf"``).

The reference's real-pretraining data path is a streaming HuggingFace ``datasets`` pipeline driven by ``hf://`` tokens in
the data path (ref/reference/hf_stream_dataloader.py:166-277): per-dataset ingestion (a text column or a named template),
SentencePiece ``encode(text) + [eos]`` without BOS and with empty documents skipped, weighted interleave of the sources,
a seeded shuffle buffer, a split of the document stream over the DP ranks, and packing of the token stream into
non-overlapping ``seq + 1`` windows.  This is the engine's own equivalent with no ``datasets`` / ``torch.utils.data``
dependency: documents come from pyarrow (parquet) or JSON-lines readers over a frozen sorted file list, so the order is a
pure function of ``(files, seed)``.  Same token grammar::

    <weight> hf://<repo>?split=<sp>&text=<col>[&template=<name>][&local_env=<ENV>][&glob=<pat>]

``local_env`` names an environment variable holding the directory of the files (the reference's offline switch); there is
no Hub access here, so a token without a usable directory is an error.  The tokenizer is a SentencePiece model file
(``FORGE_TOKENIZER`` or ``tokenizer=`` in the token); ``tokenizer=bytes`` selects a byte-level stand-in (ids 0..255, EOS
256) for tests and synthetic corpora.

Differences from the reference, on purpose: the position is RESUMABLE (documents consumed per epoch + the unpacked token
tail are in ``state_dict``; the reference re-reads from the start), and ``FORGE_HF_DATA_DUMP=1`` prints the same
``[DATAHASH] rank= batch= sha256=`` line per batch for the bitwise self-check (hf_stream_dataloader.py:262-270).
"""
from __future__ import annotations

import glob as _glob
import hashlib
import json
import os
from dataclasses import dataclass
from urllib.parse import parse_qs, urlparse

import numpy as np
import torch


def _gsm8k_qa(row) -> str:
    return f"Question: {row['question']}\nAnswer: {row['answer']}"


TEMPLATES = {"gsm8k_qa": _gsm8k_qa}


@dataclass
class SourceSpec:
    weight: float
    repo: str
    split: str
    text_col: str | None = None
    template: str | None = None
    local_env: str | None = None
    glob: str = "*.parquet"
    tokenizer: str | None = None

    def text_of(self, row: dict) -> str:
        if self.template is not None:
            fn = TEMPLATES.get(self.template)
            if fn is None:
                raise KeyError(f"unknown text template {self.template!r}; known: {sorted(TEMPLATES)}")
            return fn(row)
        if self.text_col is not None:
            return str(row.get(self.text_col, "") or "")
        raise ValueError(f"source {self.repo} has neither text= nor template= in its hf:// token")

    def files(self) -> list[str]:
        root = os.environ.get(self.local_env, "") if self.local_env else ""
        if not root or not os.path.isdir(root):
            raise FileNotFoundError(f"hf://{self.repo}: no local directory ({self.local_env or 'local_env'} is not set to one) and "
                                    "there is no network access to the Hub here")
        fs = sorted(_glob.glob(os.path.join(root, self.glob)))
        if not fs:
            raise FileNotFoundError(f"{self.local_env}={root}: no files match {self.glob!r}")
        return fs


def parse_token(weight: float, token: str) -> SourceSpec:
    if not token.startswith("hf://"):
        raise ValueError(f"not an hf:// token: {token!r}")
    u = urlparse(token)
    q = {k: v[0] for k, v in parse_qs(u.query).items()}
    if not q.get("split"):
        raise ValueError(f"hf:// token missing required split=: {token!r}")
    return SourceSpec(weight, (u.netloc + u.path).rstrip("/"), q["split"], q.get("text"), q.get("template"), q.get("local_env"),
                      q.get("glob", "*.parquet"), q.get("tokenizer"))


def parse_data_path(data_path: str) -> list[SourceSpec]:
    """``"1.0 hf://a?... 0.5 hf://b?..."`` (or the path of a file holding that) -> specs."""
    raw = open(data_path).read().split() if os.path.isfile(data_path) else data_path.split()
    if len(raw) % 2:
        raise ValueError("data path must be whitespace-separated '<weight> <token>' pairs")
    return [parse_token(float(raw[i]), raw[i + 1]) for i in range(0, len(raw), 2)]


class _ByteTokenizer:
    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def eos_id(self) -> int:
        return 256


def load_tokenizer(name: str | None):
    name = name or os.environ.get("FORGE_TOKENIZER", "")
    if name == "bytes":
        return _ByteTokenizer()
    if not name or not os.path.isfile(name):
        raise FileNotFoundError("no tokenizer: set FORGE_TOKENIZER (or tokenizer= in the hf:// token) to a SentencePiece model file, "
                                "or to 'bytes' for the byte-level stand-in")
    import sentencepiece as spm
    sp = spm.SentencePieceProcessor()
    sp.Load(name)
    return sp


def _rows_of(path: str):
    if path.endswith((".jsonl", ".json")):
        with open(path) as f:
            for ln in f:
                if ln.strip():
                    yield json.loads(ln)
        return
    import pyarrow.parquet as pq
    pf = pq.ParquetFile(path)
    for batch in pf.iter_batches(batch_size=1024):
        yield from batch.to_pylist()


class HFStream:
    """Infinite deterministic packer.  Order: per epoch, documents are drawn from the sources by a seeded weighted choice
    (``all_exhausted``: a drained source is re-opened until every source has been read once), pass through a seeded shuffle
    buffer, and document ``i`` of that stream goes to DP rank ``i % dp_size``."""

    def __init__(self, specs: list[SourceSpec], seq_len: int, micro_batch: int, dp_rank: int, dp_size: int, seed: int,
                 buffer_size: int = 10000):
        self.specs, self.seq_len, self.mbs, self.dp_rank, self.dp_size, self.seed = specs, seq_len, micro_batch, dp_rank, dp_size, seed
        self.buffer_size = buffer_size
        self.tok = load_tokenizer(next((s.tokenizer for s in specs if s.tokenizer), None))
        self.eos = int(self.tok.eos_id())
        if self.eos < 0:
            raise ValueError("tokenizer has no EOS id")
        self.dump = bool(os.environ.get("FORGE_HF_DATA_DUMP", ""))
        self.epoch, self.docs_taken, self.tail, self.batch_idx = 0, 0, [], 0
        self._docs = None

    # ---- document stream -------------------------------------------------------------------------------------------------
    def _mixed(self, epoch: int):
        rng = np.random.RandomState((self.seed + epoch) % (2 ** 31))
        iters = [self._source_rows(s) for s in self.specs]
        done = [False] * len(iters)
        w = np.array([s.weight for s in self.specs], dtype=np.float64)
        w /= w.sum()
        while not all(done):
            i = int(rng.choice(len(iters), p=w)) if len(iters) > 1 else 0
            try:
                yield self.specs[i], next(iters[i])
            except StopIteration:
                done[i] = True
                if all(done):
                    return
                iters[i] = self._source_rows(self.specs[i])   # all_exhausted: keep the mix until every source was read once

    @staticmethod
    def _source_rows(spec: SourceSpec):
        for f in spec.files():
            yield from _rows_of(f)

    def _shuffled(self, epoch: int):
        rng = np.random.RandomState((self.seed + epoch + 7919) % (2 ** 31))
        buf = []
        for item in self._mixed(epoch):
            if len(buf) < self.buffer_size:
                buf.append(item)
                continue
            j = int(rng.randint(0, self.buffer_size))
            yield buf[j]
            buf[j] = item
        rng.shuffle(buf)
        yield from buf

    def _my_docs(self):
        """This rank's documents of the current epoch from ``docs_taken`` on, as token lists (+ EOS); empty ones skipped."""
        while True:
            produced = False
            for i, (spec, row) in enumerate(self._shuffled(self.epoch)):
                if i % self.dp_size != self.dp_rank:
                    continue
                k = i // self.dp_size
                if k < self.docs_taken:
                    produced = True
                    continue
                ids = list(self.tok.encode(spec.text_of(row)))
                self.docs_taken = k + 1
                if not ids:
                    continue
                produced = True
                yield ids + [self.eos]
            if not produced:
                raise RuntimeError("the data sources produced no non-empty documents: check text= / template= and the files")
            self.epoch += 1
            self.docs_taken = 0

    # ---- batches ----------------------------------------------------------------------------------------------------------
    def state_dict(self):
        return {"kind": "hf", "epoch": self.epoch, "docs_taken": self.docs_taken, "tail": list(self.tail), "batch_idx": self.batch_idx,
                "dp_size": self.dp_size}

    def load_state_dict(self, sd):
        if int(sd.get("dp_size", self.dp_size)) != self.dp_size:
            raise ValueError("a streaming data position belongs to the DP degree it was saved at")
        self.epoch, self.docs_taken, self.tail, self.batch_idx = int(sd["epoch"]), int(sd["docs_taken"]), list(sd["tail"]), int(sd["batch_idx"])
        self._docs = None

    def seek_microbatches(self, n: int):
        self.epoch, self.docs_taken, self.tail, self.batch_idx, self._docs = 0, 0, [], 0, None
        for _ in range(int(n)):
            next(self)

    def __iter__(self):
        return self

    def __next__(self):
        if self._docs is None:
            self._docs = self._my_docs()
        win = self.seq_len + 1
        need = self.mbs * win
        while len(self.tail) < need:
            self.tail.extend(next(self._docs))
        arr = np.asarray(self.tail[:need], dtype=np.int64).reshape(self.mbs, win)
        self.tail = self.tail[need:]
        tokens, labels = torch.from_numpy(arr[:, :-1].copy()), torch.from_numpy(arr[:, 1:].copy())
        if self.dump:
            h = hashlib.sha256()
            h.update(tokens.numpy().tobytes())
            h.update(labels.numpy().tobytes())
            print(f"[DATAHASH] rank={self.dp_rank} batch={self.batch_idx} sha256={h.hexdigest()}", flush=True)
        self.batch_idx += 1
        return {"tokens": tokens, "labels": labels, "loss_mask": torch.ones(self.mbs, self.seq_len, dtype=torch.float32)}


def build_modelbest(*_args, **_kw):
    """``data_loader = "modelbest"``: the reference's third loader wraps the proprietary ``modelbest_sdk`` SSTable reader
    (train_loop.py:240-272).  The SDK is not part of this image; the branch exists so that a configuration naming it fails
    with the reason instead of an unknown-loader error."""
    try:
        import modelbest_sdk  # noqa: F401
    except ImportError as e:
        raise RuntimeError("data_loader = 'modelbest' needs the modelbest_sdk package, which is not installed; convert the corpus to "
                           "the Megatron .bin/.idx format (data_loader = 'megatron_binary') or to parquet (data_loader = 'hf')") from e
    raise RuntimeError("modelbest_sdk is importable but no adapter for it is wired in this build")
