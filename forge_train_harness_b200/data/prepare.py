"""Tokenise documents into the Megatron indexed ``.bin/.idx`` format (``data_loader = "megatron_binary"``).

    python -m forge_train_harness_b200.data.prepare --out <prefix> --tokenizer <sentencepiece.model | bytes> \
        [--text content | --template gsm8k_qa] <files: .parquet / .jsonl ...>

The reference prepares its GSM8K corpus the same way (ref/reference/gsm8k_prepare_torch.py, prepare_gsm8k_data.sh):
``encode(text) + [eos]`` per document, no BOS, empty documents skipped, one sequence per document.  The encode contract is
shared with the streaming loader (``data/hf_stream.py``), so a corpus prepared here and the same files streamed produce the
same token sequence.
"""
from __future__ import annotations

import argparse
import sys

import numpy as np

from .hf_stream import SourceSpec, _rows_of, load_tokenizer
from .sources import write_megatron_binary


def encode_documents(files, tokenizer, spec: SourceSpec) -> list[np.ndarray]:
    eos = int(tokenizer.eos_id())
    docs = []
    for f in files:
        for row in _rows_of(f):
            ids = list(tokenizer.encode(spec.text_of(row)))
            if ids:
                docs.append(np.asarray(ids + [eos], dtype=np.int32))
    return docs


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("files", nargs="+")
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--text", default=None)
    ap.add_argument("--template", default=None)
    a = ap.parse_args(argv)
    spec = SourceSpec(1.0, "local", "train", a.text, a.template)
    docs = encode_documents(sorted(a.files), load_tokenizer(a.tokenizer), spec)
    if not docs:
        print("no non-empty documents", file=sys.stderr)
        return 1
    write_megatron_binary(a.out, docs, np.int32)
    print(f"{len(docs)} documents, {sum(len(d) for d in docs)} tokens -> {a.out}.bin/.idx")
    return 0


if __name__ == "__main__":
    sys.exit(main())
