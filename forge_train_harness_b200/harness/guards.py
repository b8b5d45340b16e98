"""Static guards over the engine sources.

``framework_guard``: the hot path must stay a hand-derived engine — no autograd, no ``nn.Module`` models, no stock optimizers,
no mixed-precision autocast, no third-party training frameworks (the reference's banned-keyword scan,
harness/framework_guard.py:79-109).  ``anti_proxy_guard``: the engine must not import, shell out to, or read the reference
baseline, nor hard-code gate metrics (harness/anti_proxy_guard.py:43-80).  Comments and docstrings are ignored; the oracle op
set (``ops/torch_ops.py``) may use ``torch.nn.functional`` because it is the reference implementation tests compare against.
"""
from __future__ import annotations

import io
import os
import re
import tokenize

BANNED = ["megatron", "deepspeed", "torch.nn.Module", "torch.optim", "torch.autograd", "torch.utils.data", "torch.amp",
          ".backward(", "requires_grad=True", "torch.compile", "import triton"]
PROXY = ["baseline._ref", "baseline/_ref", "training_engine_tensor", "train_pure_mup_mtp", "model_pure_mup_mtp"]
PROXY += [p for p in os.environ.get("FORGE_REFERENCE_ROOTS", "").split(os.pathsep) if p]   # checkout paths of the reference, if any
ENGINE_DIRS = ["models", "ops", "optim", "parallel", "data", "ckpt", "engine.py", "train.py"]
# the corpus FORMAT is called Megatron binary, and the exporter writes checkpoints under Megatron-LM's state-dict names:
# both name a file format, neither imports the framework
ALLOW = {"ops/torch_ops.py": {"torch.nn.Module"}, "data/sources.py": {"megatron"}, "data/prepare.py": {"megatron"},
         "ckpt/export_megatron.py": {"megatron"}, "ckpt/import_weights.py": {"megatron"}}


def _code_only(src: str) -> str:
    """Source with comments and string literals (docstrings) blanked out."""
    out = []
    try:
        for tok in tokenize.generate_tokens(io.StringIO(src).readline):
            if tok.type in (tokenize.COMMENT, tokenize.STRING):
                continue
            out.append(tok.string)
    except tokenize.TokenError:
        return src
    return " ".join(out)


def _files(root: str):
    for d in ENGINE_DIRS:
        p = os.path.join(root, d)
        if os.path.isfile(p):
            yield d, p
        for dp, _, fns in os.walk(p):
            for fn in fns:
                if fn.endswith(".py"):
                    full = os.path.join(dp, fn)
                    yield os.path.relpath(full, root), full


def scan(root: str, words: list[str]) -> list[tuple[str, str]]:
    hits = []
    for rel, full in _files(root):
        code = re.sub(r"\s+", "", _code_only(open(full).read()))
        for w in words:
            if w in ALLOW.get(rel, set()):
                continue
            if re.sub(r"\s+", "", w) in code:
                hits.append((rel, w))
    return hits


def framework_guard(root: str | None = None) -> dict:
    root = root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hits = scan(root, BANNED)
    return {"passed": not hits, "violations": hits}


def anti_proxy_guard(root: str | None = None) -> dict:
    root = root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hits = scan(root, PROXY)
    return {"passed": not hits, "violations": hits}
