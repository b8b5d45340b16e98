"""``sm100`` op versions: thin Python wrappers over the in-tree sm_100a extension ``_C``.

Importing this module REQUIRES the extension (``forge_train_harness_b200/_C.so``, built by
``python -m forge_train_harness_b200.csrc.build``); there is no silent fallback.  Tensors are bf16
activations / weights and fp32 gradients, laid out as ``torch_ops`` documents.
"""
from __future__ import annotations

import importlib.util
import math
import os
import struct

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SO = os.path.join(_PKG, "_C.so")


def _load():
    if not os.path.exists(_SO):
        from ..csrc.build import build
        build()
    spec = importlib.util.spec_from_file_location("forge_train_harness_b200._C", _SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_C = _load()

ADAM_CHUNK = 8192  # elements per thread block of the segment AdamW kernel


from .status import STATUS_NAMES  # noqa: E402


def check_status(reset: bool = True) -> None:
    """Raise if any kernel reported a bounded wait that gave up (host sync: call after an event sync)."""
    code = _C.read_status(reset)
    if code:
        raise RuntimeError(f"sm_100a kernel reported status {code}: {STATUS_NAMES.get(code, 'unknown')}")


class Sm100Ops:
    name = "sm100"

    # ---- debug input checks ---------------------------------------------
    @staticmethod
    def check_ids(ids, lo, hi):
        """Every id in [lo, hi), else status 7 at the next status read (no host sync here: usable inside a CUDA graph)."""
        _C.check_ids(ids, int(lo), int(hi))

    @staticmethod
    def bad_index_position(reset=True):
        return int(_C.bad_index_position(bool(reset)))

    # ---- embedding -------------------------------------------------------
    @staticmethod
    def embedding_fwd(ids, weight, scale, vocab_start=0, sharded=False):
        return _C.embedding_fwd(ids, weight, float(scale), int(vocab_start))

    deterministic = False  # set by the engine from train.deterministic: fixed summation orders, no float atomics

    @staticmethod
    def set_deterministic(on: bool) -> None:
        """Deterministic mode: the embedding backward sums each token's rows in a fixed order instead of with float
        atomics, and accumulating GEMMs use one k split per output tile (fixed reduce-add order).  The attention
        backward still sums its partial dQ / dK / dV tiles with reduce-adds whose order is not fixed."""
        Sm100Ops.deterministic = bool(on)
        _C.gemm_set_deterministic(bool(on))

    @staticmethod
    def embedding_bwd(dout, ids, main_grad, scale, vocab_start=0):
        if not Sm100Ops.deterministic:
            _C.embedding_bwd(dout, ids, main_grad, float(scale), int(vocab_start))
            return
        local = ids.to(torch.int64) - int(vocab_start)
        keep = (local >= 0) & (local < main_grad.shape[0])
        rows = torch.nonzero(keep, as_tuple=False).reshape(-1)
        if rows.numel() == 0:
            return
        sorted_ids, perm = torch.sort(local[rows], stable=True)
        order = rows[perm].to(torch.int32)
        seg_id, counts = torch.unique_consecutive(sorted_ids, return_counts=True)
        seg_start = torch.zeros(seg_id.numel() + 1, dtype=torch.int32, device=ids.device)
        seg_start[1:] = torch.cumsum(counts, 0).to(torch.int32)
        _C.embedding_bwd_det(dout, order, seg_start, seg_id.to(torch.int32), main_grad, float(scale))

    # ---- RMSNorm ---------------------------------------------------------
    @staticmethod
    def rmsnorm_fwd(x, w, eps, out_scale=1.0, y_out=None):
        y, rstd = _C.rmsnorm_fwd(x, None, 0.0, w, float(eps), float(out_scale), y_out)
        return y, rstd

    @staticmethod
    def residual_rmsnorm_fwd(h, a, scale, w, eps, out_scale=1.0, y_out=None):
        r, y, rstd = _C.rmsnorm_fwd(h, a, float(scale), w, float(eps), float(out_scale), y_out)
        return r, y, rstd

    @staticmethod
    def residual_add(h, a, scale):
        return _C.residual_add(h, a, float(scale))

    @staticmethod
    def rmsnorm_bwd(dy, x, w, rstd, dw_main_grad, dres=None, out_scale=1.0):
        return _C.rmsnorm_bwd(dy, x, w, rstd, dres, dw_main_grad, float(out_scale))

    # ---- linear: tcgen05 GEMMs --------------------------------------------
    @staticmethod
    def linear_fwd(x, w, alpha=1.0):
        n = w.shape[0]
        if n % 8:
            # a vocabulary shard such as 73448 / 4 = 18362 columns: the TMA store needs 16-byte row pitch, so the result is
            # a view of a row-padded buffer; its consumers (fused CE, dgrad / wgrad GEMMs) take the row stride
            buf = torch.empty((x.shape[0], (n + 7) // 8 * 8), dtype=torch.bfloat16, device=x.device)
            return _C.gemm(x, False, w, False, buf[:, :n], float(alpha), 0, 0, 0)
        return _C.gemm(x, False, w, False, None, float(alpha), 0, 0, 0)

    @staticmethod
    def linear_dgrad(dy, w, alpha=1.0):
        return _C.gemm(dy, False, w, True, None, float(alpha), 0, 0, 0)

    @staticmethod
    def linear_wgrad(dy, x, main_grad, alpha=1.0):
        _C.gemm(dy, True, x, True, main_grad, float(alpha), 1, 0, 0)

    # ---- RoPE ---------------------------------------------------------------
    @staticmethod
    def rope_fwd_(qkv, table, seq_len, n_kv, g, d):
        _C.rope_(qkv, table, seq_len, n_kv, g, d, 1.0)
        return qkv

    # ---- per-head q/k RMSNorm (Qwen3 variant) --------------------------------
    @staticmethod
    def qk_norm_fwd(qkv, wq, wk, eps, n_kv, g, d):
        out, rstd = _C.qk_norm_fwd(qkv, wq, wk, float(eps), int(n_kv), int(g), int(d))
        return out, rstd

    @staticmethod
    def qk_norm_bwd(dqkv, qkv_pre, rstd, wq, wk, dwq_main, dwk_main, n_kv, g, d):
        """In place on ``dqkv`` (returned); the two weight gradients are accumulated into the fp32 main-grad vectors."""
        _C.qk_norm_bwd_(dqkv, qkv_pre, rstd, wq, wk, dwq_main, dwk_main, int(n_kv), int(g), int(d))
        return dqkv

    @staticmethod
    def rope_bwd_(dqkv, table, seq_len, n_kv, g, d):
        _C.rope_(dqkv, table, seq_len, n_kv, g, d, -1.0)
        return dqkv

    # ---- attention -----------------------------------------------------------
    @staticmethod
    def attention_supported(seq_len, d):
        return seq_len % 128 == 0 and d in (64, 128)

    @staticmethod
    def _require_attention_shape(seq_len, d):
        """The flash kernels tile the sequence by 128 and exist for head sizes 64 and 128.  Anything else is refused here:
        quietly handing such a shape to the PyTorch oracle would train on library kernels without anyone noticing (select
        ``OP_ATTENTION_FWD=baseline`` etc. to run the oracle on purpose)."""
        if not Sm100Ops.attention_supported(seq_len, d):
            raise ValueError(f"sm_100a attention needs seq_len to be a multiple of 128 and head_dim 64 or 128 "
                             f"(got seq_len={seq_len}, head_dim={d}); set OP_ATTENTION_FWD / OP_ATTENTION_BWD / "
                             f"OP_ATTENTION_ROPE_BWD=baseline to use the PyTorch implementation")

    @staticmethod
    def attention_fwd(qkv, seq_len, n_kv, g, d):
        Sm100Ops._require_attention_shape(seq_len, d)
        out, lse = _C.flash_fwd(qkv, seq_len, n_kv, g, d)
        return out, lse

    @staticmethod
    def attention_bwd(dout, qkv, out, lse, seq_len, n_kv, g, d):
        Sm100Ops._require_attention_shape(seq_len, d)
        return _C.flash_bwd(dout, qkv, out, lse, None, seq_len, n_kv, g, d)

    @staticmethod
    def attention_rope_bwd(dout, qkv, out, lse, table, seq_len, n_kv, g, d):
        """Attention backward with the RoPE backward folded into the gradient's bf16 write-out."""
        Sm100Ops._require_attention_shape(seq_len, d)
        return _C.flash_bwd(dout, qkv, out, lse, table, seq_len, n_kv, g, d)

    # ---- SwiGLU ---------------------------------------------------------------
    @staticmethod
    def swiglu_fwd(gate_up):
        return _C.swiglu_fwd(gate_up)

    @staticmethod
    def swiglu_bwd(dinter, gate_up):
        return _C.swiglu_bwd(dinter, gate_up)

    # ---- cross-entropy -----------------------------------------------------------
    @staticmethod
    def cross_entropy_fwd_bwd(logits, labels, mask, grad_scale=1.0, vocab_start=0, tp_group=None):
        if tp_group is None:
            return _C.cross_entropy(logits, labels, mask, float(grad_scale), int(vocab_start))
        import torch.distributed as dist
        mx, sm, tg = _C.ce_stats(logits, labels, mask, int(vocab_start))
        gmx = mx.clone()
        dist.all_reduce(gmx, op=dist.ReduceOp.MAX, group=tp_group)
        st = torch.stack([sm * torch.exp(mx - gmx), tg])
        dist.all_reduce(st, group=tp_group)
        lse = gmx + torch.log(st[0])
        _C.ce_grad(logits, labels, mask, lse, float(grad_scale), int(vocab_start))
        return (lse - st[1]) * mask

    # ---- optimizer ---------------------------------------------------------------
    @staticmethod
    def build_adam_table(segs, device):
        rows = []
        for so, fo, n, lr_mult, wd_on in segs:
            off = 0
            while off < n:
                c = min(ADAM_CHUNK, n - off)
                rows.append(struct.pack("<qqiffi", so + off, fo + off, c, float(lr_mult), 1.0 if wd_on else 0.0, 0))
                off += c
        buf = torch.frombuffer(bytearray(b"".join(rows)), dtype=torch.uint8).to(device)
        return buf, len(rows)

    @staticmethod
    def adamw_segments(master, m, v, grad_flat, param_flat, segs, lr, beta1, beta2, eps, weight_decay, step,
                       grad_scale, table=None):
        if table is None:
            table = Sm100Ops.build_adam_table(segs, master.device)
        buf, n = table
        gs = grad_scale.reshape(1).to(torch.float32)
        _C.adamw_segments(master, m, v, grad_flat, param_flat, buf, n, float(lr), float(beta1), float(beta2), float(eps),
                          float(weight_decay), int(step), gs)
        return table

    @staticmethod
    def sumsq(x):
        return _C.sumsq(x.contiguous())
