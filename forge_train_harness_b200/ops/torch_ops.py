"""Plain-PyTorch implementation of every engine op, forward and hand-derived backward.

This is the ``baseline`` version of each op: the numerical oracle the sm_100a kernels
are tested against, the CPU/gloo execution path, and the bring-up path.  No autograd
is used; every backward is the closed form.  The math follows the reference's
primitives (workload/src/training_engine_tensor/forward.py:32-350, backward.py:51-620):
norm / SwiGLU / softmax / cross-entropy in fp32, weight gradients accumulated in fp32
into a ``main_grad`` buffer, activations and input gradients in the compute dtype.

All activations are 2-D ``[M, features]`` with ``M = batch * seq`` tokens, batch-major.
The QKV activation is packed kv-group-major: for each KV group ``j`` the columns are
``[q_{j,0} .. q_{j,g-1} | k_j | v_j]``, each ``head_dim`` wide (forward.py:74-93).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rope_table(seq_len: int, head_dim: int, theta: float, device=None) -> torch.Tensor:
    """fp32 ``[S, head_dim]`` table: ``[:, :d/2] = cos``, ``[:, d/2:] = sin`` of ``pos * theta^(-2i/d)``."""
    half = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32, device=device) * 2.0 / head_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float32, device=device), inv)
    return torch.cat([ang.cos(), ang.sin()], dim=1).contiguous()


class TorchOps:
    name = "baseline"

    # ---- embedding -------------------------------------------------------
    @staticmethod
    def embedding_fwd(ids, weight, scale, vocab_start=0, sharded=False):
        """rows of ``weight`` gathered by ``ids - vocab_start`` (zero outside the shard), times ``scale``."""
        local = ids.long() - vocab_start
        out = F.embedding(local.clamp(0, weight.shape[0] - 1), weight).float() * scale
        if sharded:
            ok = (local >= 0) & (local < weight.shape[0])
            out = out * ok.unsqueeze(-1)
        return out.to(weight.dtype)

    @staticmethod
    def check_ids(ids, lo, hi):
        """Debug input check, host side: raises at once (the CUDA version reports through the status word)."""
        bad = ((ids < lo) | (ids >= hi)).nonzero()
        if bad.numel():
            pos = int(bad[0, 0])
            raise ValueError(f"index {int(ids.reshape(-1)[pos])} at position {pos} lies outside [{lo}, {hi})")

    @staticmethod
    def embedding_bwd(dout, ids, main_grad, scale, vocab_start=0):
        local = ids.long() - vocab_start
        ok = (local >= 0) & (local < main_grad.shape[0])
        g = dout.float() * scale * ok.unsqueeze(-1)
        main_grad.index_add_(0, local.clamp(0, main_grad.shape[0] - 1), g)

    # ---- RMSNorm ---------------------------------------------------------
    @staticmethod
    def rmsnorm_fwd(x, w, eps, out_scale=1.0):
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
        y = xf * rstd.unsqueeze(-1) * w.float() * out_scale
        return y.to(x.dtype), rstd

    @staticmethod
    def residual_rmsnorm_fwd(h, a, scale, w, eps, out_scale=1.0):
        """``r = h + a*scale`` (rounded to the compute dtype), then RMSNorm of ``r``."""
        r = (h.float() + a.float() * scale).to(h.dtype)
        y, rstd = TorchOps.rmsnorm_fwd(r, w, eps, out_scale)
        return r, y, rstd

    @staticmethod
    def residual_add(h, a, scale):
        return (h.float() + a.float() * scale).to(h.dtype)

    @staticmethod
    def rmsnorm_bwd(dy, x, w, rstd, dw_main_grad, dres=None, out_scale=1.0):
        """``dx = rstd * (g*w - xhat * mean(g*w*xhat))`` (+ ``dres``); ``dw += sum(g * xhat)``."""
        g = dy.float() * out_scale
        xhat = x.float() * rstd.unsqueeze(-1)
        gw = g * w.float()
        dx = rstd.unsqueeze(-1) * (gw - xhat * (gw * xhat).mean(-1, keepdim=True))
        if dres is not None:
            dx = dx + dres.float()
        dw_main_grad.add_((g * xhat).sum(0))
        return dx.to(x.dtype)

    # ---- linear ----------------------------------------------------------
    @staticmethod
    def linear_fwd(x, w, alpha=1.0):
        y = x @ w.t()
        return y if alpha == 1.0 else (y.float() * alpha).to(y.dtype)

    @staticmethod
    def linear_dgrad(dy, w, alpha=1.0):
        dx = dy @ w
        return dx if alpha == 1.0 else (dx.float() * alpha).to(dx.dtype)

    @staticmethod
    def linear_wgrad(dy, x, main_grad, alpha=1.0):
        """``main_grad += alpha * dy^T x`` with fp32 accumulation."""
        if dy.dtype == torch.float32:
            main_grad.addmm_(dy.t(), x, alpha=alpha)
        else:
            main_grad.add_((dy.t() @ x).float(), alpha=alpha)

    # ---- RoPE (rotate-half over the full head_dim), in place on q and k ----
    @staticmethod
    def _rope(qkv, table, seq_len, n_kv, g, d, sign):
        M = qkv.shape[0]
        v = qkv.view(M // seq_len, seq_len, n_kv, g + 2, d)
        half = d // 2
        cos = table[:seq_len, :half].view(1, seq_len, 1, 1, half)
        sin = table[:seq_len, half:].view(1, seq_len, 1, 1, half) * sign
        qk = v[:, :, :, : g + 1, :].float()
        x1, x2 = qk[..., :half], qk[..., half:]
        o = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
        v[:, :, :, : g + 1, :] = o.to(qkv.dtype)
        return qkv

    @staticmethod
    def rope_fwd_(qkv, table, seq_len, n_kv, g, d):
        return TorchOps._rope(qkv, table, seq_len, n_kv, g, d, 1.0)

    @staticmethod
    def rope_bwd_(dqkv, table, seq_len, n_kv, g, d):
        return TorchOps._rope(dqkv, table, seq_len, n_kv, g, d, -1.0)

    # ---- per-head q/k RMSNorm (Qwen3), in place on the packed layout -------
    @staticmethod
    def qk_norm_fwd(qkv, wq, wk, eps, n_kv, g, d):
        M = qkv.shape[0]
        v = qkv.view(M, n_kv, g + 2, d)
        qk = v[:, :, : g + 1, :].float()
        rstd = torch.rsqrt(qk.pow(2).mean(-1) + eps)  # [M, n_kv, g+1]
        w = torch.cat([wq.float().expand(g, d), wk.float().view(1, d)], 0)  # [g+1, d]
        out = qkv.clone()
        out.view(M, n_kv, g + 2, d)[:, :, : g + 1, :] = (qk * rstd.unsqueeze(-1) * w).to(qkv.dtype)
        return out, rstd

    @staticmethod
    def qk_norm_bwd(dqkv, qkv_pre, rstd, wq, wk, dwq_main, dwk_main, n_kv, g, d):
        M = dqkv.shape[0]
        gq = dqkv.view(M, n_kv, g + 2, d)[:, :, : g + 1, :].float()
        x = qkv_pre.view(M, n_kv, g + 2, d)[:, :, : g + 1, :].float()
        w = torch.cat([wq.float().expand(g, d), wk.float().view(1, d)], 0)
        xhat = x * rstd.unsqueeze(-1)
        gw = gq * w
        dx = rstd.unsqueeze(-1) * (gw - xhat * (gw * xhat).mean(-1, keepdim=True))
        dwfull = (gq * xhat).sum((0, 1))  # [g+1, d]
        dwq_main.add_(dwfull[:g].sum(0))
        dwk_main.add_(dwfull[g])
        out = dqkv.clone()
        out.view(M, n_kv, g + 2, d)[:, :, : g + 1, :] = dx.to(dqkv.dtype)
        return out

    # ---- causal GQA attention on the packed layout -------------------------
    @staticmethod
    def _split(qkv, seq_len, n_kv, g, d):
        M = qkv.shape[0]
        B = M // seq_len
        v = qkv.view(B, seq_len, n_kv, g + 2, d)
        q = v[:, :, :, :g, :].permute(0, 2, 3, 1, 4)  # [B, n_kv, g, S, d]
        k = v[:, :, :, g, :].permute(0, 2, 1, 3)  # [B, n_kv, S, d]
        vv = v[:, :, :, g + 1, :].permute(0, 2, 1, 3)
        return q, k, vv

    @staticmethod
    def attention_fwd(qkv, seq_len, n_kv, g, d):
        """Returns ``out [M, n_kv*g*d]`` (head order = kv group major) and ``lse [B, n_kv*g, S]`` fp32."""
        q, k, v = TorchOps._split(qkv, seq_len, n_kv, g, d)
        B = q.shape[0]
        s = torch.einsum("bjgsd,bjtd->bjgst", q.float(), k.float()) / math.sqrt(d)
        mask = torch.ones(seq_len, seq_len, dtype=torch.bool, device=qkv.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
        lse = torch.logsumexp(s, dim=-1)  # [B, n_kv, g, S]
        p = torch.exp(s - lse.unsqueeze(-1))
        o = torch.einsum("bjgst,bjtd->bjgsd", p, v.float())
        out = o.permute(0, 3, 1, 2, 4).reshape(B * seq_len, n_kv * g * d).to(qkv.dtype)
        return out, lse.reshape(B, n_kv * g, seq_len).contiguous()

    @staticmethod
    def attention_bwd(dout, qkv, out, lse, seq_len, n_kv, g, d):
        """Returns the packed ``dqkv`` (same layout as ``qkv``)."""
        q, k, v = TorchOps._split(qkv, seq_len, n_kv, g, d)
        B = q.shape[0]
        qf, kf, vf = q.float(), k.float(), v.float()
        do = dout.view(B, seq_len, n_kv, g, d).permute(0, 2, 3, 1, 4).float()
        o = out.view(B, seq_len, n_kv, g, d).permute(0, 2, 3, 1, 4).float()
        scale = 1.0 / math.sqrt(d)
        s = torch.einsum("bjgsd,bjtd->bjgst", qf, kf) * scale
        mask = torch.ones(seq_len, seq_len, dtype=torch.bool, device=qkv.device).tril()
        p = torch.exp(s - lse.view(B, n_kv, g, seq_len, 1)).masked_fill(~mask, 0.0)
        dv = torch.einsum("bjgst,bjgsd->bjtd", p, do)
        dp = torch.einsum("bjgsd,bjtd->bjgst", do, vf)
        delta = (do * o).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dq = torch.einsum("bjgst,bjtd->bjgsd", ds, kf)
        dk = torch.einsum("bjgst,bjgsd->bjtd", ds, qf)
        dqkv = torch.empty_like(qkv)
        dv5 = dqkv.view(B, seq_len, n_kv, g + 2, d)
        dv5[:, :, :, :g, :] = dq.permute(0, 3, 1, 2, 4).to(qkv.dtype)
        dv5[:, :, :, g, :] = dk.permute(0, 2, 1, 3).to(qkv.dtype)
        dv5[:, :, :, g + 1, :] = dv.permute(0, 2, 1, 3).to(qkv.dtype)
        return dqkv

    @staticmethod
    def attention_rope_bwd(dout, qkv, out, lse, table, seq_len, n_kv, g, d):
        dqkv = TorchOps.attention_bwd(dout, qkv, out, lse, seq_len, n_kv, g, d)
        return TorchOps.rope_bwd_(dqkv, table, seq_len, n_kv, g, d)

    # ---- SwiGLU on packed [gate | up] ------------------------------------
    @staticmethod
    def swiglu_fwd(gate_up):
        g, u = gate_up.float().chunk(2, dim=-1)
        return (F.silu(g) * u).to(gate_up.dtype)

    @staticmethod
    def swiglu_bwd(dinter, gate_up):
        g, u = gate_up.float().chunk(2, dim=-1)
        d = dinter.float()
        sig = torch.sigmoid(g)
        dg = d * u * sig * (1.0 + g * (1.0 - sig))
        du = d * g * sig
        return torch.cat([dg, du], dim=-1).to(gate_up.dtype)

    # ---- fused cross-entropy: loss + in-place logits gradient --------------
    @staticmethod
    def cross_entropy_fwd_bwd(logits, labels, mask, grad_scale=1.0, vocab_start=0, tp_group=None):
        """Per-token NLL (fp32 ``[M]``, zero where ``mask`` is 0); ``logits`` is overwritten by
        ``(softmax - onehot) * mask * grad_scale``.  With a TP group the vocabulary is sharded
        (columns ``vocab_start ..``) and max / sum-exp / target-logit are reduced over the group
        (model_minicpm4_8b_tp.py:350-398)."""
        import torch.distributed as dist
        lf = logits.float()
        mx = lf.max(-1).values
        if tp_group is not None:
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=tp_group)
        ex = torch.exp(lf - mx.unsqueeze(-1))
        se = ex.sum(-1)
        local = labels.long() - vocab_start
        ok = (local >= 0) & (local < logits.shape[1])
        tgt = lf.gather(1, local.clamp(0, logits.shape[1] - 1).unsqueeze(1)).squeeze(1) * ok
        if tp_group is not None:
            dist.all_reduce(se, group=tp_group)
            dist.all_reduce(tgt, group=tp_group)
        mf = mask.float()
        nll = (torch.log(se) + mx - tgt) * mf
        grad = ex / se.unsqueeze(-1)
        rows = torch.nonzero(ok, as_tuple=False).squeeze(1)
        grad[rows, local[rows]] -= 1.0
        grad = grad * (mf * grad_scale).unsqueeze(-1)
        logits.copy_(grad.to(logits.dtype))
        return nll

    # ---- AdamW on fp32 master + low-precision write-back --------------------
    @staticmethod
    def adamw_segments(master, m, v, grad_flat, param_flat, segs, lr, beta1, beta2, eps, weight_decay, step,
                       grad_scale, table=None):
        """Decoupled-weight-decay Adam (``torch._fused_adamw_`` semantics, train_loop.py:1227-1231).

        ``master/m/v`` are this rank's flat fp32 shard; each segment ``(shard_off, flat_off, n,
        lr_mult, wd_on)`` maps a run of the shard to the flat gradient / parameter buffers.  The
        gradient is multiplied by ``grad_scale`` (0-dim tensor: clip coefficient / token count)
        and ``param_flat`` receives the master rounded to the compute dtype."""
        bc1 = 1.0 - beta1 ** step
        bc2 = 1.0 - beta2 ** step
        for so, fo, n, lr_mult, wd_on in segs:
            w, mm, vv = master[so:so + n], m[so:so + n], v[so:so + n]
            g = grad_flat[fo:fo + n] * grad_scale
            l = lr * lr_mult
            w.mul_(1.0 - l * (weight_decay if wd_on else 0.0))
            mm.lerp_(g, 1.0 - beta1)
            vv.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
            denom = (vv.sqrt() / math.sqrt(bc2)).add_(eps)
            w.addcdiv_(mm, denom, value=-l / bc1)
            param_flat[fo:fo + n].copy_(w)

    @staticmethod
    def sumsq(x):
        return x.float().pow(2).sum()
