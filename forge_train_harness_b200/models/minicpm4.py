"""MiniCPM4-architecture decoder as a static op list with a hand-derived backward.

Forward (per layer): RMSNorm -> QKV GEMM -> [per-head q/k RMSNorm] -> RoPE -> causal GQA
attention -> out-proj GEMM -> residual*depth_scale fused with the FFN RMSNorm -> FC1 GEMM ->
SwiGLU -> FC2 GEMM -> residual*depth_scale fused with the next layer's attention RMSNorm;
then final RMSNorm -> LM-head GEMM scaled by 1/width_mult -> fused cross-entropy
(workload/src/training_engine_tensor/train_loop.py:504-718).  The backward is the reverse
walk with closed-form gradients and fp32 weight-gradient accumulation into ``main_grad``
(train_loop.py:778-1110); no autograd is involved.  The optional Eagle/MTP branch follows
ref/reference/model_pure_mup_mtp.py:287-322, 393-433.  muP: embedding * mup_emb_scale,
residual branches * mup_depth_scale/sqrt(L), logits / width_mult.

One ``ModelChunk`` is a pipeline model chunk (a run of layers, optionally with the embedding
and/or the head).  Tensor / sequence parallelism enters only through ``TPComm`` and the local
geometry, so the same op list serves TP = 1 and TP > 1.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..config.schema import ModelConfig
from ..parallel.tp import TPComm
from . import params as P
from .store import ChunkSpec, ParamStore


@dataclass
class LayerCache:
    x: torch.Tensor = None  # residual stream entering the layer
    rstd1: torch.Tensor = None
    n1f: torch.Tensor = None  # normed input of the QKV GEMM (gathered under SP)
    qkv_pre: torch.Tensor = None  # only with qk_norm
    qk_rstd: torch.Tensor = None
    qkv: torch.Tensor = None  # after RoPE
    att: torch.Tensor = None
    lse: torch.Tensor = None
    h: torch.Tensor = None  # residual stream after attention
    rstd2: torch.Tensor = None
    n2f: torch.Tensor = None
    gu: torch.Tensor = None
    inter: torch.Tensor = None
    m: torch.Tensor = None  # FC2 output, pending residual
    dropped: bool = False  # whole-layer recompute: only ``x`` was kept, the rest is rebuilt in the backward pass


@dataclass
class ChunkCache:
    layers: list = field(default_factory=list)
    ids: torch.Tensor = None
    x_last: torch.Tensor = None  # input of the final norm
    rstd_f: torch.Tensor = None
    nf: torch.Tensor = None  # final-norm output (sharded rows under SP)
    nff: torch.Tensor = None
    dlogits: torch.Tensor = None
    mtp: dict = None
    slot: int = 0  # which in-flight micro-batch of this chunk the cache belongs to (names the gather buffers it holds)


class ModelChunk:
    def __init__(self, cfg: ModelConfig, store: ParamStore, spec: ChunkSpec, ops, tp: TPComm,
                 rope_table: torch.Tensor, capture=None):
        self.cfg, self.store, self.spec, self.ops, self.tp = cfg, store, spec, ops, tp
        self.geo = P.tp_geometry(cfg, tp.size, tp.rank)
        self.rope = rope_table
        self.ds = cfg.depth_scale(0)
        self.ds_mtp = cfg.depth_scale(cfg.mtp_num_layers)
        self.capture = capture  # optional hook: capture(kind, fqn, tensor)
        # debug input checks (train.debug_checks / FORGE_DEBUG_CHECKS=1): token ids and labels must lie in the GLOBAL vocabulary
        # range; the kernels themselves only skip ids outside the LOCAL range, which is legitimate under vocabulary parallelism
        self.debug_checks = False
        self.recompute = False
        self.recompute_num_layers = 0  # last n layers of the chunk keep only their input (-1: all)
        self.on_grads_final = None  # callable(prefix): every parameter under `prefix` has its final gradient of the step
        self._free_slots: list = []   # in-flight micro-batch slots released by finished backward passes
        self._n_slots = 0
        # CUDA-graph replay of the layer loops (forward and backward, one pair per in-flight slot); see enable_graphs()
        self.graph_pool = None
        self._graphs: dict = {}
        self.graph_replays = 0

    # ------------------------------------------------------------------
    def _cap(self, kind, fqn, t):
        if self.capture is not None:
            self.capture(kind, fqn, t)

    def _embed(self, ids):
        ops, geo, tp = self.ops, self.geo, self.tp
        w = self.store.p("tok_embeddings.weight")
        if self.debug_checks:
            ops.check_ids(ids, 0, self.cfg.padded_vocab_size)
        e = ops.embedding_fwd(ids, w, self.cfg.emb_scale, geo.vocab_start, tp.size > 1)
        if tp.size > 1:
            e = tp.row_output_fwd(e)
        return e

    def _embed_bwd(self, dx, ids):
        tp = self.tp
        if tp.size > 1:
            dx = tp.row_output_bwd(dx)
        self.ops.embedding_bwd(dx, ids, self.store.g("tok_embeddings.weight"), self.cfg.emb_scale,
                               self.geo.vocab_start)

    # ------------------------------------------------------------------
    def _layer_fwd(self, prefix, x, pending, ds, seq_len, slot=0):
        """``pending`` is the previous FC2 output still to be added (None at a chunk start).  ``slot`` numbers the
        in-flight micro-batch: with the one-kernel TP paths the gathered inputs of QKV / FC1 stay in per-(layer, slot)
        buffers until the backward pass has used them, and the norms write their rows straight into those buffers."""
        ops, st, tp, geo, cfg = self.ops, self.store, self.tp, self.geo, self.cfg
        c = LayerCache()
        w_an = st.p(prefix + "attention_norm.weight")
        k1, k2 = (id(self), prefix, 1, slot), (id(self), prefix, 2, slot)
        out1 = tp.col_slot(k1, x.shape[0], x.shape[1], x.dtype)
        kw1 = {} if out1 is None else {"y_out": out1}
        if pending is None:
            n1, c.rstd1 = ops.rmsnorm_fwd(x, w_an, cfg.norm_epsilon, **kw1)
        else:
            x, n1, c.rstd1 = ops.residual_rmsnorm_fwd(x, pending, ds, w_an, cfg.norm_epsilon, **kw1)
        c.x = x
        self._cap("fwd", prefix + "attention_norm", n1)
        qkv, c.n1f = tp.col_linear_fwd(ops, n1, st.p(prefix + "wqkv.weight"), key=k1)
        self._cap("fwd", prefix + "wqkv", qkv)
        if cfg.qk_norm:
            c.qkv_pre = qkv
            qkv, c.qk_rstd = ops.qk_norm_fwd(qkv, st.p(prefix + "q_norm.weight"), st.p(prefix + "k_norm.weight"),
                                             cfg.norm_epsilon, geo.n_kv_local, geo.g_local, geo.head_dim)
        ops.rope_fwd_(qkv, self.rope, seq_len, geo.n_kv_local, geo.g_local, geo.head_dim)
        c.qkv = qkv
        c.att, c.lse = ops.attention_fwd(qkv, seq_len, geo.n_kv_local, geo.g_local, geo.head_dim)
        a = tp.row_linear_fwd(ops, c.att, st.p(prefix + "wo.weight"))
        self._cap("fwd", prefix + "wo", a)
        out2 = tp.col_slot(k2, x.shape[0], x.shape[1], x.dtype)
        kw2 = {} if out2 is None else {"y_out": out2}
        c.h, n2, c.rstd2 = ops.residual_rmsnorm_fwd(x, a, ds, st.p(prefix + "ffn_norm.weight"), cfg.norm_epsilon, **kw2)
        self._cap("fwd", prefix + "ffn_norm", n2)
        c.gu, c.n2f = tp.col_linear_fwd(ops, n2, st.p(prefix + "wfc1.weight"), key=k2)
        self._cap("fwd", prefix + "wfc1", c.gu)
        c.inter = ops.swiglu_fwd(c.gu)
        c.m = tp.row_linear_fwd(ops, c.inter, st.p(prefix + "w2.weight"))
        self._cap("fwd", prefix + "w2", c.m)
        if self.recompute:
            c.inter = None
        return c

    def _layer_bwd(self, prefix, c: LayerCache, g_next, ds, seq_len):
        """``g_next`` = dL/d(h + m*ds).  Returns dL/dx (without the previous layer's pending scale)."""
        ops, st, tp, geo, cfg = self.ops, self.store, self.tp, self.geo, self.cfg
        self._cap("bwd", prefix + "w2", g_next)
        inter = c.inter if c.inter is not None else ops.swiglu_fwd(c.gu)
        d_inter, dm = tp.row_linear_dgrad(ops, g_next, st.p(prefix + "w2.weight"), ds)
        ops.linear_wgrad(dm, inter, st.g(prefix + "w2.weight"), ds)
        d_gu = ops.swiglu_bwd(d_inter, c.gu)
        ops.linear_wgrad(d_gu, c.n2f, st.g(prefix + "wfc1.weight"))
        d_n2 = tp.col_linear_dgrad(ops, d_gu, st.p(prefix + "wfc1.weight"))
        g_h = ops.rmsnorm_bwd(d_n2, c.h, st.p(prefix + "ffn_norm.weight"), c.rstd2,
                              st.g(prefix + "ffn_norm.weight"), g_next)
        self._cap("bwd", prefix + "wo", g_h)
        d_att, da = tp.row_linear_dgrad(ops, g_h, st.p(prefix + "wo.weight"), ds)
        ops.linear_wgrad(da, c.att, st.g(prefix + "wo.weight"), ds)
        d_qkv = ops.attention_rope_bwd(d_att, c.qkv, c.att, c.lse, self.rope, seq_len, geo.n_kv_local, geo.g_local,
                                       geo.head_dim)
        if cfg.qk_norm:
            d_qkv = ops.qk_norm_bwd(d_qkv, c.qkv_pre, c.qk_rstd, st.p(prefix + "q_norm.weight"),
                                    st.p(prefix + "k_norm.weight"), st.g(prefix + "q_norm.weight"),
                                    st.g(prefix + "k_norm.weight"), geo.n_kv_local, geo.g_local, geo.head_dim)
        self._cap("bwd", prefix + "wqkv", d_qkv)
        ops.linear_wgrad(d_qkv, c.n1f, st.g(prefix + "wqkv.weight"))
        d_n1 = tp.col_linear_dgrad(ops, d_qkv, st.p(prefix + "wqkv.weight"))
        g_x = ops.rmsnorm_bwd(d_n1, c.x, st.p(prefix + "attention_norm.weight"), c.rstd1,
                              st.g(prefix + "attention_norm.weight"), g_h)
        return g_x

    # ------------------------------------------------------------------
    def _head_fwd(self, x, pending, ds, labels, mask, grad_scale, norm_name, cache_out: dict):
        """Final norm -> LM head (alpha = 1/width_mult) -> fused CE.  Returns per-token NLL."""
        ops, st, tp, geo, cfg = self.ops, self.store, self.tp, self.geo, self.cfg
        w = st.p(norm_name)
        if pending is None:
            nf, rstd = ops.rmsnorm_fwd(x, w, cfg.norm_epsilon)
        else:
            x, nf, rstd = ops.residual_rmsnorm_fwd(x, pending, ds, w, cfg.norm_epsilon)
        nff = tp.col_input_fwd(nf)
        alpha = 1.0 / cfg.width_mult
        logits = ops.linear_fwd(nff, st.p(st.head_weight_name()), alpha)
        self._cap("fwd", "output", logits)
        if self.debug_checks:
            ops.check_ids(labels, 0, cfg.padded_vocab_size)
        nll = ops.cross_entropy_fwd_bwd(logits, labels, mask, grad_scale, geo.vocab_start,
                                        tp.group if tp.size > 1 else None)
        cache_out.update(x_last=x, rstd_f=rstd, nf=nf, nff=nff, dlogits=logits)
        return nll

    def _head_bwd(self, c: dict, norm_name, extra_dnf=None):
        ops, st, tp, cfg = self.ops, self.store, self.tp, self.cfg
        alpha = 1.0 / cfg.width_mult
        wname = st.head_weight_name()
        ops.linear_wgrad(c["dlogits"], c["nff"], st.g(wname), alpha)
        d_nf = tp.col_input_bwd(ops.linear_dgrad(c["dlogits"], st.p(wname), alpha))
        if extra_dnf is not None:
            d_nf = d_nf + extra_dnf
        return ops.rmsnorm_bwd(d_nf, c["x_last"], st.p(norm_name), c["rstd_f"], st.g(norm_name), None)

    # ------------------------------------------------------------------
    def forward(self, batch: dict, x_in: torch.Tensor | None = None):
        """Returns ``(x_out, cache)``; on a head chunk ``x_out`` is ``{"nll": ..., "mtp_nll": ...}``."""
        cfg, ops, tp = self.cfg, self.ops, self.tp
        S = batch["seq_len"]
        cache = ChunkCache()
        if self._free_slots:
            cache.slot = self._free_slots.pop()
        else:
            cache.slot = self._n_slots
            self._n_slots += 1
        if self.spec.has_embedding:
            cache.ids = batch["ids"]
            x = self._embed(batch["ids"])
            self._cap("fwd", "tok_embeddings", x)
        else:
            x = x_in
        if self.graph_pool is not None:
            x, pending = self._graphed_layers_fwd(x, cache, S)
        else:
            x, pending = self._layers_fwd(x, cache, S)
        if not self.spec.has_head:
            return x, cache
        hc: dict = {}
        labels, mask = batch["labels"], batch["mask"]
        out = {"nll": self._head_fwd(x, pending, self.ds, labels, mask, 1.0, "norm.weight", hc)}
        cache.x_last, cache.rstd_f, cache.nf, cache.nff, cache.dlogits = (
            hc["x_last"], hc["rstd_f"], hc["nf"], hc["nff"], hc["dlogits"])
        if cfg.mtp_num_layers and "mtp_ids" in batch:
            out["mtp_nll"] = self._mtp_fwd(batch, cache, S)
        return out, cache

    def _layers_fwd(self, x, cache: ChunkCache, S):
        """The chunk's layer loop.  Returns ``(x, pending)``: on a head chunk the last FC2 output is still to be added (the
        final norm fuses that add); otherwise the add is done here and ``pending`` is None."""
        pending = None
        n = len(self.spec.layers)
        n_rc = n if self.recompute_num_layers < 0 else min(max(self.recompute_num_layers, 0), n)
        for idx, li in enumerate(self.spec.layers):
            c = self._layer_fwd(f"layers.{li}.", x, pending, self.ds, S, cache.slot)
            x, pending = c.h, c.m
            if idx >= n - n_rc:
                c = LayerCache(x=c.x, dropped=True)   # the layer's input is all the backward pass needs to run it again
            cache.layers.append(c)
        if not self.spec.has_head and pending is not None:
            x, pending = self.ops.residual_add(x, pending, self.ds), None
        return x, pending

    def _layers_bwd(self, g, cache: ChunkCache, S):
        done = self.on_grads_final
        for li, c in zip(reversed(self.spec.layers), reversed(cache.layers)):
            if c.dropped:
                # c.x already contains the previous layer's residual, so the layer runs from it with nothing pending
                c = self._layer_fwd(f"layers.{li}.", c.x, None, self.ds, S, cache.slot)
            g = self._layer_bwd(f"layers.{li}.", c, g, self.ds, S)
            if done is not None:
                done(f"layers.{li}.")
        return g

    # -- CUDA-graph replay of the layer loops ------------------------------------------------------------------------
    def enable_graphs(self, pool=True) -> None:
        """From now on the layer loops of ``forward`` / ``run_backward`` are captured once per in-flight slot and replayed.
        Everything a replay touches has a fixed address: the loop's input is copied into a static tensor, the per-layer
        caches are the tensors the forward capture of the slot allocated (the backward graph of the slot reads them),
        all-gather buffers are the per-(layer, slot) symmetric buffers, and the cross-rank ordering of the fused TP kernels
        is numbered on the device.  Every graph has a memory pool of its OWN: a pipeline schedule replays the graphs in an
        order other than the capture order and keeps several slots' caches alive at once, and in a shared pool the
        temporaries of one graph may be handed to a later capture as its long-lived tensors, which the first graph's next
        replay would then overwrite.  Embedding, LM head, loss, pipeline send / recv and the library
        collectives stay outside the graphs.  Call after at least one eager step (lazy allocations, symmetric-memory
        rendezvous of the call sites) and on every rank of the model-parallel group at the same step."""
        self.graph_pool = pool

    def _capture(self, fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            out = fn()
        return g, out

    def _graphed_layers_fwd(self, x, cache: ChunkCache, S):
        ent = self._graphs.get(("F", cache.slot))
        if ent is None:
            x_in = x.clone()
            sc = ChunkCache()
            sc.slot = cache.slot
            g, (x_out, pending) = self._capture(lambda: self._layers_fwd(x_in, sc, S))
            ent = {"g": g, "x_in": x_in, "layers": sc.layers, "x_out": x_out, "pending": pending}
            self._graphs[("F", cache.slot)] = ent
        else:
            ent["x_in"].copy_(x)
        ent["g"].replay()
        self.graph_replays += 1
        cache.layers = ent["layers"]
        return ent["x_out"], ent["pending"]

    def _graphed_layers_bwd(self, g_top, cache: ChunkCache, S):
        ent = self._graphs.get(("B", cache.slot))
        if ent is None:
            g_in = g_top.clone()
            g, g_x = self._capture(lambda: self._layers_bwd(g_in, cache, S))
            ent = {"g": g, "g_in": g_in, "g_x": g_x}
            self._graphs[("B", cache.slot)] = ent
        else:
            ent["g_in"].copy_(g_top)
        ent["g"].replay()
        self.graph_replays += 1
        return ent["g_x"]

    def run_backward(self, batch: dict, cache: ChunkCache, g_out: torch.Tensor | None = None):
        """Accumulates weight gradients; returns dL/dx_in (None on an embedding chunk)."""
        S = batch["seq_len"]
        done = self.on_grads_final
        if self.spec.has_head:
            extra = self._mtp_bwd(batch, cache, S) if cache.mtp is not None else None
            g = self._head_bwd({"dlogits": cache.dlogits, "nff": cache.nff, "x_last": cache.x_last,
                                "rstd_f": cache.rstd_f}, "norm.weight", extra)
            cache.dlogits = None
            if done is not None:
                done("mtp.")
                done("norm.weight")
                if not self.cfg.tie_embeddings:   # a tied head shares the embedding's gradient, final only at the very end
                    done("output.weight")
        else:
            g = g_out
        if self.graph_pool is not None:
            g = self._graphed_layers_bwd(g, cache, S)
        else:
            g = self._layers_bwd(g, cache, S)
        self._free_slots.append(cache.slot)  # the gather buffers of this micro-batch may be reused
        if self.spec.has_embedding:
            self._cap("bwd", "tok_embeddings", g)
            self._embed_bwd(g, cache.ids)
            return None
        return g

    # ------------------------------------------------------------------
    # Eagle / MTP branch (single extra layer, shared embedding and LM head)
    # ------------------------------------------------------------------
    def _mtp_fwd(self, batch, cache: ChunkCache, S):
        cfg, ops, st, tp = self.cfg, self.ops, self.store, self.tp
        # Under tensor / sequence parallelism the branch needs nothing of its own: the embedding and the extra layer go
        # through the same TP-aware paths as the main stack, the two input norms and eagle_fc act row-wise on whatever rows
        # this rank holds (eagle_fc is a replicated weight whose row-partial gradient is summed with the other replicated
        # weights), and the shared LM head is the vocabulary-parallel one.
        m: dict = {}
        m["ids"] = batch["mtp_ids"]
        emb = self._embed(m["ids"])
        m["emb"] = emb
        a, m["rstd_a"] = ops.rmsnorm_fwd(emb, st.p("mtp.emb_input_layernorm.weight"), cfg.norm_epsilon)
        m["hn"] = cache.nf
        b, m["rstd_b"] = ops.rmsnorm_fwd(cache.nf, st.p("mtp.hidden_input_layernorm.weight"), cfg.norm_epsilon)
        m["cat"] = torch.cat([a, b], dim=-1)
        h0 = ops.linear_fwd(m["cat"], st.p("mtp.eagle_fc.weight"))
        m["layer"] = self._layer_fwd("mtp.layer.", h0, None, self.ds_mtp, S)
        hc: dict = {}
        w = cfg.mtp_loss_weight
        nll = self._head_fwd(m["layer"].h, m["layer"].m, self.ds_mtp, batch["mtp_labels"], batch["mtp_mask"],
                             w, "mtp.final_layernorm.weight", hc)
        m["head"] = hc
        cache.mtp = m
        return nll

    def _mtp_bwd(self, batch, cache: ChunkCache, S):
        """Returns the MTP branch's gradient w.r.t. the main final-norm output."""
        cfg, ops, st = self.cfg, self.ops, self.store
        m = cache.mtp
        g = self._head_bwd(m["head"], "mtp.final_layernorm.weight")
        g_h0 = self._layer_bwd("mtp.layer.", m["layer"], g, self.ds_mtp, S)
        ops.linear_wgrad(g_h0, m["cat"], st.g("mtp.eagle_fc.weight"))
        d_cat = ops.linear_dgrad(g_h0, st.p("mtp.eagle_fc.weight"))
        H = cfg.hidden_size
        d_a, d_b = d_cat[:, :H].contiguous(), d_cat[:, H:].contiguous()
        d_emb = ops.rmsnorm_bwd(d_a, m["emb"], st.p("mtp.emb_input_layernorm.weight"), m["rstd_a"],
                                st.g("mtp.emb_input_layernorm.weight"), None)
        self._embed_bwd(d_emb, m["ids"])
        d_nf = ops.rmsnorm_bwd(d_b, m["hn"], st.p("mtp.hidden_input_layernorm.weight"), m["rstd_b"],
                               st.g("mtp.hidden_input_layernorm.weight"), None)
        cache.mtp = None
        return d_nf
