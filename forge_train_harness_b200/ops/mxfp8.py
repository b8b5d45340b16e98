"""MXFP8 linear layers: e4m3 payloads with one e8m0 scale per 32 elements of the contraction dimension.

The reference has no fp8 path (all of its matmuls are bf16 ``torch.matmul``, workload/src/training_engine_tensor/forward.py:83,195,198,300
and backward.py:79,90,389,394); this is the block-scaled option of the 8B tensor-parallel target, built on
``csrc/mxfp8_sm100.cu``.  Three things live here:

* a plain PyTorch statement of the format (``quantize_ref`` / ``dequantize_ref``) that runs on CPU and is the oracle of
  the CUDA quantisation kernels and of the block-scaled GEMM (fp32 matmul of the dequantised operands);
* thin wrappers over the extension (``quantize`` / ``gemm``);
* ``Mxfp8Linear``: the three products of a linear layer.  Scale blocks always run along the contraction dimension, so
  the forward uses row-quantised ``x`` and ``w``, the data gradient row-quantised ``dy`` and column-quantised ``w``, the
  weight gradient column-quantised ``dy`` and ``x``.  Weight copies are cached per parameter in fixed buffers and
  re-quantised in place after every optimizer step;
* ``Mxfp8Ops``: an op table that routes the three linear products through ``Mxfp8Linear`` (``parallel.fp8 = "mxfp8"``).

Scale storage: for every 128 rows x 4 scale blocks one 512-byte chunk, byte ``(r % 32) * 16 + (r // 32 % 4) * 4 + kb % 4``,
chunks ordered ``[ceil(rows / 128)][ceil(K / 128)]`` — the layout one ``tcgen05.cp.32x128b.warpx4`` moves into tensor memory.
"""
from __future__ import annotations

import torch

E4M3_MAX = 448.0


def sf_bytes(rows: int, k: int) -> int:
    return ((rows + 127) // 128) * ((k // 32 + 3) // 4) * 512


def _chunk_index(rows: int, kblocks: int, device):
    r = torch.arange(rows, device=device)[:, None]
    kb = torch.arange(kblocks, device=device)[None, :]
    k_chunks = (kblocks + 3) // 4
    return ((r // 128) * k_chunks + kb // 4) * 512 + (r % 32) * 16 + (r // 32 % 4) * 4 + kb % 4


def quantize_ref(x: torch.Tensor, colwise: bool = False):
    """``(payload uint8 [rows, K], scale chunks uint8)`` of ``x`` (``x.T`` if ``colwise``); blocks of 32 along ``K``."""
    m = (x.t() if colwise else x).float().contiguous()
    rows, k = m.shape
    assert k % 32 == 0
    blk = m.view(rows, k // 32, 32)
    amax = blk.abs().amax(dim=2)
    v = (amax * (1.0 / E4M3_MAX)).to(torch.float32)
    bits = v.view(torch.int32)
    e = (bits >> 23) & 0xFF
    e = torch.where((bits & 0x7FFFFF) != 0, e + 1, e).clamp(max=254)
    inv = torch.where(e == 254, torch.tensor(0x00400000, dtype=torch.int32, device=x.device),
                      ((254 - e) << 23).to(torch.int32)).view(torch.float32)
    q = (blk * inv[:, :, None]).to(torch.float8_e4m3fn).view(torch.uint8).view(rows, k)
    sf = torch.zeros(sf_bytes(rows, k), dtype=torch.uint8, device=x.device)
    sf[_chunk_index(rows, k // 32, x.device).reshape(-1)] = e.to(torch.uint8).reshape(-1)
    return q, sf


def dequantize_ref(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    rows, k = q.shape
    e = sf[_chunk_index(rows, k // 32, q.device).reshape(-1)].view(rows, k // 32).to(torch.int32)
    scale = torch.where(e == 0, torch.tensor(0x00400000, dtype=torch.int32, device=q.device), e << 23).view(torch.float32)
    return (q.view(torch.float8_e4m3fn).float().view(rows, k // 32, 32) * scale[:, :, None]).view(rows, k)


def _ext():
    from .cuda_ops import _C
    return _C


def quantize(x: torch.Tensor, colwise: bool = False):
    if x.is_cuda:
        return tuple(_ext().mxfp8_quant(x, bool(colwise)))
    return quantize_ref(x, colwise)


def gemm(a, sfa, b, sfb, out=None, alpha: float = 1.0, epi: int = 0):
    """``alpha * A @ B.T`` on quantised operands; ``epi`` 0 = bf16, 1 = fp32 ``out +=``, 2 = fp32 store."""
    if a.is_cuda:
        return _ext().gemm_mxfp8(a, sfa, b, sfb, out, float(alpha), int(epi))
    r = alpha * (dequantize_ref(a, sfa) @ dequantize_ref(b, sfb).t())
    if epi == 1:
        out += r
        return out
    r = r.to(torch.bfloat16 if epi == 0 else torch.float32)
    if out is not None:
        out.copy_(r)
        return out
    return r


class Mxfp8Linear:
    """Forward / dgrad / wgrad of ``y = alpha * x @ w.T`` in MXFP8 with cached weight copies.

    A weight is quantised on first use and the copies live in fixed buffers (a captured CUDA graph may hold their
    addresses); ``refresh()`` re-quantises every cached weight into the same buffers and is called by the engine after
    each optimizer step and after a checkpoint load.
    """

    def __init__(self):
        self._w = {}     # (data_ptr, shape) -> [weight view, row-quantised (q, sf), col-quantised (q, sf) or None]

    def _weight(self, w, need_col):
        key = (w.data_ptr(), tuple(w.shape))
        ent = self._w.get(key)
        if ent is None:
            ent = [w, quantize(w, False), None]
            self._w[key] = ent
        if need_col and ent[2] is None:
            ent[2] = quantize(w, True)
        return ent

    def refresh(self):
        for ent in self._w.values():
            w = ent[0]
            for slot, colwise in ((1, False), (2, True)):
                if ent[slot] is not None:
                    q, sf = quantize(w, colwise)
                    ent[slot][0].copy_(q)
                    ent[slot][1].copy_(sf)

    @staticmethod
    def supported(*dims) -> bool:
        return all(d % 32 == 0 for d in dims)

    def fwd(self, x, w, alpha=1.0):
        xq, xs = quantize(x, False)
        wq, ws = self._weight(w, False)[1]
        return gemm(xq, xs, wq, ws, None, alpha, 0)

    def dgrad(self, dy, w, alpha=1.0):
        dq, dsf = quantize(dy, False)
        wq, ws = self._weight(w, True)[2]          # [K, N]: contraction over N
        return gemm(dq, dsf, wq, ws, None, alpha, 0)

    def wgrad(self, dy, x, main_grad, alpha=1.0):
        dq, dsf = quantize(dy, True)               # [N, M]: contraction over the tokens
        xq, xs = quantize(x, True)                 # [K, M]
        return gemm(dq, dsf, xq, xs, main_grad, alpha, 1)


class Mxfp8Ops:
    """An op table whose three linear products run in MXFP8 wherever every dimension is a multiple of 32; everything else
    (and the ragged vocabulary head / embedding products) stays on the wrapped table."""

    def __init__(self, base):
        from . import OP_NAMES
        for n in OP_NAMES:
            if n not in ("linear_fwd", "linear_dgrad", "linear_wgrad"):
                setattr(self, n, getattr(base, n))
        self.base = base
        self.lin = Mxfp8Linear()
        self.name = getattr(base, "name", "ops") + "+mxfp8"
        self.versions = dict(getattr(base, "versions", {}), linear_fwd="mxfp8", linear_dgrad="mxfp8", linear_wgrad="mxfp8")
        self.mx_calls = 0

    @staticmethod
    def _plain(t):
        return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.dtype == torch.bfloat16

    def linear_fwd(self, x, w, alpha=1.0):
        if self._plain(x) and self._plain(w) and Mxfp8Linear.supported(x.shape[0], x.shape[1], w.shape[0]):
            self.mx_calls += 1
            return self.lin.fwd(x, w, alpha)
        return self.base.linear_fwd(x, w, alpha)

    def linear_dgrad(self, dy, w, alpha=1.0):
        if self._plain(dy) and self._plain(w) and Mxfp8Linear.supported(dy.shape[0], dy.shape[1], w.shape[1]):
            self.mx_calls += 1
            return self.lin.dgrad(dy, w, alpha)
        return self.base.linear_dgrad(dy, w, alpha)

    def linear_wgrad(self, dy, x, main_grad, alpha=1.0):
        if self._plain(dy) and self._plain(x) and main_grad.dtype == torch.float32 and \
                Mxfp8Linear.supported(dy.shape[0], dy.shape[1], x.shape[1]):
            self.mx_calls += 1
            return self.lin.wgrad(dy, x, main_grad, alpha)
        return self.base.linear_wgrad(dy, x, main_grad, alpha)

    def after_optimizer_step(self):
        self.lin.refresh()
