"""ParamStore: the local parameters of one rank as views into flat buffers.

One flat compute-dtype parameter buffer and one flat fp32 gradient buffer hold every
local parameter (train_loop.py:1585-1625 keeps the same flat-buffer discipline so the
gradient collective and the norm run on one tensor).  The buffer order is the REVERSE of
the forward order, cut into buckets of ``bucket_elems`` elements, so that buckets fill
front-to-back while the manual backward walks the layers in reverse — the layout the
Megatron distributed optimizer uses (reversed ``named_parameters``, 40 M-element buckets).
Every bucket is padded to a multiple of ``dp * ALIGN`` elements so each data-parallel rank
owns an equal, 16-byte-aligned slice of every bucket.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config.schema import ModelConfig
from . import params as P

ALIGN = 256  # elements; keeps every param start 512-byte aligned in bf16 (TMA wants 16 B)


@dataclass(frozen=True)
class ChunkSpec:
    """One pipeline model chunk: a contiguous run of layers, optionally with embedding / head."""
    layers: tuple[int, ...]
    has_embedding: bool
    has_head: bool


def pipeline_chunks(cfg: ModelConfig, pp: int, vpp: int, pp_rank: int, layer_split=()) -> list[ChunkSpec]:
    """Layer assignment for interleaved pipelining: model chunk ``v*pp + p`` lives on stage ``p``.  ``layer_split`` gives
    the number of layers of every chunk in chunk order (empty: an even split)."""
    n_chunks = pp * vpp
    if layer_split:
        counts = [int(x) for x in layer_split]
        if len(counts) != n_chunks or sum(counts) != cfg.num_layers or min(counts) < 1:
            raise ValueError(f"pipeline_layer_split needs {n_chunks} positive entries that sum to {cfg.num_layers}")
    else:
        if cfg.num_layers % n_chunks:
            raise ValueError("num_layers must be divisible by pipeline stages * virtual stages")
        counts = [cfg.num_layers // n_chunks] * n_chunks
    starts = [sum(counts[:c]) for c in range(n_chunks)]
    out = []
    for v in range(vpp):
        c = v * pp + pp_rank
        out.append(ChunkSpec(tuple(range(starts[c], starts[c] + counts[c])), c == 0, c == n_chunks - 1))
    return out


@dataclass
class Bucket:
    start: int
    end: int  # padded end
    names: list[str]


class ParamStore:
    def __init__(self, cfg: ModelConfig, chunks: list[ChunkSpec], *, tp: int = 1, tp_rank: int = 0,
                 dp: int = 1, dtype=torch.bfloat16, device="cpu", bucket_elems: int = 40_000_000,
                 pp: int = 1):
        self.cfg, self.tp, self.tp_rank, self.dp, self.dtype = cfg, tp, tp_rank, dp, dtype
        self.device = torch.device(device)
        self.chunks = chunks
        layers = {li for c in chunks for li in c.layers}
        has_emb = any(c.has_embedding for c in chunks)
        has_head = any(c.has_head for c in chunks)
        # The last stage needs the embedding table too when the LM head is tied to it or when the MTP branch embeds its own
        # input tokens; it then holds a second copy whose gradient is summed with the first stage's.
        shares_embedding = cfg.tie_embeddings or bool(cfg.mtp_num_layers)
        self.specs: list[P.ParamSpec] = []
        for s in P.full_param_specs(cfg):
            if s.layer == -1:
                keep = has_emb or (shares_embedding and has_head)
            elif s.layer == 10 ** 6:
                keep = has_head
            else:
                keep = s.layer in layers
            if keep:
                self.specs.append(s)
        # A tied LM head on a last stage that does not also hold the embedding is a second copy
        # of tok_embeddings.weight; its gradient is summed with the first stage's (embed group).
        self.tied_copy = shares_embedding and has_head and not has_emb
        self.spec_by_name = {s.name: s for s in self.specs}
        self.shapes = {s.name: P.local_shape(s, cfg, tp, tp_rank) for s in self.specs}

        # ---- flat layout: reversed forward order, bucketed -------------------
        order = list(reversed(self.specs))
        self.offsets: dict[str, tuple[int, int]] = {}
        self.buckets: list[Bucket] = []
        pad_to = dp * ALIGN
        cur, bstart, names = 0, 0, []
        for s in order:
            n = 1
            for d in self.shapes[s.name]:
                n *= d
            self.offsets[s.name] = (cur, n)
            names.append(s.name)
            cur += (n + ALIGN - 1) // ALIGN * ALIGN
            if cur - bstart >= bucket_elems:
                cur = bstart + ((cur - bstart) + pad_to - 1) // pad_to * pad_to
                self.buckets.append(Bucket(bstart, cur, names))
                bstart, names = cur, []
        if names:
            cur = bstart + ((cur - bstart) + pad_to - 1) // pad_to * pad_to
            self.buckets.append(Bucket(bstart, cur, names))
        self.numel = cur
        self.flat_param = torch.zeros(self.numel, dtype=dtype, device=self.device)
        self.flat_grad = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        self.params: dict[str, torch.Tensor] = {}
        self.grads: dict[str, torch.Tensor] = {}
        for s in self.specs:
            o, n = self.offsets[s.name]
            self.params[s.name] = self.flat_param[o:o + n].view(self.shapes[s.name])
            self.grads[s.name] = self.flat_grad[o:o + n].view(self.shapes[s.name])

    def rebind(self, flat_param: torch.Tensor, flat_grad: torch.Tensor) -> None:
        """Move the flat buffers (e.g. into symmetric memory); every parameter / gradient view is rebuilt."""
        assert flat_param.numel() == self.numel and flat_grad.numel() == self.numel
        self.flat_param, self.flat_grad = flat_param, flat_grad
        for s in self.specs:
            o, n = self.offsets[s.name]
            self.params[s.name] = self.flat_param[o:o + n].view(self.shapes[s.name])
            self.grads[s.name] = self.flat_grad[o:o + n].view(self.shapes[s.name])

    # -- access --------------------------------------------------------------
    def p(self, name: str) -> torch.Tensor:
        return self.params[name]

    def g(self, name: str) -> torch.Tensor:
        return self.grads[name]

    def head_weight_name(self) -> str:
        return "tok_embeddings.weight" if self.cfg.tie_embeddings else "output.weight"

    def zero_grad(self) -> None:
        self.flat_grad.zero_()

    # -- init / load -----------------------------------------------------------
    def init_reference(self, seed: int, init_ones: bool = True) -> None:
        """Layout-invariant init: full tensors from one generator, then slice the local shard."""
        wanted = set(self.params)
        for spec, full in P.iter_full_init(self.cfg, seed, init_ones, wanted):
            if full is None:
                continue
            self.load_full(spec.name, full)

    def init_device(self, seed: int, init_ones: bool = True) -> None:
        """Every shard drawn on its own device.  The stream of a parameter is keyed by its NAME (not by its position in this
        rank's list): two pipeline stages then never draw the same numbers for different layers, while the two copies of a
        tied embedding (first and last stage), DP replicas and TP-replicated tensors still come out identical."""
        import zlib
        for s in self.specs:
            tmp = torch.empty(self.shapes[s.name], dtype=torch.float32, device=self.device)
            P.device_init_(tmp, s, self.cfg, seed + 7919 * self.tp_rank * (s.kind != "replicated"),
                           zlib.crc32(s.name.encode()) & 0x7FFFFFFF, init_ones)
            self.params[s.name].copy_(tmp)

    def load_full(self, name: str, full: torch.Tensor) -> None:
        """Copy the local shard of a FULL logical tensor into this rank's parameter."""
        spec = self.spec_by_name[name]
        dim, idx = P.shard_rows(spec, self.cfg, self.tp, self.tp_rank)
        t = full if idx is None else full.index_select(dim, idx)
        self.params[name].copy_(t.to(self.device))

    def load_canonical_state(self, state: dict[str, torch.Tensor]) -> None:
        """Load ``{reference FQN: full fp32 tensor}`` (evals/harness_hook/_canonical_state.py:80-117)."""
        for name in self.params:
            if name not in state:
                raise KeyError(f"canonical state lacks {name}")
            self.load_full(name, state[name].float())

    def named_full_shapes(self):
        return [(s.name, s.full_shape) for s in self.specs]
