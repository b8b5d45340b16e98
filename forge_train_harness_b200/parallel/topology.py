"""Process topology: rank <-> (pp, dp, tp) coordinates and the process groups built on them.

Rank order is TP innermost, DP next, PP outermost — ``global = pp*(dp*tp) + dp*tp_size + tp`` —
which reduces to the reference's ``global_rank = dp_rank * tp + tp_rank`` when PP = 1
(ref/reference/train_minicpm4_8b_tp.py:17-21, evals/harness_dptp/__init__.py:98-141: TP
groups are contiguous blocks, DP groups are strided sets).  Every rank creates every group
in the same order, as ``torch.distributed.new_group`` requires.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist


@dataclass
class Topology:
    world_size: int = 1
    rank: int = 0
    tp: int = 1
    pp: int = 1
    dp: int = 1
    tp_rank: int = 0
    dp_rank: int = 0
    pp_rank: int = 0
    tp_group: object = None
    dp_group: object = None
    pp_group: object = None
    embed_group: object = None  # first + last pipeline stage (tied embedding grads)
    kv_group: object = None  # TP ranks sharing one replicated KV head
    tp_ranks: list[int] = field(default_factory=lambda: [0])
    dp_ranks: list[int] = field(default_factory=lambda: [0])
    pp_ranks: list[int] = field(default_factory=lambda: [0])

    def coords(self, rank: int) -> tuple[int, int, int]:
        tp_r = rank % self.tp
        dp_r = (rank // self.tp) % self.dp
        pp_r = rank // (self.tp * self.dp)
        return pp_r, dp_r, tp_r

    def rank_of(self, pp_r: int, dp_r: int, tp_r: int) -> int:
        return pp_r * (self.dp * self.tp) + dp_r * self.tp + tp_r

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.pp - 1

    @property
    def prev_stage_rank(self) -> int:
        return self.rank_of((self.pp_rank - 1) % self.pp, self.dp_rank, self.tp_rank)

    @property
    def next_stage_rank(self) -> int:
        return self.rank_of((self.pp_rank + 1) % self.pp, self.dp_rank, self.tp_rank)


def ranks_per_node() -> int:
    """Processes per node as the launcher states it (``LOCAL_WORLD_SIZE``; one node when it is not set)."""
    v = os.environ.get("LOCAL_WORLD_SIZE")
    if v:
        return max(1, int(v))
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size()
    return max(1, int(os.environ.get("WORLD_SIZE") or "1"))


def spans_nodes(ranks) -> bool:
    """True when ``ranks`` (global ranks of one process group) live on more than one node.  The peer-memory kernels (fused DP
    reduce-scatter / parameter push, all-gather->GEMM, GEMM->reduce-scatter) read and write other GPUs' memory over NVLink and
    so serve groups inside one NVSwitch domain; a group that crosses nodes keeps the library collectives.  Every rank
    derives the same answer from the launcher's environment, so the choice of path cannot differ between ranks."""
    n = ranks_per_node()
    return len({int(r) // n for r in ranks}) > 1


def build_topology(tp: int = 1, pp: int = 1, kv_replicas: int = 1) -> Topology:
    """Create all groups.  Works without an initialised process group (world size 1)."""
    if not (dist.is_available() and dist.is_initialized()):
        if tp * pp != 1:
            raise RuntimeError("TP/PP > 1 needs torch.distributed to be initialised")
        return Topology()
    world, rank = dist.get_world_size(), dist.get_rank()
    if world % (tp * pp):
        raise ValueError(f"world size {world} is not divisible by TP*PP = {tp * pp}")
    dp = world // (tp * pp)
    t = Topology(world_size=world, rank=rank, tp=tp, pp=pp, dp=dp)
    t.pp_rank, t.dp_rank, t.tp_rank = t.coords(rank)

    def make(rank_lists, single_ok=True):
        mine, mine_ranks = None, None
        for ranks in rank_lists:
            g = dist.new_group(ranks) if len(ranks) > 1 or not single_ok else None
            if rank in ranks:
                mine, mine_ranks = g, ranks
        return mine, mine_ranks

    t.tp_group, t.tp_ranks = make([[t.rank_of(p, d, x) for x in range(tp)] for p in range(pp) for d in range(dp)])
    t.dp_group, t.dp_ranks = make([[t.rank_of(p, d, x) for d in range(dp)] for p in range(pp) for x in range(tp)])
    t.pp_group, t.pp_ranks = make([[t.rank_of(p, d, x) for p in range(pp)] for d in range(dp) for x in range(tp)])
    if pp > 1:
        t.embed_group, _ = make([[t.rank_of(0, d, x), t.rank_of(pp - 1, d, x)] for d in range(dp) for x in range(tp)])
    if kv_replicas > 1:
        t.kv_group, _ = make([[t.rank_of(p, d, k * kv_replicas + i) for i in range(kv_replicas)]
                              for p in range(pp) for d in range(dp) for k in range(tp // kv_replicas)])
    return t


def init_distributed(backend: str | None = None, timeout_s: float = 1800.0) -> bool:
    """Initialise ``torch.distributed`` from the torchrun environment (RANK / WORLD_SIZE / MASTER_*).

    One process per GPU; NCCL on CUDA, gloo on CPU (train_loop.py:2675-2686).  Returns True if
    this call created the process group."""
    import datetime
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1 and "RANK" not in os.environ:
        return False
    if dist.is_initialized():
        return False
    use_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    kwargs = {}
    if use_cuda and backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        kwargs["device_id"] = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return True
