"""Process-group layout helpers: one call brings up zbal and the "zbal" torch.distributed backend, and a
mesh cuts the world into tensor- / expert- / data- / pipeline-parallel groups.

    ctx = parallel.init(heap_bytes=8 << 30)                  # reads RANK / WORLD_SIZE / LOCAL_RANK / MASTER_*
    mesh = parallel.Mesh(tp=2, pp=2)                         # dp = world / (tp * pp); rank = (pp_i * dp + dp_i) * tp + tp_i
    dist.all_reduce(t, group=mesh.tp_group)                  # zbal kernels over NVLink

Every group a mesh creates is evenly spaced in rank order (tp: step 1, dp: step tp, pp: step tp * dp), which
is what the zbal communicators support natively; irregular groups still work through the NCCL fallback.
The reference ships no mesh helper: its backend is used through plain ``dist.new_group``
(app/zbal/doc/user_guide/get_started.md:48-240); this module packages that recipe.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class Context:
    rank: int
    world: int
    local_rank: int
    device: torch.device


def init(heap_bytes: int = 4 << 30, backend: str = "zbal", comm_group_cap: int = 32) -> Context:
    """Bootstraps zbal (symmetric heap of ``heap_bytes`` per rank) and the default process group."""
    from .. import zbal
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank % max(1, torch.cuda.device_count()))))
    torch.cuda.set_device(local)
    if not zbal.is_initialized():
        zbal.zbal_init(world, local, rank, heap_bytes, start_config_server=True, comm_group_cap=comm_group_cap)
    if not dist.is_initialized():
        dist.init_process_group(backend, rank=rank, world_size=world)
    return Context(rank, world, local, torch.device("cuda", local))


def shutdown() -> None:
    from .. import zbal
    if dist.is_initialized():
        torch.cuda.synchronize()
        dist.destroy_process_group()
    zbal.zbal_uninit()


class Mesh:
    def __init__(self, tp: int = 1, pp: int = 1, ep: Optional[int] = None, world: Optional[int] = None, rank: Optional[int] = None):
        self.world = dist.get_world_size() if world is None else world
        self.rank = dist.get_rank() if rank is None else rank
        if self.world % (tp * pp) != 0:
            raise ValueError(f"world {self.world} does not divide by tp * pp = {tp * pp}")
        self.tp, self.pp, self.dp = tp, pp, self.world // (tp * pp)
        self.ep = ep or self.dp * tp                       # experts are spread over a pipeline stage's ranks by default
        if (self.dp * tp) % self.ep != 0:
            raise ValueError(f"ep {self.ep} does not divide the {self.dp * tp} ranks of a pipeline stage")
        self.tp_rank = self.rank % tp
        self.dp_rank = (self.rank // tp) % self.dp
        self.pp_rank = self.rank // (tp * self.dp)
        self.tp_group = self.dp_group = self.pp_group = self.ep_group = None
        self._build()

    @staticmethod
    def ranks_of(kind: str, rank: int, tp: int, dp: int, pp: int, ep: int) -> List[int]:
        """Members of the group of ``kind`` that ``rank`` belongs to (pure function; also used by the tests)."""
        t, d, p = rank % tp, (rank // tp) % dp, rank // (tp * dp)
        if kind == "tp":
            return [(p * dp + d) * tp + i for i in range(tp)]
        if kind == "dp":
            return [(p * dp + i) * tp + t for i in range(dp)]
        if kind == "pp":
            return [(i * dp + d) * tp + t for i in range(pp)]
        if kind == "ep":
            stage = p * dp * tp
            within = rank - stage
            first = stage + within // ep * ep
            return list(range(first, first + ep))
        raise ValueError(kind)

    def _build(self) -> None:
        # every rank must create every group, in the same order (torch.distributed's rule)
        for kind in ("tp", "dp", "pp", "ep"):
            seen = set()
            for r in range(self.world):
                members = tuple(self.ranks_of(kind, r, self.tp, self.dp, self.pp, self.ep))
                if members in seen:
                    continue
                seen.add(members)
                g = dist.new_group(list(members)) if len(members) > 1 and dist.is_initialized() else None
                if self.rank in members:
                    setattr(self, f"{kind}_group", g)
                    setattr(self, f"{kind}_ranks", list(members))

    @property
    def prev_stage(self) -> Optional[int]:
        return None if self.pp_rank == 0 else self.rank - self.tp * self.dp

    @property
    def next_stage(self) -> Optional[int]:
        return None if self.pp_rank == self.pp - 1 else self.rank + self.tp * self.dp
