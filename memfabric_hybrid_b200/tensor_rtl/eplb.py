"""Expert re-placement for MoE load balancing (EPLB): moves expert weights between expert-parallel ranks when
the placement of logical experts onto physical slots changes.

A placement is a list ``placement[slot] = logical expert`` over all physical slots of one layer; rank r owns the
slots ``[r * local, (r + 1) * local)``. Redundant copies of a hot expert are allowed (a logical id may appear in
several slots). ``ExpertMigrator.plan`` pairs every slot of the new placement with a source slot of the old one
(a copy already on the destination rank first, else the copies round-robin, so that replicas of one expert do
not all pull from one rank), packs the tensors of a moving expert (w13, w2, scales, ...) into ONE flat buffer,
and describes each move as a ``PTensor`` living on ``[src_rank]`` that must end up on ``[dst_rank]``; any
executor of this package carries the plan out. ``apply`` writes the received experts into their slots.

Parity: app/tensorRTL/examples/eplb/experts_transform_manager.py:236-420 of the reference (pack, plan with one
PTensor per moving expert, execute, local moves through temporaries, unpack). The serving-engine hooks of that
example (load statistics, the planner process) are the caller's: this class starts from the two placements.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .pack import pack_tensors, unpack_tensors
from .plan import PTensor, PTensorSet


def pair_slots(old: Sequence[int], new: Sequence[int], local: int) -> List[Tuple[int, int]]:
    """[(source slot in ``old``, destination slot in ``new``)] for every slot whose expert changes.
    Deterministic, so every rank computes the same pairing."""
    if len(old) != len(new) or local <= 0 or len(old) % local:
        raise ValueError("placements must have the same length, a multiple of the experts per rank")
    holders: Dict[int, List[int]] = {}
    for slot, e in enumerate(old):
        holders.setdefault(e, []).append(slot)
    turn: Dict[int, int] = {}
    pairs = []
    for dst, e in enumerate(new):
        if old[dst] == e:
            continue                       # already in place
        if e not in holders:
            raise KeyError(f"expert {e} of the new placement is held by no slot of the old one")
        same_rank = [s for s in holders[e] if s // local == dst // local]
        if same_rank:
            src = same_rank[0]
        else:
            k = turn.get(e, 0)
            turn[e] = k + 1
            src = holders[e][k % len(holders[e])]
        pairs.append((src, dst))
    return pairs


def balanced_placement(load: Sequence[float], ep_size: int, slots_per_rank: int, previous: Optional[Sequence[int]] = None,
                       tolerance: float = 0.05) -> List[int]:
    """The planner of the EPLB flow: from the tokens each LOGICAL expert received (``load[e]``, e.g. a moving average of the
    router's counts summed over ranks) to a placement ``placement[slot] = logical expert`` over ``ep_size * slots_per_rank``
    physical slots that evens out the expert work per rank. Spare slots (slots beyond the number of logical experts) become
    extra copies of the hottest experts: a copy is added, one at a time, to the expert with the largest load per copy. The
    copies are then packed onto ranks heaviest first, each onto the rank with the least work so far that still has a free
    slot (and, when possible, no copy of the same expert yet).
    ``previous``: the placement in force. Weights that stay where they are cost nothing to migrate, so among the ranks whose
    work is within ``tolerance`` (a fraction of the mean work per rank) of the least loaded one, a rank that already holds
    the expert is preferred, and inside a rank an expert keeps its slot.
    Deterministic: every rank computes the same placement."""
    E, P = len(load), ep_size * slots_per_rank
    if E == 0 or P < E:
        raise ValueError(f"{P} physical slots cannot hold {E} logical experts")
    if previous is not None and len(previous) != P:
        raise ValueError(f"the previous placement has {len(previous)} slots, this layout {P}")
    copies = [1] * E
    for _ in range(P - E):
        e = max(range(E), key=lambda i: (load[i] / copies[i], -i))
        copies[e] += 1
    items = sorted(((load[e] / copies[e], e) for e in range(E) for _ in range(copies[e])), key=lambda t: (-t[0], t[1]))
    work = [0.0] * ep_size
    held: List[List[int]] = [[] for _ in range(ep_size)]
    # copies of each expert that a rank holds today and that the new placement has not claimed yet
    there: List[Dict[int, int]] = [{} for _ in range(ep_size)]
    if previous is not None:
        for slot, e in enumerate(previous):
            d = there[slot // slots_per_rank]
            d[e] = d.get(e, 0) + 1
    slack = tolerance * (sum(load) / ep_size)
    for w, e in items:
        free = [r for r in range(ep_size) if len(held[r]) < slots_per_rank]
        fresh = [r for r in free if e not in held[r]] or free
        least = min(work[q] for q in fresh)
        r = min(fresh, key=lambda q: (0 if (work[q] <= least + slack and there[q].get(e, 0) > 0) else 1, work[q], q))
        held[r].append(e)
        work[r] += w
        if there[r].get(e, 0) > 0:
            there[r][e] -= 1
    if previous is None:
        return [e for r in range(ep_size) for e in held[r]]
    out: List[int] = []
    for r in range(ep_size):                      # inside a rank: an expert that is here already keeps its slot
        old = list(previous[r * slots_per_rank:(r + 1) * slots_per_rank])
        row: List[Optional[int]] = [None] * slots_per_rank
        rest = []
        for e in held[r]:
            spot = next((i for i, o in enumerate(old) if o == e and row[i] is None), None)
            if spot is None:
                rest.append(e)
            else:
                row[spot] = e
        it = iter(rest)
        out.extend(e if e is not None else next(it) for e in row)
    return out


def replica_table(placement: Sequence[int], num_logical: int, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(table [num_logical, max copies] int32 of physical slots, -1 padded; counts [num_logical] int32)."""
    slots: List[List[int]] = [[] for _ in range(num_logical)]
    for slot, e in enumerate(placement):
        slots[e].append(slot)
    if any(not s for s in slots):
        raise ValueError("a logical expert has no physical slot")
    width = max(len(s) for s in slots)
    table = torch.tensor([s + [-1] * (width - len(s)) for s in slots], dtype=torch.int32, device=device)
    counts = torch.tensor([len(s) for s in slots], dtype=torch.int32, device=device)
    return table, counts


def remap_topk(topk_idx: torch.Tensor, table: torch.Tensor, counts: torch.Tensor, token_offset: int = 0) -> torch.Tensor:
    """Logical expert ids [T, K] -> physical slot ids: token t uses copy (t + token_offset) mod copies(e), so the tokens of a
    replicated expert spread evenly over its copies. Negative ids (unselected) pass through."""
    T = topk_idx.shape[0]
    valid = topk_idx >= 0
    e = topk_idx.clamp_min(0).long()
    tok = (torch.arange(T, device=topk_idx.device) + token_offset).view(T, 1)
    which = tok % counts[e].long()
    phys = table[e, which]
    return torch.where(valid, phys, topk_idx.to(phys.dtype)).to(torch.int32)


class ExpertMigrator:
    def __init__(self, rank: int, ep_size: int, experts_per_rank: int, backend: str = "nccl"):
        self.rank, self.ep_size, self.local = rank, ep_size, experts_per_rank
        self.backend = backend
        self._moves: List[Tuple[int, int]] = []
        self._remote: List[Tuple[int, PTensor, Optional[dict]]] = []   # (destination slot, tensor, pack metadata)
        self._local: List[Tuple[int, torch.Tensor, dict]] = []         # (destination slot, packed copy, metadata)
        self._set: Optional[PTensorSet] = None

    def plan(self, old: Sequence[int], new: Sequence[int], experts: Sequence[torch.Tensor]) -> List:
        """``experts``: this rank's weight tensors, each of shape [experts_per_rank, ...]. Returns the transfer list
        for an executor (empty when nothing crosses ranks)."""
        for w in experts:
            if w.shape[0] != self.local:
                raise ValueError(f"expert tensor of shape {tuple(w.shape)} does not have {self.local} local experts")
        self._moves = pair_slots(old, new, self.local)
        self._remote, self._local = [], []
        # the layout of a packed expert is the same on every rank: take it from local slot 0
        probe, meta = pack_tensors([w[0] for w in experts], torch.int8)
        numel = probe.numel()
        pts = []
        for src, dst in self._moves:
            sr, dr = src // self.local, dst // self.local
            if sr == dr:
                if sr == self.rank:    # a move inside this rank: keep a copy now, slots may be overwritten in any order
                    packed, m = pack_tensors([w[src % self.local] for w in experts], torch.int8)
                    self._local.append((dst % self.local, packed, m))
                continue
            if self.rank not in (sr, dr):
                continue
            shard = pack_tensors([w[src % self.local] for w in experts], torch.int8)[0] if self.rank == sr else None
            pt = PTensor(shard, torch.int8, 1, [sr], (numel,), 0, rank=self.rank, backend=self.backend)
            pts.append((pt, [dr]))
            self._remote.append((dst % self.local, pt, meta))
        self._set = None
        if not pts:
            return []
        self._set = PTensorSet([p for p, _ in pts])
        self._set.transfer_map([m for _, m in pts])
        return self._set.get_transfer_list()

    def apply(self, experts: Sequence[torch.Tensor]) -> int:
        """After the executor finished: writes received and locally moved experts into their slots. Returns the
        number of slots of this rank that changed."""
        changed = 0
        for slot, packed, meta in self._local:
            for w, t in zip(experts, unpack_tensors(packed, meta)):
                w[slot].copy_(t)
            changed += 1
        for slot, pt, meta in self._remote:
            got = pt.collect_tensor()
            if got is None:            # this rank was the source of the move
                continue
            for w, t in zip(experts, unpack_tensors(got, meta)):
                w[slot].copy_(t)
            changed += 1
        self._local, self._remote = [], []
        return changed

    @property
    def moves(self) -> List[Tuple[int, int]]:
        return list(self._moves)

