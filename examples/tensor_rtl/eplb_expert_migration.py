"""Expert-parallel load balancing: 4 EP ranks hold 3 physical expert slots each (8 logical experts plus 4
redundant copies of hot ones). The router's measured load changes (experts 5 and 7 got hot): ``balanced_placement``
plans which experts get the spare slots and where everything sits, ``ExpertMigrator`` moves the experts whose slot
changed with one all-to-all-v, every rank checks its slots against the new placement, and ``replica_table`` /
``remap_topk`` spread the tokens of an expert over its copies. Counterpart of the reference's examples/eplb flow
without the serving engine around it.

    python examples/tensor_rtl/eplb_expert_migration.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import _launch  # noqa: E402

OLD = [0, 1, 2,  3, 4, 5,  6, 7, 0,  1, 2, 3]      # slot -> logical expert; rank r owns slots 3r .. 3r+2
LOAD = [10, 10, 10, 10, 10, 90, 10, 60]            # tokens per logical expert in the last window: 5 and 7 got hot


def new_placement():
    from tensor_rtl import balanced_placement
    return balanced_placement(LOAD, 4, 3, previous=OLD)   # the same list on every rank; experts stay where they can


def rank_loads(placement, world, local):
    """Tokens per rank when every expert's load is split evenly over its copies."""
    copies = [placement.count(e) for e in range(len(LOAD))]
    out = [0.0] * world
    for slot, e in enumerate(placement):
        out[slot // local] += LOAD[e] / copies[e]
    return out


def weights_of(expert: int):
    """(w13 [8, 4] bf16, w2 [4, 4] bf16, scale [4] fp32) of a logical expert: recognisable values."""
    w13 = torch.full((8, 4), float(expert), dtype=torch.bfloat16) + torch.arange(4, dtype=torch.bfloat16)
    w2 = torch.full((4, 4), float(-expert), dtype=torch.bfloat16)
    return w13, w2, torch.full((4,), expert + 0.5)


def main(rank: int, world: int, port: int) -> str:
    import torch.distributed as dist
    from tensor_rtl import All2AllVExcutor, ExpertMigrator
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    from tensor_rtl import remap_topk, replica_table
    NEW = new_placement()
    local = len(OLD) // world
    mine = [weights_of(e) for e in OLD[rank * local:(rank + 1) * local]]
    experts = [torch.stack([m[i] for m in mine]) for i in range(3)]          # [local, ...] per weight kind
    mig = ExpertMigrator(rank, world, local, backend="gloo")
    tasks = mig.plan(OLD, NEW, experts)
    ex = All2AllVExcutor()
    ex.execute(tasks)          # every rank calls it, also with an empty list (it is a collective)
    ex.wait()
    changed = mig.apply(experts)
    ok = True
    for s, e in enumerate(NEW[rank * local:(rank + 1) * local]):
        ok &= all(torch.equal(experts[i][s], w) for i, w in enumerate(weights_of(e)))
    want_changed = sum(1 for s in range(rank * local, (rank + 1) * local) if OLD[s] != NEW[s])
    # routing after the move: every (token, choice) lands on a slot that holds the chosen expert, spread over its copies
    g = torch.Generator().manual_seed(rank)
    topk = torch.multinomial(torch.tensor(LOAD, dtype=torch.float32).expand(256, -1), 2, generator=g).to(torch.int32)
    table, counts = replica_table(NEW, len(LOAD))
    phys = remap_topk(topk, table, counts, token_offset=rank)
    ok &= bool((torch.tensor(NEW)[phys.long()] == topk).all())
    before, after = rank_loads(OLD, world, local), rank_loads(NEW, world, local)
    ok &= max(after) / (sum(after) / world) < 1.25 < max(before) / (sum(before) / world)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print(f"placement {NEW}; hottest rank / mean: {max(before) / (sum(before) / world):.2f} -> {max(after) / (sum(after) / world):.2f}")
    return "ok" if ok and changed == want_changed else f"mismatch (changed {changed}, expected {want_changed})"


if __name__ == "__main__":
    res = _launch.run(main, 4, _launch.free_port())
    print(res)
    sys.exit(0 if all(r == "ok" for r in res) else 1)
