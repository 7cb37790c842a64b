"""Expert-parallel load balancing: 4 EP ranks hold 3 physical expert slots each (8 logical experts plus 4
redundant copies of hot ones). A new placement arrives; ``ExpertMigrator`` moves the experts whose slot changed
with one all-to-all-v and every rank checks its slots against the new placement. Counterpart of the reference's
examples/eplb flow without the serving engine around it.

    python examples/tensor_rtl/eplb_expert_migration.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import _launch  # noqa: E402

OLD = [0, 1, 2,  3, 4, 5,  6, 7, 0,  1, 2, 3]      # slot -> logical expert; rank r owns slots 3r .. 3r+2
NEW = [0, 5, 5,  3, 4, 0,  6, 7, 7,  2, 1, 3]      # expert 5 and 7 got hot: extra copies; some slots just swap


def weights_of(expert: int):
    """(w13 [8, 4] bf16, w2 [4, 4] bf16, scale [4] fp32) of a logical expert: recognisable values."""
    w13 = torch.full((8, 4), float(expert), dtype=torch.bfloat16) + torch.arange(4, dtype=torch.bfloat16)
    w2 = torch.full((4, 4), float(-expert), dtype=torch.bfloat16)
    return w13, w2, torch.full((4,), expert + 0.5)


def main(rank: int, world: int, port: int) -> str:
    import torch.distributed as dist
    from tensor_rtl import All2AllVExcutor, ExpertMigrator
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
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
    dist.barrier()
    dist.destroy_process_group()
    return "ok" if ok and changed == want_changed else f"mismatch (changed {changed}, expected {want_changed})"


if __name__ == "__main__":
    res = _launch.run(main, 4, _launch.free_port())
    print(res)
    sys.exit(0 if all(r == "ok" for r in res) else 1)
