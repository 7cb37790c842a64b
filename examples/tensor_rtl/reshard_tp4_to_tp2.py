"""Weights sharded TP4 on ranks 0-3 are resharded to TP2 on ranks 2-3 (a training layout handed to a smaller
serving group), with the all-to-all-v executor over gloo; swap in BatchP2PExecutor or MemoryFabricExecutor
without touching the plan. Counterpart of the reference's examples/verl weight-reshard flow, reduced to its core.

    python examples/tensor_rtl/reshard_tp4_to_tp2.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import _launch  # noqa: E402


def main(rank: int, world: int, port: int) -> str:
    import torch.distributed as dist
    from tensor_rtl import All2AllVExcutor, PTensor, PTensorSet
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    old, new = [0, 1, 2, 3], [2, 3]
    full = {"qkv.weight": torch.arange(48 * 16, dtype=torch.float32).reshape(48, 16),       # column-parallel: shard rows
            "o.weight": torch.arange(16 * 48, dtype=torch.float32).reshape(16, 48) * 0.5}   # row-parallel: shard columns
    dims = {"qkv.weight": 0, "o.weight": 1}
    pts = []
    for name, w in full.items():
        shard = w.chunk(len(old), dims[name])[old.index(rank)].contiguous() if rank in old else None
        pts.append(PTensor(shard, w.dtype, w.ndim, old, tuple(w.shape), dims[name], rank=rank, backend="gloo"))
    ps = PTensorSet(pts)
    ps.transfer_map(new)
    ex = All2AllVExcutor()
    ex.execute(ps.get_transfer_list())
    ex.wait()
    ok = True
    for (name, w), got in zip(full.items(), ps.collect_tensor()):
        if rank in new:
            ok &= torch.equal(got, w.chunk(len(new), dims[name])[new.index(rank)])
        else:
            ok &= got is None
    dist.barrier()
    dist.destroy_process_group()
    return "ok" if ok else "mismatch"


if __name__ == "__main__":
    res = _launch.run(main, 4, _launch.free_port())
    print(res)
    sys.exit(0 if all(r == "ok" for r in res) else 1)
