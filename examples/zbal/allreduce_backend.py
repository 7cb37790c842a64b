"""``torch.distributed`` on the "zbal" backend with tensors from the symmetric allocator. Needs GPUs.

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/zbal/allreduce_backend.py

Importing ``zbal`` registers the backend; ``zbal_init`` maps every rank's slice of the symmetric heap into every
process; tensors created under ``switch_to_allocator()`` live in that heap, so the collective kernels read and
write them in place on the peers (no staging copies). The flow of app/zbal/doc/user_guide/get_started.md of the
reference.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import zbal  # noqa: E402


def main() -> int:
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    zbal.zbal_init(world, local, rank, 2 << 30, start_config_server=True)
    dist.init_process_group("zbal", rank=rank, world_size=world)
    with zbal.switch_to_allocator():
        grads = torch.full((8 << 20,), float(rank + 1), device="cuda", dtype=torch.bfloat16)
    dist.all_reduce(grads, op=dist.ReduceOp.AVG)
    want = sum(range(1, world + 1)) / world
    ok = bool((grads.float() - want).abs().max() < 0.05)
    shard = torch.full((1 << 20,), float(rank), device="cuda")
    full = torch.empty(world << 20, device="cuda")
    dist.all_gather_into_tensor(full, shard)
    ok &= bool(torch.equal(full.view(world, -1)[:, 0].cpu(), torch.arange(world, dtype=torch.float32)))
    free, total = zbal.mem_get_info()
    print(f"rank {rank}: all_reduce/all_gather {'ok' if ok else 'WRONG'}; symmetric heap {total - free >> 20} of {total >> 20} MiB in use")
    del grads
    torch.cuda.synchronize()
    dist.destroy_process_group()
    zbal.zbal_uninit()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
