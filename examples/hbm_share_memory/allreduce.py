"""A user kernel on the symmetric shared memory: every rank keeps an fp32 vector in its slice and a small
kernel (csrc/kernels/mf_shm_example.cu, written against csrc/include/smem_shm_device.cuh) sums the
vectors of all ranks by reading the peers' slices over NVLink.

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/hbm_share_memory/allreduce.py

With one process it runs as a world of one. Counterpart of examples/hbm_share_memory/AllReduce of the reference.
"""
import ctypes as C
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import memfabric_hybrid_b200.api as mf  # noqa: E402
from memfabric_hybrid_b200 import _native as N  # noqa: E402
from memfabric_hybrid_b200.api import shm  # noqa: E402
from memfabric_hybrid_b200.ops.heap import tensor_at  # noqa: E402


def run(rank: int, world: int, device: int, store_url: str, n: int = 1 << 20) -> float:
    torch.cuda.set_device(device)
    torch.zeros(1, device="cuda")
    cu = N.cuda()
    cu.mf_example_shm_allreduce.restype = C.c_int
    cu.mf_example_shm_allreduce.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32, C.c_void_p, C.c_void_p]
    assert mf.initialize() == 0
    cfg = shm.ShmConfig()
    cfg.start_store = rank == 0
    assert shm.initialize(store_url, world, rank, device, cfg) == 0
    s = shm.create(0, world, rank, shm.USER_OFFSET + 4 * n)
    ctx = s.device_context()
    mine = s.gva + rank * s.symmetric_size
    tensor_at(mine, (shm.USER_OFFSET,), torch.uint8).zero_()       # the flag area starts from zero
    x = tensor_at(mine + shm.USER_OFFSET, (n,), torch.float32)     # this rank's vector, inside its slice
    x.copy_(torch.arange(n, device="cuda", dtype=torch.float32) % 97 + rank)
    out = torch.empty(n, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    s.barrier()
    for epoch in (1, 2):                                           # twice: the flags need no reset between calls
        rc = cu.mf_example_shm_allreduce(C.byref(ctx), x.data_ptr(), out.data_ptr(), n, epoch, status.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
        assert rc == 0, rc
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a peer did not arrive"
    expect = (torch.arange(n, device="cuda", dtype=torch.float32) % 97) * world + sum(range(world))
    err = float((out - expect).abs().max())
    s.barrier()
    s.destroy()
    shm.uninitialize(0)
    mf.uninitialize()
    return err


if __name__ == "__main__":
    r, w = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    url = f"tcp://{os.environ.get('MASTER_ADDR', '127.0.0.1')}:{int(os.environ.get('MASTER_PORT', 29500)) + 23}"
    e = run(r, w, int(os.environ.get("LOCAL_RANK", 0)), url)
    print(f"rank {r}/{w}: max abs error {e}")
    sys.exit(0 if e == 0.0 else 1)
