"""Neighbour exchange on the symmetric shared memory with a user kernel (csrc/kernels/mf_shm_example.cu,
k_example_shift): every rank PUTs its vector into the next rank's slice and is told by a one-way device signal
when its own box has been filled; then every rank GETs the previous rank's vector between two device barriers.

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/hbm_share_memory/shift_put_get.py

With one process it runs as a world of one (the neighbour is the rank itself). Counterpart of
examples/hbm_share_memory/ShiftPutGet of the reference.
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
    fn = cu.mf_example_shm_shift
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_int, C.c_uint32, C.c_void_p, C.c_void_p]
    assert mf.initialize() == 0
    cfg = shm.ShmConfig()
    cfg.start_store = rank == 0
    assert shm.initialize(store_url, world, rank, device, cfg) == 0
    s = shm.create(0, world, rank, shm.USER_OFFSET + 8 * n)
    ctx = s.device_context()
    mine = s.gva + rank * s.symmetric_size
    tensor_at(mine, (shm.USER_OFFSET,), torch.uint8).zero_()            # the flag area starts from zero
    src = tensor_at(mine + shm.USER_OFFSET, (n,), torch.float32)        # what this rank hands on
    box = tensor_at(mine + shm.USER_OFFSET + 4 * n, (n,), torch.float32)  # where a neighbour's vector lands
    base = torch.arange(n, device="cuda", dtype=torch.float32) % 251
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    prev = (rank - 1) % world
    stream = torch.cuda.current_stream().cuda_stream
    err = 0.0
    for mode in (0, 1):                                                 # put, then get
        src.copy_(base + 1000 * mode + rank)
        box.fill_(-1.0)
        torch.cuda.synchronize()
        s.barrier()                                                     # everybody's src and box are ready
        assert fn(C.byref(ctx), src.data_ptr(), box.data_ptr(), n, mode, 1, status.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0, "a neighbour did not arrive"
        err = max(err, float((box - (base + 1000 * mode + prev)).abs().max()))
        s.barrier()
    s.destroy()
    shm.uninitialize(0)
    mf.uninitialize()
    return err


if __name__ == "__main__":
    r, w = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    url = f"tcp://{os.environ.get('MASTER_ADDR', '127.0.0.1')}:{int(os.environ.get('MASTER_PORT', 29500)) + 29}"
    e = run(r, w, int(os.environ.get("LOCAL_RANK", 0)), url)
    print(f"rank {r}/{w}: max abs error {e}")
    sys.exit(0 if e == 0.0 else 1)
