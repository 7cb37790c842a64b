"""Device-side API of the symmetric shared memory beyond the collectives: the user's extra context as a kernel sees it."""
import ctypes as C

import pytest
import torch

from conftest import free_port
from mp_util import run_ranks

pytestmark = pytest.mark.gpu


def _ctx_rank(rank, world, url):
    import torch
    import memfabric_hybrid_b200.api as mf
    from memfabric_hybrid_b200 import _native as N
    from memfabric_hybrid_b200.api import shm
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    cu = N.cuda()
    cu.mf_example_shm_read_context.restype = C.c_int
    cu.mf_example_shm_read_context.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
    assert mf.initialize() == 0
    cfg = shm.ShmConfig()
    cfg.start_store = True
    assert shm.initialize(url, 1, 0, 0, cfg) == 0
    s = shm.create(0, 1, 0, shm.USER_OFFSET + (1 << 20))
    ctx = s.device_context()
    out = torch.full((4096,), 0xEE, dtype=torch.uint8, device="cuda")
    size = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # nothing set yet: the kernel reads size 0 and copies nothing
    assert cu.mf_example_shm_read_context(C.byref(ctx), out.data_ptr(), 4096, size.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(size.item()) == 0 and int(out.min()) == 0xEE
    for blob in (b"tile=128;lanes=4;peer-map=0,1,2,3", bytes(range(256)) * 9 + b"end"):
        assert s.set_context(blob) == 0
        assert cu.mf_example_shm_read_context(C.byref(ctx), out.data_ptr(), 4096, size.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert int(size.item()) == len(blob)
        assert bytes(out[:len(blob)].cpu().tolist()) == blob
    assert s.set_context(b"") != 0 and s.set_context(b"x" * 65537) != 0
    mf.get_and_clear_last_err_msg()
    s.destroy()
    shm.uninitialize(0)
    mf.uninitialize()
    return 0


def test_extra_context_is_readable_from_a_kernel():
    """smem_shm_set_extra_context on the host, smem_shm_get_extra_context_addr / _size in a kernel."""
    assert run_ranks(_ctx_rank, 1, (f"tcp://127.0.0.1:{free_port()}",), timeout=120) == [0]


def _helpers_rank(rank, world, url, sync):
    """smem_shm_roce_write / _read and smem_shm_copy_gm2ub / _ub2gm in a kernel: bytes go to the peer's slice, come back,
    and pass through shared memory, bit for bit (odd length: the byte tail of the vector copies is exercised too)."""
    import torch
    import memfabric_hybrid_b200.api as mf
    from memfabric_hybrid_b200 import _native as N
    from memfabric_hybrid_b200.api import shm
    dev = rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    torch.zeros(1, device="cuda")
    cu = N.cuda()
    cu.mf_example_shm_copy_helpers.restype = C.c_int
    cu.mf_example_shm_copy_helpers.argtypes = [C.c_void_p] * 5 + [C.c_uint64, C.c_uint32, C.c_uint32, C.c_void_p, C.c_int, C.c_void_p]
    assert mf.initialize() == 0
    cfg = shm.ShmConfig()
    cfg.start_store = rank == 0
    assert shm.initialize(url, world, rank, dev, cfg) == 0
    nbytes = (3 << 20) + 13
    s = shm.create(0, world, rank, shm.USER_OFFSET + (8 << 20))
    ctx = s.device_context()
    box = s.local_ptr() + shm.USER_OFFSET if hasattr(s, "local_ptr") else int(ctx.base) + rank * int(ctx.symmetric_size) + shm.USER_OFFSET
    src = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device="cuda", generator=torch.Generator("cuda").manual_seed(rank))
    back = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    via = torch.zeros(32768, dtype=torch.uint8, device="cuda")
    ok = torch.zeros(1, dtype=torch.int32, device="cuda")
    peer = (rank + 1) % world
    sync.wait()      # every rank's slice is mapped before anybody stores into it
    assert cu.mf_example_shm_copy_helpers(C.byref(ctx), src.data_ptr(), box, back.data_ptr(), via.data_ptr(), nbytes, 32768, peer,
                                          ok.data_ptr(), 32, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    good = int(ok.item()) == 1 and torch.equal(back, src) and torch.equal(via, src[:32768])
    sync.wait()      # nobody unmaps a slice a peer still reads
    s.destroy()
    shm.uninitialize(0)
    mf.uninitialize()
    return 0 if good else 1


def test_copy_helpers_single_gpu():
    assert run_ranks(_helpers_rank, 1, (f"tcp://127.0.0.1:{free_port()}",), timeout=120, with_barrier=True) == [0]


@pytest.mark.multigpu
def test_copy_helpers_two_gpus():
    assert run_ranks(_helpers_rank, 2, (f"tcp://127.0.0.1:{free_port()}",), timeout=180, with_barrier=True) == [0, 0]
