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
