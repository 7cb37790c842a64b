"""The all-reduce entry point that allocates nothing, called through its exported C symbol.

Some callers cannot allocate device memory when they need a collective (an inference engine that gave all
free HBM to its KV cache, a plugin whose host forbids cudaMalloc), so the library carries the staging and
flag scratch itself. The result must equal what the regular entry point produces on an emulated heap, on
two calls in a row (the second call reuses the scratch the first one left behind)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sym():
    from memfabric_hybrid_b200 import _native
    lib = _native.cuda()
    fn = lib.mf_allreduce_stacked_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_uint64, C.c_int, C.c_int, C.c_float, C.c_void_p]
    lib.mf_noalloc_strerror.restype = C.c_char_p
    lib.mf_noalloc_strerror.argtypes = [C.c_int]
    return lib, fn


@pytest.mark.parametrize("world,n,dtype,code", [(4, 50_000, torch.bfloat16, 0), (8, 200_000, torch.float32, 2), (2, 8, torch.bfloat16, 0)])
def test_no_alloc_matches_regular_entry_point(world, n, dtype, code):
    from memfabric_hybrid_b200.ops.heap import EmulatedHeap
    from memfabric_hybrid_b200.ops.collectives import Communicator
    lib, fn = _sym()
    heap = EmulatedHeap(world, (1 << 20) + 4 * (1 << 20) + 4096)
    comm = Communicator(heap, stage_bytes=1 << 20)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        torch.manual_seed(100 * call + n)
        x = torch.randn(world, n, device="cuda").to(dtype)
        want = comm.all_reduce(x, scale=1.0 / world, algo="oneshot")
        got = torch.empty_like(x)
        before = torch.cuda.memory_allocated()
        rc = fn(x.data_ptr(), got.data_ptr(), world, n, code, 0, 1.0 / world, stream)
        assert rc == 0, lib.mf_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(got.float(), want.float(), **tol)
        assert torch.equal(got, want), "same kernel, same order of additions: the bits must agree"
    assert heap.status()[0] == 0


def test_no_alloc_rejects_oversize_and_bad_arguments():
    lib, fn = _sym()
    x = torch.zeros(2, 16, device="cuda")
    too_many = (1 << 20) // 4 + 1
    assert fn(x.data_ptr(), x.data_ptr(), 2, too_many, 2, 0, 1.0, None) == -2
    assert b"1 MiB" in lib.mf_noalloc_strerror(-2)
    assert fn(x.data_ptr(), x.data_ptr(), 9, 16, 2, 0, 1.0, None) == -1
    assert fn(None, x.data_ptr(), 2, 16, 2, 0, 1.0, None) == -1
