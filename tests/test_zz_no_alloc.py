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
    lib.mf_noalloc_status.restype = C.c_int
    lib.mf_noalloc_status.argtypes = [C.POINTER(C.c_uint32), C.c_int]
    return lib, fn


def _status(lib):
    """(code, words) of the status words inside the built-in scratch of the current device."""
    words = (C.c_uint32 * 4)()
    return lib.mf_noalloc_status(words, 0), list(words)


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
        # independent of any kernel of this library: the fp32 sum of the stacked vectors, on every row
        oracle = (x.float().sum(0) / world).expand(world, n)
        torch.testing.assert_close(got.float(), oracle, **tol)
        assert _status(lib) == (0, [0, 0, 0, 0]), "a bounded wait inside the call ran out"
    assert heap.status()[0] == 0


_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2, torch.int32: 3}


@pytest.mark.parametrize("dtype,op", [(torch.float16, "sum"), (torch.int32, "sum"), (torch.float32, "max"), (torch.float32, "min"),
                                      (torch.bfloat16, "max")])
def test_no_alloc_against_a_torch_oracle_on_a_side_stream(dtype, op):
    """Other dtypes and operators, checked only against PyTorch, on a non-blocking side stream (the stream kind on which
    work queued elsewhere would not be ordered with the call), twice in a row."""
    lib, fn = _sym()
    world, n = 4, 33_333
    side = torch.cuda.Stream()
    for call in range(2):
        torch.manual_seed(7 * call + n)
        if dtype == torch.int32:
            x = torch.randint(-1000, 1000, (world, n), device="cuda", dtype=torch.int32)
        else:
            x = torch.randn(world, n, device="cuda").to(dtype)
        got = torch.full_like(x, 77)
        torch.cuda.synchronize()          # the inputs are complete before the side stream reads them
        with torch.cuda.stream(side):
            rc = fn(x.data_ptr(), got.data_ptr(), world, n, _DT[dtype], {"sum": 0, "max": 1, "min": 2}[op], 1.0, side.cuda_stream)
        assert rc == 0, lib.mf_noalloc_strerror(rc).decode()
        side.synchronize()
        assert _status(lib) == (0, [0, 0, 0, 0])
        if op == "sum":
            want = x.sum(0) if dtype == torch.int32 else x.float().sum(0)
        else:
            want = getattr(x.float(), op)(0).values
        want = want.expand(world, n)
        if dtype == torch.int32:
            assert torch.equal(got, want.to(torch.int32))
        elif op == "sum":
            torch.testing.assert_close(got.float(), want, rtol=1e-2, atol=1e-2)
        else:
            assert torch.equal(got.float(), want), "a maximum or minimum of representable values is exact"


def test_no_alloc_rejects_oversize_and_bad_arguments():
    lib, fn = _sym()
    x = torch.zeros(2, 16, device="cuda")
    too_many = (1 << 20) // 4 + 1
    assert fn(x.data_ptr(), x.data_ptr(), 2, too_many, 2, 0, 1.0, None) == -2
    assert b"1 MiB" in lib.mf_noalloc_strerror(-2)
    assert fn(x.data_ptr(), x.data_ptr(), 9, 16, 2, 0, 1.0, None) == -1
    assert fn(None, x.data_ptr(), 2, 16, 2, 0, 1.0, None) == -1
    assert lib.mf_noalloc_status(None, 0) == -1
    assert b"bounded wait" in lib.mf_noalloc_strerror(-5)
