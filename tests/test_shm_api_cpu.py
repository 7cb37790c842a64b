"""The symmetric shared-memory API over the fake device backend (host memory stands in for HBM): every
rank sees every slice at gva + r * symmetric_size, plus the control-plane helpers."""
import ctypes as C
import os
import time

from conftest import free_port
from mp_util import run_ranks


def _rank(rank, world, url):
    os.environ["MF_DEVICE_BACKEND"] = "fake"
    import memfabric_hybrid_b200.api as mf
    from memfabric_hybrid_b200.api import shm
    assert mf.initialize() == 0
    cfg = shm.ShmConfig()
    cfg.start_store = rank == 0
    assert shm.initialize(url, world, rank, 0, cfg) == 0
    s = shm.create(0, world, rank, 4 << 20)
    assert (s.local_rank, s.rank_size) == (rank, world) and s.symmetric_size >= 4 << 20
    assert s.query_support_data_operation() != 0 and s.set_context(b"ctx-%d" % rank) == 0
    # every rank writes a tag into its own slice; after a barrier every rank reads all slices directly
    mine = s.gva + rank * s.symmetric_size
    C.memmove(mine, bytes([0xA0 + rank]) * 64, 64)
    assert s.barrier() == 0
    for r in range(world):
        assert C.string_at(s.gva + r * s.symmetric_size, 64) == bytes([0xA0 + r]) * 64
    assert s.all_gather(bytes([rank, rank * 2])) == b"".join(bytes([r, r * 2]) for r in range(world))
    sub, srank = rank % 2, rank // 2
    assert s.subgroup_barrier(f"g{sub}", world // 2, srank) == 0
    assert s.subgroup_all_gather(f"g{sub}", world // 2, srank, bytes([rank])) == bytes(range(sub, world, 2))
    assert s.topology_can_reach((rank + 1) % world) > 0
    v = s.atomic_alloc_value(8)
    vals = s.all_gather(bytes([v]))
    assert len(set(vals)) == world and all(x < 8 for x in vals)
    assert s.atomic_release_value(v) == 0
    # global exit: rank 0 announces a status, the others' callbacks receive it
    got = []
    cb_holder = lambda status: got.append(status)  # noqa: E731
    if rank != 0:
        assert s.register_exit(cb_holder) == 0
    assert s.barrier() == 0
    if rank == 0:
        s.global_exit(42)
    else:
        end = time.time() + 10
        while not got and time.time() < end:
            time.sleep(0.02)
        assert got == [42]
    assert s.barrier() == 0
    assert s.destroy() == 0
    shm.uninitialize(0)
    mf.uninitialize()
    return True


def test_symmetric_memory_and_control_plane():
    url = f"tcp://127.0.0.1:{free_port()}"
    assert run_ranks(_rank, 4, (url,), timeout=120) == [True] * 4
