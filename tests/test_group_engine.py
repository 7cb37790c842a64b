"""The group engine over a live config store: barrier / all-gather rounds, sub-groups, unique numbers,
dynamic join / leave, and eviction of a member whose link broke. Ranks are threads of one process, each
with its own store connection."""
import ctypes as C
import os
import threading
import time

import pytest


import hooks as H  # noqa: E402
from conftest import free_port  # noqa: E402


@pytest.fixture()
def server():
    port = free_port()
    h = H.start_server(port, world=8)
    yield port
    H.lib().mf_t_server_stop(h)


def _run(n, fn):
    out, errs = [None] * n, []

    def wrap(r):
        try:
            out[r] = fn(r)
        except BaseException as e:  # noqa: BLE001
            errs.append((r, repr(e)))
    ts = [threading.Thread(target=wrap, args=(r,)) for r in range(n)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(60)
    assert not errs, errs
    return out


def test_static_barrier_allgather_subgroups_numbers(server):
    l = H.lib()
    n = 4

    def rank(r):
        st = H.Store.connect(server, world=8, rank=r)
        g = l.mf_t_group_new(st.h, n, r, 10000, 0, H.CHANGE_CB(0))
        assert g
        for round_ in range(5):                      # more rounds than the key garbage-collection lag
            assert l.mf_t_group_barrier(g) == 0
            recv = C.create_string_buffer(4 * n)
            mine = bytes([r, round_, 0xAB, r + round_])
            assert l.mf_t_group_allgather(g, mine, 4, recv, 4 * n) == 0
            assert recv.raw == b"".join(bytes([p, round_, 0xAB, p + round_]) for p in range(n))
        # sub-groups {0, 2} and {1, 3} run at the same time under different keys
        sub, srank = r % 2, r // 2
        key = f"pair{sub}".encode()
        assert l.mf_t_group_sub_barrier(g, key, 2, srank) == 0
        recv = C.create_string_buffer(2)
        assert l.mf_t_group_sub_allgather(g, key, 2, srank, bytes([r]), 1, recv, 2) == 0
        assert recv.raw == bytes([sub, sub + 2])
        v = C.c_int32(-1)
        assert l.mf_t_group_alloc_number(g, 16, C.byref(v)) == 0
        l.mf_t_group_barrier(g)
        l.mf_t_group_free(g)
        st.close()
        return v.value
    nums = _run(n, rank)
    assert len(set(nums)) == n and all(0 <= v < 16 for v in nums)


def test_barrier_times_out_when_a_rank_never_arrives(server):
    l = H.lib()
    st = H.Store.connect(server, world=8, rank=0)
    g = l.mf_t_group_new(st.h, 2, 0, 300, 0, H.CHANGE_CB(0))
    t0 = time.time()
    assert l.mf_t_group_barrier(g) == H.ERR_TIMEOUT
    assert 0.25 <= time.time() - t0 < 5
    l.mf_t_group_free(g)
    st.close()


def test_dynamic_join_leave_and_link_down(server):
    l = H.lib()
    n = 3
    events = [[] for _ in range(n)]
    stores, groups, cbs = [None] * n, [None] * n, [None] * n
    start = threading.Barrier(n)

    def info(g):
        v, s, e, b = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint64()
        l.mf_t_group_info(g, C.byref(v), C.byref(s), C.byref(e), C.byref(b))
        return v.value, s.value, e.value, b.value

    def wait_for(pred, what, secs=10):
        end = time.time() + secs
        while time.time() < end:
            if pred():
                return
            time.sleep(0.02)
        raise AssertionError(f"timed out waiting for {what}")

    def rank(r):
        stores[r] = H.Store.connect(server, world=8, rank=r)
        cbs[r] = H.CHANGE_CB(lambda ev, who, r=r: (events[r].append((ev, who)), 0)[1])
        groups[r] = l.mf_t_group_new(stores[r].h, n, r, 10000, 1, cbs[r])
        assert l.mf_t_group_start_listen(groups[r]) == 0
        start.wait()
        time.sleep(0.05 * r)                         # joins are serialised by the store anyway; stagger to keep logs readable
        assert l.mf_t_group_join(groups[r]) == 0 and l.mf_t_group_joined(groups[r]) == 1
        return True
    _run(n, rank)
    # the joiner's record is visible (odd version: event in flight) before the closing update (even version) reaches everyone
    wait_for(lambda: all(info(g)[1] == n and info(g)[3] == 0b111 and info(g)[0] % 2 == 0 for g in groups) and
             len({info(g)[0] for g in groups}) == 1, "all three members visible everywhere, no event in flight")
    assert (0, 2) in events[0] and (0, 2) in events[1]              # the earlier members were told about rank 2

    # rank 1 leaves in an orderly way
    assert l.mf_t_group_leave(groups[1]) == 0
    wait_for(lambda: info(groups[0])[3] == 0b101 and info(groups[2])[3] == 0b101, "rank 1 gone")
    assert (1, 1) in events[0] and (1, 1) in events[2]

    # rank 2's connection dies: the survivor evicts it through the link-down path
    H.lib().mf_t_client_set_reconnect(stores[2].h, 0, 10)
    H.lib().mf_t_client_crash(stores[2].h)
    wait_for(lambda: info(groups[0])[3] == 0b001, "rank 2 evicted after its link broke")
    assert (3, 2) in events[0]
    assert l.mf_t_group_size(groups[0]) == 1
    for r in range(n):
        l.mf_t_group_free(groups[r])
        stores[r].close()
