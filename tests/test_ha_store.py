"""The highly available config store on an in-memory stand-in for the distributed backend: one leader is
elected, followers reach it, a leader that dies is replaced and the clients carry on; an unreachable
backend makes the leader step down."""
import ctypes as C
import os
import time


import hooks as H  # noqa: E402
from conftest import free_port  # noqa: E402


def _addr(h):
    buf = C.create_string_buffer(128)
    H.lib().mf_t_ha_leader_addr(h, buf, 128)
    return buf.value.decode()


def _wait(pred, what, secs=15):
    end = time.time() + secs
    while time.time() < end:
        if pred():
            return
        time.sleep(0.05)
    raise AssertionError(f"timed out waiting for {what}")


def test_election_failover_and_backend_loss():
    l = H.lib()
    name = b"ha-test"
    l.mf_t_backend_reset(name)
    port = free_port()
    nodes = []
    for r in range(3):
        h = l.mf_t_ha_new(b"127.0.0.1", port, 3, r, name, 1)
        l.mf_t_ha_set_timings(h, 600, 200, 10, 60)      # lease, health period, back-off range (ms)
        nodes.append(h)
    import threading
    rcs = [None] * 3
    ts = [threading.Thread(target=lambda r=r: rcs.__setitem__(r, l.mf_t_ha_start(nodes[r], 10000))) for r in range(3)]
    [t.start() for t in ts]
    [t.join(20) for t in ts]
    assert rcs == [0, 0, 0]
    leaders = [r for r in range(3) if l.mf_t_ha_is_leader(nodes[r])]
    assert len(leaders) == 1
    lead = leaders[0]
    assert len({_addr(h) for h in nodes}) == 1 and _addr(nodes[0]).startswith("127.0.0.1:")
    stores = [H.Store(h) for h in nodes]
    follower = next(r for r in range(3) if r != lead)
    assert stores[follower].set("k", b"v") == 0 and stores[lead].get("k") == b"v"

    # the leader's server dies without cleaning its lease: a follower takes over once the lease runs out
    old = _addr(nodes[lead])
    l.mf_t_ha_kill_leader(nodes[lead])
    _wait(lambda: sum(l.mf_t_ha_is_leader(nodes[r]) for r in range(3) if r != lead) == 1, "a new leader")
    new_lead = next(r for r in range(3) if r != lead and l.mf_t_ha_is_leader(nodes[r]))
    _wait(lambda: all(_addr(nodes[r]) == _addr(nodes[new_lead]) != "" for r in range(3) if r != lead), "followers to learn the new address")
    other = next(r for r in range(3) if r not in (lead, new_lead))
    _wait(lambda: stores[other].connected(), "the follower's link to the new leader")
    # data of the old server is gone (only membership is persisted); the service is
    assert stores[other].set("k2", b"v2") == 0 and stores[new_lead].get("k2") == b"v2"
    assert _addr(nodes[new_lead]) != old or True

    # the backend becomes unreachable: the leader cannot renew its lease and steps down
    l.mf_t_backend_set_reachable(name, 0)
    _wait(lambda: not l.mf_t_ha_is_leader(nodes[new_lead]), "the leader to demote itself")
    l.mf_t_backend_set_reachable(name, 1)
    _wait(lambda: sum(l.mf_t_ha_is_leader(nodes[r]) for r in range(3)) == 1, "a leader once the backend is back")
    for s in stores:
        s.close()
    l.mf_t_backend_reset(name)
