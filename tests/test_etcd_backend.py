"""The etcd v3 backend of the highly available config store (native client over etcd's JSON gateway), against an
in-process stand-in for the gateway: keys with and without a lease, prefix reads, named locks, authentication, an
unreachable service, and the store's leader election running on it, through the test hooks and through an etcd:// URL."""
import ctypes as C
import threading
import time

import pytest

import hooks as H  # noqa: E402
from conftest import free_port  # noqa: E402
from fake_etcd import FakeEtcd


class Etcd:
    def __init__(self, port, instance=b"", user=None, password=None, timeout_ms=2000):
        self.l = H.lib()
        self.h = self.l.mf_t_etcd_new(b"127.0.0.1", port, instance, user, password, timeout_ms)

    def close(self):
        if self.h:
            self.l.mf_t_etcd_free(self.h)
            self.h = None

    def put(self, k, v, ttl_ms=0):
        return self.l.mf_t_etcd_put(self.h, k.encode(), v, len(v), ttl_ms)

    def get(self, k):
        buf = C.create_string_buffer(1 << 16)
        n = self.l.mf_t_etcd_get(self.h, k.encode(), buf, len(buf))
        return n if n < 0 else buf.raw[:n]

    def keys(self, prefix):
        buf = C.create_string_buffer(1 << 16)
        n = self.l.mf_t_etcd_prefix_get(self.h, prefix.encode(), buf, len(buf))
        assert n >= 0, n
        return [tuple(line.split("=", 1)) for line in buf.raw[:n].decode().splitlines()]

    def error(self):
        buf = C.create_string_buffer(512)
        self.l.mf_t_etcd_last_error(self.h, buf, 512)
        return buf.value.decode()

    def __getattr__(self, name):   # delete, clear, exist, lock, try_lock, unlock, connect
        fn = getattr(self.l, "mf_t_etcd_" + name)
        return lambda *a: fn(self.h, *[x.encode() if isinstance(x, str) else x for x in a])


@pytest.fixture
def etcd():
    f = FakeEtcd()
    yield f
    f.close()


def test_keys_values_prefixes_and_instances(etcd):
    a, b = Etcd(etcd.port, b"poolA"), Etcd(etcd.port, b"poolB")
    try:
        assert a.connect() == 0
        assert a.get("/x/1") == H.ERR_NOT_EXIST and a.exist("/x/1") == 0
        blob = bytes(range(256)) * 3 + b"\0tail"
        assert a.put("/x/1", blob) == 0 and a.get("/x/1") == blob
        assert a.put("/x/2", b"") == 0 and a.get("/x/2") == b""          # an empty value is a value
        assert a.put("/x/10", b"ten") == 0 and a.put("/y/1", b"other") == 0 and a.put("plain", b"p") == 0
        assert a.put("/x/1", b"again") == 0 and a.get("/x/1") == b"again"
        assert a.keys("/x/") == [("/x/1", "again"), ("/x/10", "ten"), ("/x/2", "")]   # sorted by key, names as written
        assert a.keys("pla") == [("plain", "p")]
        # another instance id is another key space in the same etcd
        assert b.get("/x/1") == H.ERR_NOT_EXIST and b.keys("/x/") == []
        assert b.put("/x/1", b"theirs") == 0 and a.get("/x/1") == b"again"
        root = b"/memfabric_hybrid/config_store/clusters/poolA/"
        assert root + b"x/1" in etcd.kv and root + b"plain" in etcd.kv
        assert a.delete("/x/10") == 0 and a.delete("/x/10") == H.ERR_NOT_EXIST
        assert a.clear("/x/") == 0 and a.keys("/x/") == [] and a.get("/y/1") == b"other"
        assert b.get("/x/1") == b"theirs"                                   # clearing one instance leaves the other alone
        # a key without an instance id is stored as given
        c = Etcd(etcd.port)
        assert c.put("/memfabric_hybrid/raw", b"r") == 0 and etcd.kv[b"/memfabric_hybrid/raw"]["value"] == b"r"
        c.close()
    finally:
        a.close()
        b.close()


def test_a_key_with_a_ttl_expires_and_is_renewed_by_writing_it_again(etcd):
    a = Etcd(etcd.port, b"ttl")
    try:
        assert a.put("/leader", b"10.0.0.1:4000", 900) == 0          # rounded up to a 1 s lease
        assert len(etcd.leases) == 1 and a.get("/leader") == b"10.0.0.1:4000"
        time.sleep(0.6)
        assert a.put("/leader", b"10.0.0.1:4000", 900) == 0          # the renewal: a new lease, the old one revoked
        assert len(etcd.leases) == 1
        time.sleep(0.6)
        assert a.get("/leader") == b"10.0.0.1:4000"                   # 1.2 s after the first write: alive thanks to the second
        time.sleep(0.7)
        assert a.get("/leader") == H.ERR_NOT_EXIST and len(etcd.leases) == 0
        assert a.put("/leader", b"x", 900) == 0 and a.put("/leader", b"y") == 0   # rewritten without a TTL: stays
        time.sleep(1.2)
        assert a.get("/leader") == b"y"
    finally:
        a.close()


def test_named_locks_exclude_wait_and_are_freed_when_the_holder_closes(etcd):
    a, b, c = Etcd(etcd.port, b"lk"), Etcd(etcd.port, b"lk"), Etcd(etcd.port, b"lk")
    try:
        assert a.try_lock("backend") == 0
        assert a.try_lock("backend") == H.ERR_IN_USE                 # not re-entrant
        assert b.try_lock("backend") == H.ERR_IN_USE
        assert b.try_lock("other") == 0 and b.unlock("other") == 0   # names are independent
        assert b.unlock("backend") == H.ERR_NOT_EXIST                # only the holder unlocks
        assert len(etcd.leases) == 1                                  # the losers' leases were revoked
        got = []
        t = threading.Thread(target=lambda: got.append((b.lock("backend"), time.monotonic())))
        t.start()
        time.sleep(0.4)
        assert not got
        t0 = time.monotonic()
        assert a.unlock("backend") == 0
        t.join(5)
        assert got and got[0][0] == 0 and got[0][1] - t0 < 1.0
        assert c.try_lock("backend") == H.ERR_IN_USE
        b.close()                                                     # the holder goes away without unlocking
        assert c.try_lock("backend") == 0 and c.unlock("backend") == 0
        assert len(etcd.leases) == 0
    finally:
        a.close()
        b.close()
        c.close()


def test_authentication_and_a_token_that_ran_out():
    f = FakeEtcd(users={"mf": "secret"})
    try:
        bad = Etcd(f.port, b"", b"mf", b"wrong")
        assert bad.connect() == H.ERR_NOT_CONNECTED and "credentials" in bad.error()
        bad.close()
        anon = Etcd(f.port)
        assert anon.put("/k", b"v") != 0 and "401" in anon.error()
        anon.close()
        a = Etcd(f.port, b"", b"mf", b"secret")
        assert a.connect() == 0 and a.put("/k", b"v") == 0 and a.get("/k") == b"v"
        assert f.calls.count("/auth/authenticate") == 2              # one failed log-in above, one for this client
        f.tokens.clear()                                              # the server forgets its tokens (they ran out)
        assert a.get("/k") == b"v"                                    # 401 -> one new log-in -> the call again
        assert f.calls.count("/auth/authenticate") == 3
        a.close()
    finally:
        f.close()


def test_unreachable_or_failing_service():
    port = free_port()
    a = Etcd(port, timeout_ms=300)
    t0 = time.monotonic()
    assert a.connect() == H.ERR_NOT_CONNECTED and a.put("/k", b"v") == H.ERR_NOT_CONNECTED
    assert time.monotonic() - t0 < 2.0 and "cannot reach etcd" in a.error()
    a.close()
    f = FakeEtcd()
    try:
        b = Etcd(f.port)
        assert b.put("/k", b"v") == 0
        f.down = True
        assert b.get("/k") == -1 and "503" in b.error() and b.connect() == H.ERR_NOT_CONNECTED
        f.down = False
        assert b.get("/k") == b"v"
        b.close()
    finally:
        f.close()


def _addr(h):
    buf = C.create_string_buffer(128)
    H.lib().mf_t_ha_leader_addr(h, buf, 128)
    return buf.value.decode()


def _wait(pred, what, secs=20):
    end = time.time() + secs
    while time.time() < end:
        if pred():
            return
        time.sleep(0.05)
    raise AssertionError(f"timed out waiting for {what}")


def test_leader_election_and_failover_on_etcd(etcd):
    l = H.lib()
    port = free_port()
    nodes = []
    for r in range(3):
        h = l.mf_t_ha_new_etcd(b"127.0.0.1", port, 3, r, b"127.0.0.1", etcd.port, b"ha", 1)
        l.mf_t_ha_set_timings(h, 1000, 300, 10, 60)      # lease, health period, back-off range (ms)
        nodes.append(h)
    rcs = [None] * 3
    ts = [threading.Thread(target=lambda r=r: rcs.__setitem__(r, l.mf_t_ha_start(nodes[r], 15000))) for r in range(3)]
    [t.start() for t in ts]
    [t.join(30) for t in ts]
    assert rcs == [0, 0, 0]
    leaders = [r for r in range(3) if l.mf_t_ha_is_leader(nodes[r])]
    assert len(leaders) == 1
    lead = leaders[0]
    root = b"/memfabric_hybrid/config_store/clusters/ha"
    assert etcd.kv[root + b"/memfabric_hybrid/config_store/meta/leader"]["value"].decode() == _addr(nodes[lead])
    assert etcd.kv[root + b"/memfabric_hybrid/config_store/meta/leader"]["lease"] != 0
    stores = [H.Store(h) for h in nodes]
    follower = next(r for r in range(3) if r != lead)
    assert stores[follower].set("k", b"v") == 0 and stores[lead].get("k") == b"v"
    # the leader's server dies: its key lapses with the lease and one of the others takes over
    l.mf_t_ha_kill_leader(nodes[lead])
    _wait(lambda: sum(l.mf_t_ha_is_leader(nodes[r]) for r in range(3) if r != lead) == 1, "a new leader")
    new_lead = next(r for r in range(3) if r != lead and l.mf_t_ha_is_leader(nodes[r]))
    other = next(r for r in range(3) if r not in (lead, new_lead))
    _wait(lambda: _addr(nodes[other]) == _addr(nodes[new_lead]) != "" and stores[other].connected(), "the follower to reach the new leader")
    assert stores[other].set("k2", b"v2") == 0 and stores[new_lead].get("k2") == b"v2"
    # two leaders: the key in etcd names another server that answers (elected while this one looked dead from there):
    # the leader in office steps down and everybody follows the key
    port2 = free_port()
    usurper = H.start_server(port2, world=3)
    try:
        lkey = root + b"/memfabric_hybrid/config_store/meta/leader"
        etcd.kv[lkey]["value"] = f"127.0.0.1:{port2}".encode()
        etcd.kv[lkey]["lease"] = 0
        _wait(lambda: not any(l.mf_t_ha_is_leader(nodes[r]) for r in range(3) if r != lead), "the leader in office to step down")
        _wait(lambda: all(_addr(nodes[r]) == f"127.0.0.1:{port2}" for r in range(3) if r != lead), "everybody to follow the key")
        _wait(lambda: stores[other].connected() and stores[new_lead].connected(), "both links to the server the key names")
        assert stores[other].set("k3", b"v3") == 0 and stores[new_lead].get("k3") == b"v3"
    finally:
        del etcd.kv[lkey]                                  # that server goes away again: a new election
        l.mf_t_server_stop(usurper)
    _wait(lambda: sum(l.mf_t_ha_is_leader(nodes[r]) for r in range(3) if r != lead) == 1, "a leader after the other server left")
    new_lead = next(r for r in range(3) if r != lead and l.mf_t_ha_is_leader(nodes[r]))
    # etcd stops answering: the leader cannot renew and steps down; it comes back: there is a leader again
    etcd.down = True
    _wait(lambda: not l.mf_t_ha_is_leader(nodes[new_lead]), "the leader to demote itself")
    etcd.down = False
    _wait(lambda: sum(l.mf_t_ha_is_leader(nodes[r]) for r in range(3)) == 1, "a leader once etcd answers again")
    for s in stores:
        s.close()


def test_store_url_with_the_etcd_scheme(etcd, monkeypatch):
    from memfabric_hybrid_b200 import api
    monkeypatch.setenv("MF_CONFIG_STORE_PORT", str(free_port()))
    url = f"etcd://127.0.0.1:{etcd.port}#urltest"
    assert api.create_config_store(url) == 0
    try:
        leader = etcd.kv[b"/memfabric_hybrid/config_store/clusters/urltest/memfabric_hybrid/config_store/meta/leader"]
        assert leader["value"].startswith(b"127.0.0.1:") and leader["lease"] != 0
    finally:
        api.destroy_config_store(url)
    # nobody answers at the address: a clear refusal instead of a store
    dead = f"etcd://127.0.0.1:{free_port()}#urltest"
    assert api.create_config_store(dead) != 0


def _pool_over_etcd(rank, world, url, port, sync):
    """A two-rank DRAM pool whose config store is elected over etcd: the whole public path behind an etcd:// URL."""
    import os
    os.environ["MF_CONFIG_STORE_PORT"] = str(port)
    os.environ["MF_DEVICE_BACKEND"] = "none"
    import numpy as np
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    MiB = 1 << 20
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id = rank
    cfg.start_store = True                      # every rank may lead; etcd decides
    cfg.operation_timeout = 30
    assert bm.initialize(url, world, 0, cfg) == 0, mf.get_last_err_msg()
    h = bm.create2(id=0, local_dram_size=8 * MiB, max_dram_size=8 * MiB, data_op_type=bm.BmDataOpType.HOST_SHM)
    assert h.join() == 0, mf.get_last_err_msg()
    sync.wait(60)
    peer = h.peer_rank_ptr(1 - rank, bm.BmMemType.HOST)
    me = h.peer_rank_ptr(rank, bm.BmMemType.HOST)
    src = np.full(MiB, 0x30 + rank, dtype=np.uint8)
    end = time.time() + 30
    while h.copy_data(src.ctypes.data, peer, MiB, bm.BmCopyType.H2G, 0) != 0:
        assert time.time() < end, mf.get_last_err_msg()
        time.sleep(0.05)
    mf.get_and_clear_last_err_msg()
    sync.wait(60)
    got = np.zeros(MiB, dtype=np.uint8)
    assert h.copy_data(me, got.ctypes.data, MiB, bm.BmCopyType.G2H, 0) == 0, mf.get_last_err_msg()
    ok = bool((got == 0x30 + (1 - rank)).all())
    sync.wait(60)
    assert h.leave() == 0
    sync.wait(60)
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    return ok


def test_memory_pool_brought_up_over_an_etcd_url(etcd):
    from mp_util import run_ranks
    url = f"etcd://127.0.0.1:{etcd.port}#pooltest"
    assert run_ranks(_pool_over_etcd, 2, (url, free_port()), timeout=180, with_barrier=True) == [True, True]
    root = b"/memfabric_hybrid/config_store/clusters/pooltest/"
    assert etcd.kv[root + b"memfabric_hybrid/config_store/data/world_size"]["value"] == b"2"
    assert any(k.startswith(root + b"memfabric_hybrid/config_store/meta/leader") for k in etcd.kv)


def _rank0_returns(rank, world, url, port, sync2):
    """A new process takes the place of the rank that died with the store's first leader."""
    import os
    os.environ["MF_CONFIG_STORE_PORT"] = str(port)
    os.environ["MF_DEVICE_BACKEND"] = "none"
    import numpy as np
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    MiB = 1 << 20
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id, cfg.start_store, cfg.operation_timeout = 0, False, 40
    assert bm.initialize(url, world, 0, cfg) == 0, mf.get_last_err_msg()
    h = bm.create2(id=0, local_dram_size=4 * MiB, max_dram_size=4 * MiB, data_op_type=bm.BmDataOpType.HOST_SHM)
    assert h.join() == 0, mf.get_last_err_msg()           # imports the survivors' slices from the records they republished
    sync2.wait(60)
    src = np.full(MiB, 0x70, dtype=np.uint8)
    for r in (1, 2):
        assert h.copy_data(src.ctypes.data, h.peer_rank_ptr(r, bm.BmMemType.HOST) + 2 * MiB, MiB, bm.BmCopyType.H2G, 0) == 0, mf.get_last_err_msg()
    sync2.wait(60)
    got = np.zeros(MiB, dtype=np.uint8)
    assert h.copy_data(h.peer_rank_ptr(0, bm.BmMemType.HOST), got.ctypes.data, MiB, bm.BmCopyType.G2H, 0) == 0
    ok = bool((got[:MiB // 2] == 0x41).all() and (got[MiB // 2:] == 0x42).all())      # what ranks 1 and 2 wrote into the new slice
    sync2.wait(60)
    assert h.leave() == 0
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    return ok


def _pool_survives_leader(rank, world, url, port, sync2, sync):
    """Three ranks; the process that leads the config store dies without a word. The pool's data path keeps working and
    the control path comes back on a newly elected leader."""
    import os
    os.environ["MF_CONFIG_STORE_PORT"] = str(port)
    os.environ["MF_DEVICE_BACKEND"] = "none"
    os.environ["MF_STORE_RECOVER_MS"] = "3000"   # how long a new leader waits for the old one's members (default 60 s)
    import numpy as np
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    MiB = 1 << 20
    if rank != 0:
        sync.wait(60)                            # rank 0 goes first: it becomes the leader
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id = rank
    cfg.start_store = rank in (0, 1)             # ranks 0 and 1 may lead, rank 2 only follows
    cfg.operation_timeout = 40
    assert bm.initialize(url, world, 0, cfg) == 0, mf.get_last_err_msg()
    if rank == 0:
        sync.wait(60)
    h = bm.create2(id=0, local_dram_size=4 * MiB, max_dram_size=4 * MiB, data_op_type=bm.BmDataOpType.HOST_SHM)
    events = []
    h.set_group_event_handler(lambda r, ev: events.append((r, int(ev))))
    assert h.join() == 0, mf.get_last_err_msg()
    sync.wait(60)
    nxt = (rank + 1) % world
    src = np.full(MiB, 0x40 + rank, dtype=np.uint8)
    end = time.time() + 30
    while h.copy_data(src.ctypes.data, h.peer_rank_ptr(nxt, bm.BmMemType.HOST), MiB, bm.BmCopyType.H2G, 0) != 0:
        assert time.time() < end, mf.get_last_err_msg()
        time.sleep(0.05)
    mf.get_and_clear_last_err_msg()
    sync.wait(60)
    if rank == 0:
        os._exit(0)                              # the leader's process is gone: no leave, no goodbye to the store
    # the survivors' slices are mapped in each other: copies between them need no store
    other = 3 - rank
    got = np.zeros(MiB, dtype=np.uint8)
    assert h.copy_data(src.ctypes.data, h.peer_rank_ptr(other, bm.BmMemType.HOST) + MiB, MiB, bm.BmCopyType.H2G, 0) == 0, mf.get_last_err_msg()
    time.sleep(0.5)
    assert h.copy_data(h.peer_rank_ptr(rank, bm.BmMemType.HOST) + MiB, got.ctypes.data, MiB, bm.BmCopyType.G2H, 0) == 0
    assert (got == 0x40 + other).all()
    # the control path returns with the new leader (elected once the dead leader's address stops answering; the followers
    # notice their broken links, look the new address up in etcd and re-arm their watches); the dead rank is evicted when
    # the new leader's recovery window closes
    end = time.time() + 60
    while not any(r == 0 for r, _ in events) and time.time() < end:
        time.sleep(0.05)
    assert any(r == 0 for r, _ in events), events    # the survivors were told that rank 0 is gone
    return _after_failover(h, bm, mf, np, rank, sync2, events)


def _after_failover(h, bm, mf, np, rank, sync2, events):
    MiB = 1 << 20
    rc = 0
    if sync2 is not None:
        # a new rank 0 joins: it found this rank's exchange record in the new leader's store
        seen = len(events)
        end = time.time() + 60
        while not any(r == 0 for r, _ in events[seen:]) and time.time() < end:   # the JOIN of the returning rank
            time.sleep(0.05)
        assert any(r == 0 for r, _ in events[seen:]), events
        sync2.wait(60)
        half = np.full(MiB // 2, 0x40 + rank, dtype=np.uint8)
        assert h.copy_data(half.ctypes.data, h.peer_rank_ptr(0, bm.BmMemType.HOST) + (rank - 1) * (MiB // 2), MiB // 2, bm.BmCopyType.H2G, 0) == 0, mf.get_last_err_msg()
        sync2.wait(60)
        got = np.zeros(MiB, dtype=np.uint8)
        assert h.copy_data(h.peer_rank_ptr(rank, bm.BmMemType.HOST) + 2 * MiB, got.ctypes.data, MiB, bm.BmCopyType.G2H, 0) == 0
        assert (got == 0x70).all()
        sync2.wait(60)
        time.sleep(1.5)                          # the returned rank leaves first
    # leaving is a membership change agreed through the store
    end = time.time() + 60
    rc = -1
    while time.time() < end:
        rc = h.leave()
        if rc == 0:
            break
        mf.get_and_clear_last_err_msg()
        time.sleep(0.5)
    assert rc == 0, f"leave after the leader died: {rc} {mf.get_last_err_msg()}"
    time.sleep(1.0 if rank == 1 else 0.0)        # whoever leads now stays until the other has left
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    return True


def test_pool_survives_the_death_of_the_store_leader(etcd):
    """Four processes, an election, lease and recovery timers: on a loaded machine a step can miss its window once in a
    while, so the scenario gets a second go (a fresh instance name and port) before it counts as failed."""
    try:
        _failover_scenario(etcd, "failover")
    except AssertionError:
        _failover_scenario(etcd, "failover2")


def _failover_scenario(etcd, instance):
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    url = f"etcd://127.0.0.1:{etcd.port}#{instance}"
    port = free_port()
    sync = ctx.Barrier(3)
    q = ctx.Queue()

    def child(rank):
        pass
    from mp_util import _child
    sync2 = ctx.Barrier(3)                      # the two survivors and the process that returns as rank 0
    procs = [ctx.Process(target=_child, args=(_pool_survives_leader, r, 3, (url, port, sync2 if r else None), q, {}, sync)) for r in range(3)]
    [p.start() for p in procs]
    procs[0].join(90)                           # the first leader's process has exited ...
    time.sleep(7.0)                             # ... a new leader is elected and its recovery window (3 s) has closed
    back = ctx.Process(target=_child, args=(_rank0_returns, 0, 3, (url, port, sync2), q, {}, None))
    back.start()
    key = b"/memfabric_hybrid/config_store/clusters/" + instance.encode() + b"/memfabric_hybrid/config_store/meta/leader"
    first = None
    end = time.time() + 120
    results = {}
    while len(results) < 3 and time.time() < end:
        if first is None and key in etcd.kv:
            first = etcd.kv[key]["value"]
        try:
            r, st, val = q.get(timeout=0.5)
            results[r] = (st, val)
        except Exception:  # noqa: BLE001  (queue empty)
            pass
    for p in procs + [back]:
        p.join(10)
        if p.is_alive():
            p.kill()
    assert results.get(1) == ("ok", True) and results.get(2) == ("ok", True) and results.get(0) == ("ok", True), results
    assert procs[0].exitcode == 0 and first is not None
