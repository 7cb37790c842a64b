"""The TCP config store: every operation of the protocol, blocking reads, watches, automatic ranks,
link-down notification, and a client that survives a server restart."""
import os
import threading
import time

import pytest


import hooks as H  # noqa: E402
from conftest import free_port  # noqa: E402


@pytest.fixture()
def server():
    port = free_port()
    h = H.start_server(port, world=4)
    yield port, h
    H.lib().mf_t_server_stop(h)


def test_every_operation(server):
    port, srv = server
    a, b = H.Store.connect(port, rank=0), H.Store.connect(port, rank=1)
    assert a.connected() and a.set("k", b"v1") == 0 and b.get("k") == b"v1"
    assert b.get("missing") == H.ERR_NOT_EXIST
    t0 = time.time()
    assert b.get("missing", timeout_ms=200) == H.ERR_TIMEOUT and time.time() - t0 >= 0.18
    # a blocking GET is released by the SET
    got = []
    th = threading.Thread(target=lambda: got.append(b.get("late", timeout_ms=5000)))
    th.start()
    time.sleep(0.1)
    a.set("late", b"here")
    th.join(5)
    assert got == [b"here"]
    # ADD creates at zero, counts in decimal text; APPEND grows; WRITE patches at an offset and zero-fills
    assert a.add("n", 5) == 5 and b.add("n", -2) == 3 and a.get("n") == b"3"
    assert a.append("log", b"ab") == 2 and b.append("log", b"cde") == 5 and a.get("log") == b"abcde"
    assert a.write("blob", 4, b"XY") == 0 and a.get("blob") == b"\0\0\0\0XY"
    assert a.write("blob", 1, b"q") == 0 and a.get("blob") == b"\0q\0\0XY"
    # CAS: empty expectation = "only if absent"; a lost swap reports what is there
    assert a.cas("lock", b"", b"A") == (0, b"A")
    rc, cur = b.cas("lock", b"", b"B")
    assert rc == H.ERR_IN_USE and cur == b"A"
    assert b.cas("lock", b"A", b"B")[0] == 0 and a.get("lock") == b"B"
    # prefix listing, removal (quiet or not), key count on the server
    for i in range(3):
        a.set(f"dir/x{i}", b"1")
    assert sorted(b.keys("dir/")) == ["dir/x0", "dir/x1", "dir/x2"]
    assert a.remove("dir/x1") == 0 and a.remove("dir/x1") != 0 and a.remove("dir/x1", quiet=True) == 0
    assert sorted(b.keys("dir/")) == ["dir/x0", "dir/x2"]
    assert H.lib().mf_t_server_keys(srv) >= 7
    # a prefixed view scopes every key
    p = a.prefixed("ns/")
    p.set("k", b"scoped")
    assert a.get("ns/k") == b"scoped" and p.get("k") == b"scoped" and p.keys("") == ["k"]
    p.close()
    a.close()
    b.close()


def test_watch_and_unwatch(server):
    port, _ = server
    a, b = H.Store.connect(port, rank=0), H.Store.connect(port, rank=1)
    seen, ev = [], threading.Event()

    def on(rc, key, val):
        seen.append((rc, key, val))
        ev.set()
    a.set("cfg", b"1")
    wid = b.watch("cfg", on)
    assert ev.wait(2) and seen[-1] == (0, "cfg", b"1")        # an existing key reports at once
    ev.clear()
    a.set("cfg", b"2")
    assert ev.wait(2) and seen[-1] == (0, "cfg", b"2")
    ev.clear()
    assert b.unwatch(wid) == 0
    a.set("cfg", b"3")
    assert not ev.wait(0.3)
    a.close()
    b.close()


def test_auto_rank_and_link_down(server):
    port, _ = server
    cs = [H.Store.connect(port, rank=0xFFFFFFFF) for _ in range(3)]
    ranks = [c.auto_rank() for c in cs]
    assert all(rc == 0 for rc, _ in ranks) and sorted(r for _, r in ranks) == [0, 1, 2]
    watcher = cs[0]
    down, ev = [], threading.Event()
    watcher.watch_rank(lambda r: (down.append(r), ev.set()))
    victim = cs[2]
    vr = ranks[2][1]
    assert watcher.alive(vr)
    H.lib().mf_t_client_set_reconnect(victim.h, 0, 10)
    H.lib().mf_t_client_crash(victim.h)                        # socket closed without a goodbye
    assert ev.wait(5) and down == [vr]
    assert not watcher.alive(vr)
    # the freed rank is handed to the next newcomer
    late = H.Store.connect(port, rank=0xFFFFFFFF)
    assert late.auto_rank() == (0, vr)
    for c in cs + [late]:
        c.close()


def test_client_reconnects_after_server_restart():
    port = free_port()
    srv = H.start_server(port, world=2)
    H.lib().mf_t_server_set_backend(srv, b"restart-test", 1)
    c = H.Store.connect(port, world=2, rank=0)
    H.lib().mf_t_client_set_reconnect(c.h, 50, 100)
    c.set("before", b"x")
    H.lib().mf_t_server_stop(srv)
    time.sleep(0.3)
    assert not c.connected()
    srv = H.start_server(port, world=2)
    H.lib().mf_t_server_set_backend(srv, b"restart-test", 0)
    deadline = time.time() + 10
    while not c.connected() and time.time() < deadline:
        time.sleep(0.05)
    assert c.connected()
    # keys are not persisted (only membership is); the client works again on the new server
    assert c.get("before") == H.ERR_NOT_EXIST and c.set("after", b"y") == 0 and c.get("after") == b"y"
    c.close()
    H.lib().mf_t_server_stop(srv)
    H.lib().mf_t_backend_reset(b"restart-test")
