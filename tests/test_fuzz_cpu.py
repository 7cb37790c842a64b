"""Malformed input at the places where bytes arrive from outside the process: frames sent to the config-store server,
replies sent to a store client, exchange blobs handed to the memory layer, configuration strings. The byte streams of a
real client / server conversation are recorded through a forwarding proxy and replayed with mutations (bit flips,
truncation, inflated length fields, splices, noise). Whatever arrives, the process must neither crash nor hang, and the
service must keep working for well-behaved peers. The sanitizer tier runs this file against the ASAN + UBSAN build.
Seeds are fixed: a failure reproduces."""
import ctypes as C
import os
import random
import socket
import threading
import time

import hooks as H  # noqa: E402
from conftest import free_port  # noqa: E402

SEED = int(os.environ.get("MF_FUZZ_SEED", "0"))   # other values explore other mutations
LIGHT = 4 if os.environ.get("MF_FUZZ_LIGHT") else 1   # the ThreadSanitizer tier runs a quarter of the rounds (it is 10 x slower)


class RecordingProxy:
    """Forwards one connection at a time to ``target`` and keeps what each side sent."""

    def __init__(self, target):
        self.target = target
        self.up, self.down = [], []          # client -> server chunks, server -> client chunks
        self.lsock = socket.socket()
        self.lsock.bind(("127.0.0.1", 0))
        self.lsock.listen(8)
        self.port = self.lsock.getsockname()[1]
        self.run = True
        self.t = threading.Thread(target=self._accept, daemon=True)
        self.t.start()

    def _accept(self):
        while self.run:
            try:
                c, _ = self.lsock.accept()
            except OSError:
                return
            s = socket.create_connection(("127.0.0.1", self.target))
            threading.Thread(target=self._pump, args=(c, s, self.up), daemon=True).start()
            threading.Thread(target=self._pump, args=(s, c, self.down), daemon=True).start()

    @staticmethod
    def _pump(a, b, log):
        try:
            while True:
                d = a.recv(65536)
                if not d:
                    break
                log.append(d)
                b.sendall(d)
        except OSError:
            pass
        for s in (a, b):
            try:
                s.shutdown(socket.SHUT_RDWR)
            except OSError:
                pass

    def close(self):
        self.run = False
        self.lsock.close()


def _mutate(rng: random.Random, data: bytes) -> bytes:
    b = bytearray(data)
    kind = rng.randrange(8)
    if kind == 0 and b:                                   # bit flips
        for _ in range(rng.randint(1, 8)):
            i = rng.randrange(len(b))
            b[i] ^= 1 << rng.randrange(8)
    elif kind == 1 and b:                                 # truncation
        del b[rng.randrange(len(b)):]
    elif kind == 2 and len(b) >= 4:                       # a 32-bit field becomes huge / negative / zero
        i = rng.randrange(len(b) - 3)
        b[i:i + 4] = rng.choice([b"\xff\xff\xff\xff", b"\xff\xff\xff\x7f", b"\x00\x00\x00\x80", b"\x00\x00\x00\x00", b"\x00\x00\x01\x00"])
    elif kind == 3 and len(b) >= 8:                       # a 64-bit field
        i = rng.randrange(len(b) - 7)
        b[i:i + 8] = rng.choice([b"\xff" * 8, b"\xff" * 7 + b"\x7f", b"\x00" * 8])
    elif kind == 4 and b:                                 # a stretch repeated
        i = rng.randrange(len(b))
        j = min(len(b), i + rng.randint(1, 64))
        b[i:i] = b[i:j] * rng.randint(1, 4)
    elif kind == 5:                                       # noise in the middle
        i = rng.randrange(len(b) + 1)
        b[i:i] = bytes(rng.getrandbits(8) for _ in range(rng.randint(1, 128)))
    elif kind == 6:                                       # noise only
        b = bytearray(rng.getrandbits(8) for _ in range(rng.randint(1, 512)))
    elif kind == 7 and len(b) > 16:                       # the head kept (handshake), the tail scrambled
        cut = rng.randrange(8, len(b))
        tail = list(b[cut:])
        rng.shuffle(tail)
        b[cut:] = bytes(tail)
    return bytes(b)


def _record_conversation():
    port = free_port()
    srv = H.start_server(port, world=4)
    proxy = RecordingProxy(port)
    st = H.Store.connect(proxy.port, world=4, rank=1)
    assert st.set("fz/a", b"value-a") == 0 and st.get("fz/a") == b"value-a"
    assert st.add("fz/n", 5) == 5
    st.append("fz/l", b"one")
    st.cas("fz/c", b"", b"first")
    st.write("fz/w", 4, b"abcd")
    st.keys("fz/")
    st.get("fz/missing", timeout_ms=50)
    st.remove("fz/a")
    st.close()
    time.sleep(0.2)
    proxy.close()
    return port, srv, b"".join(proxy.up), b"".join(proxy.down)


def test_store_server_survives_malformed_frames():
    port, srv, up, _ = _record_conversation()
    assert len(up) > 100
    rng = random.Random(20240611 + SEED)
    try:
        for i in range(400 // LIGHT):
            payload = _mutate(rng, up)
            if rng.random() < 0.3:
                payload = _mutate(rng, payload)
            s = socket.socket()
            s.settimeout(0.5)
            try:
                s.connect(("127.0.0.1", port))
                s.sendall(payload)
                if rng.random() < 0.5:
                    try:
                        s.recv(4096)
                    except OSError:
                        pass
            except OSError:
                pass
            finally:
                s.close()
            if i % 50 == 49:      # the service is intact for a well-behaved client in between
                st = H.Store.connect(port, world=4, rank=2)
                assert st.set(f"ok/{i}", b"v") == 0 and st.get(f"ok/{i}") == b"v"
                st.close()
        st = H.Store.connect(port, world=4, rank=3)
        assert st.set("after", b"fuzz") == 0 and st.get("after") == b"fuzz"
        assert H.lib().mf_t_server_keys(srv) < 10_000          # garbage did not turn into a flood of keys
        st.close()
    finally:
        H.lib().mf_t_server_stop(srv)


def test_store_client_survives_malformed_replies():
    port, srv, _, down = _record_conversation()
    H.lib().mf_t_server_stop(srv)
    assert len(down) > 50
    rng = random.Random(77 + SEED)
    lsock = socket.socket()
    lsock.bind(("127.0.0.1", 0))
    lsock.listen(16)
    fport = lsock.getsockname()[1]
    state = {"payload": b"", "run": True}

    def serve():
        while state["run"]:
            try:
                c, _ = lsock.accept()
            except OSError:
                return
            try:
                c.settimeout(0.3)
                try:
                    c.recv(4096)                      # the client's handshake
                except OSError:
                    pass
                c.sendall(state["payload"])
                time.sleep(0.05)
            except OSError:
                pass
            finally:
                c.close()
    threading.Thread(target=serve, daemon=True).start()
    try:
        for i in range(120 // LIGHT):
            state["payload"] = down if i == 0 else _mutate(rng, down)
            t0 = time.monotonic()
            try:
                st = H.Store.connect(fport, world=4, rank=1, timeout_ms=400)
            except ConnectionError:
                assert time.monotonic() - t0 < 5.0
                continue
            # the handshake passed: requests meet whatever follows in the stream, then a closed link
            st.get("fz/a", timeout_ms=100)
            st.set("x", b"y")
            st.close()
            assert time.monotonic() - t0 < 8.0
        # a link that breaks at the very moment its owner lets go of the client (the worker thread starts a redial while
        # the caller shuts down): many quick rounds of "handshake answered, connection dropped, client closed at once"
        state["payload"] = down
        for i in range(60 // LIGHT):
            try:
                st = H.Store.connect(fport, world=4, rank=1, timeout_ms=400)
            except ConnectionError:
                continue
            if i % 3 == 0:
                time.sleep(0.001 * (i % 7))
            st.close()
    finally:
        state["run"] = False
        lsock.close()


def test_parsers_refuse_garbage_without_crashing(tmp_path):
    """Store URLs, TLS settings, fail-point files and the etcd gateway's replies."""
    from memfabric_hybrid_b200 import api
    from fake_etcd import FakeEtcd
    rng = random.Random(5 + SEED)
    alphabet = "tcpetdrg:/#.0123456789[]-_@ ;,=\\\x00\xff"
    for _ in range(300):
        url = "".join(rng.choice(alphabet) for _ in range(rng.randint(0, 40)))
        if rng.random() < 0.5:
            url = rng.choice(["tcp://", "etcd://", "reg://"]) + url
        if url.startswith("tcp://127.0.0.1:") or url.startswith("reg://"):
            continue                                     # could be a valid address: would start a server
        rc = api.create_config_store(url.replace("\x00", ""))
        assert rc != 0 or url == "", url
    api.get_and_clear_last_err_msg()
    keys = ["tlsCaPath", "tlsCaFile", "tlsCert", "tlsPk", "tlsPkPwd", "tlsCrlPath", "tlsCrlFile", "packagePath", "decrypterLibPath", "bogus"]
    for _ in range(200):
        parts = []
        for _ in range(rng.randint(0, 6)):
            parts.append(rng.choice(keys) + rng.choice([":", "=", " : ", ""]) + "".join(rng.choice("/ab.,;: \t") for _ in range(rng.randint(0, 12))))
        info = rng.choice([";", "; ", "\n", ";;"]).join(parts).encode()
        api.set_conf_store_tls(True, info.decode())     # accepted or refused, never a crash
    api.set_conf_store_tls(False, "")
    # fail-point configuration
    l = H.lib()
    conf = tmp_path / "fp.conf"
    for i in range(40):
        lines = []
        for _ in range(rng.randint(0, 8)):
            lines.append(" ".join("".join(rng.choice("ABC_abc019-+. \t#") for _ in range(rng.randint(0, 12))) for _ in range(rng.randint(0, 5))))
        conf.write_text("\n".join(lines))
        l.mf_t_fip_init(str(conf).encode())
        l.mf_t_fip_reload()
        l.mf_t_fip_exit()
    # an etcd that answers nonsense
    f = FakeEtcd()
    try:
        replies = [b"", b"{", b"[]", b"null", b'{"kvs":17}', b'{"kvs":[{"value":"!!!not base64"}]}', b'{"kvs":[[]]}', b'{"ID":"x"}',
                   b'{"kvs":[{"key":"' + b"A" * 70000 + b'"}]}', b"{" * 200, b'{"a":' * 100 + b"1" + b"}" * 100, b'"\\u12"', b'{"succeeded":"yes"}',
                   bytes(rng.getrandbits(8) for _ in range(300))]
        orig = f._handle
        box = {"i": 0}

        class Raw(dict):
            pass
        import json as _json
        real_dumps = _json.dumps

        def fake_handle(op, body):
            return 200, Raw(raw=replies[box["i"] % len(replies)])
        f._handle = fake_handle
        import fake_etcd as FE
        FE.json.dumps = lambda obj, *a, **k: obj["raw"].decode("latin-1") if isinstance(obj, Raw) else real_dumps(obj, *a, **k)
        try:
            h = l.mf_t_etcd_new(b"127.0.0.1", f.port, b"fz", None, None, 500)
            buf = C.create_string_buffer(1 << 17)
            for i in range(len(replies)):
                box["i"] = i
                l.mf_t_etcd_get(h, b"/k", buf, len(buf))
                l.mf_t_etcd_prefix_get(h, b"/", buf, len(buf))
                l.mf_t_etcd_put(h, b"/k", b"v", 1, 1000)
                assert l.mf_t_etcd_try_lock(h, b"lk") != 0 or l.mf_t_etcd_unlock(h, b"lk") in (0, -1)
            l.mf_t_etcd_free(h)
        finally:
            FE.json.dumps = real_dumps
            f._handle = orig
    finally:
        f.close()


def _exchange_records(rank, world):
    """Runs in a child process (host-memory backend): the records of a rank that is gone, then damaged copies of them."""
    l = H.lib()
    MiB = 1 << 20
    rs = l.mf_t_ex_record_size()
    import os
    warm = l.mf_t_ex_new(21, 1, 2, 64 * MiB, 2 * MiB)     # first use starts the descriptor channel's listener
    assert warm
    l.mf_t_ex_free(warm)
    fds = len(os.listdir("/proc/self/fd"))
    for _ in range(5):                                     # a pool that goes away takes its memory file with it
        h = l.mf_t_ex_new(21, 1, 2, 64 * MiB, 2 * MiB)
        assert h
        l.mf_t_ex_free(h)
    assert len(os.listdir("/proc/self/fd")) == fds
    peer = l.mf_t_ex_new(21, 1, 2, 64 * MiB, 2 * MiB)
    assert peer
    buf = C.create_string_buffer(2 * rs)
    assert l.mf_t_ex_export(peer, buf) == 2
    good = buf.raw
    l.mf_t_ex_free(peer)                                  # its memory file is gone with it: mapping it can only fail
    me = l.mf_t_ex_new(21, 0, 2, 64 * MiB, 2 * MiB)
    assert me
    try:
        assert l.mf_t_ex_import(me, good, 2, 0) == 0      # well-formed records are accepted ...
        assert l.mf_t_ex_import(me, good, 2, 1) != 0      # ... and mapping the vanished peer fails cleanly
        assert l.mf_t_ex_mapped_bytes(me, 1) == 0 and l.mf_t_ex_mapped_bytes(me, 0) == 2 * MiB
        rng = random.Random(99 + SEED)
        used = C.c_uint32.from_buffer_copy(good[rs - 4:rs]).value      # descLen of the first record
        assert 0 < used <= rs - 4
        # every 64-bit field of the slice record pushed to extremes (offsets and sizes that wrap when added among them)
        slice_rec = good[rs:]
        for pos in range(0, 160, 4):
            for val in (b"\xff" * 8, b"\x00\xf0\xff\xff\xff\xff\xff\xff", b"\x00" * 7 + b"\x80", b"\x01" + b"\x00" * 7):
                rec = slice_rec[:pos] + val + slice_rec[pos + 8:]
                l.mf_t_ex_import(me, good[:rs] + rec, 2, 1)
                assert l.mf_t_ex_mapped_bytes(me, 1) == 0
        for i in range(600):
            recs = bytearray(good)
            for _ in range(rng.randint(1, 6)):
                k = rng.randrange(4)
                at = rng.randrange(rs) + rng.choice([0, rs])
                if k == 0:
                    recs[at] ^= 1 << rng.randrange(8)
                elif k == 1:
                    recs[at:at + 4] = rng.choice([b"\xff\xff\xff\xff", b"\x00\x00\x00\x00", b"\xff\xff\xff\x7f"])[:len(recs) - at]
                elif k == 2:
                    recs[at] = rng.getrandbits(8)
                else:
                    which = rng.choice([0, rs])
                    recs[which + rs - 4:which + rs] = rng.choice([b"\xff\xff\xff\xff", b"\x00\x05\x00\x00", b"\x01\x00\x00\x00", b"\x00\x00\x00\x00"])
            l.mf_t_ex_import(me, bytes(recs[:2 * rs]), 2, rng.randrange(2))
            assert l.mf_t_ex_mapped_bytes(me, 1) <= 64 * MiB and l.mf_t_ex_mapped_bytes(me, 0) == 2 * MiB
        assert l.mf_t_ex_import(me, good, 2, 0) == 0      # still in working order
    finally:
        l.mf_t_ex_free(me)
    return True


def test_memory_layer_refuses_damaged_exchange_records():
    from mp_util import run_ranks
    assert run_ranks(_exchange_records, 1, (), timeout=240, env={"MF_DEVICE_BACKEND": "none"}) == [True]


def test_group_engine_survives_damaged_membership_records():
    """Members of a dynamic group watch the membership record in the store; a rogue client overwrites it with damaged
    copies (wrong sizes, rank numbers far outside a group, flipped bits). Nobody may crash or stall."""
    l = H.lib()
    port = free_port()
    srv = H.start_server(port, world=8)
    rng = random.Random(4242 + SEED)
    n = 2
    stores, groups, cbs, events = [None] * n, [None] * n, [None] * n, []
    try:
        for r in range(n):
            stores[r] = H.Store.connect(port, world=8, rank=r)
            cbs[r] = H.CHANGE_CB(lambda ev, who: (events.append((ev, who)), 0)[1])
            groups[r] = l.mf_t_group_new(stores[r].h, n, r, 3000, 1, cbs[r])
            assert l.mf_t_group_start_listen(groups[r]) == 0
            assert l.mf_t_group_join(groups[r]) == 0
        rogue = H.Store.connect(port, world=8, rank=5)
        good = rogue.get("EVENT")
        assert isinstance(good, bytes) and len(good) >= 20
        for i in range(200 // LIGHT):
            rec = bytearray(good)
            k = rng.randrange(5)
            if k == 0:
                for _ in range(rng.randint(1, 6)):
                    rec[rng.randrange(len(rec))] ^= 1 << rng.randrange(8)
            elif k == 1:
                rec = rec[:rng.randrange(len(rec))]
            elif k == 2:
                rec += bytes(rng.getrandbits(8) for _ in range(rng.randint(1, 64)))
            elif k == 3:                                   # version moves on, event and ranks are nonsense
                rec[0:4] = (int.from_bytes(good[0:4], "little") + 2 * i + 1).to_bytes(4, "little")
                rec[8:20] = bytes(rng.getrandbits(8) for _ in range(12))
            else:
                rec[12:16] = b"\\xff\\xff\\xff\\xff"
                rec[16:20] = b"\\xff\\xff\\xff\\x7f"
                rec[0:4] = (int.from_bytes(good[0:4], "little") + 2 * i + 1).to_bytes(4, "little")
            assert rogue.set("EVENT", bytes(rec)) == 0
            if i % 10 == 0:
                time.sleep(0.01)
        time.sleep(0.3)
        v, s, e, b = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint64()
        for g in groups:
            l.mf_t_group_info(g, C.byref(v), C.byref(s), C.byref(e), C.byref(b))      # still answers
        rogue.set("EVENT", good)
        rogue.close()
    finally:
        for g in groups:
            if g:
                l.mf_t_group_free(g)
        for st in stores:
            if st:
                st.close()
        l.mf_t_server_stop(srv)
