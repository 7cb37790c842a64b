"""PD-style transfer between two processes without a GPU: host buffers registered on both sides, the
Prefill side writes into and reads from the Decode side's memory (the engine moves the bytes with
process_vm_writev/readv when no device is present), and learns when its peer goes away."""
import ctypes as C
import os
import threading
import time

import numpy as np

from conftest import free_port
from mp_util import run_ranks

N_BYTES = 1 << 20


def _decode(session, tmp, sync):
    from memfabric_hybrid_b200.api import TransferEngine
    eng = TransferEngine()
    assert eng.initialize(f"tcp://{session}", session, "Decode", 0) == 0
    buf = np.zeros(N_BYTES, dtype=np.uint8)
    assert eng.register_memory(buf.ctypes.data, N_BYTES) == 0
    with open(os.path.join(tmp, "addr"), "w") as f:
        f.write(str(buf.ctypes.data))
    sync.wait(60)      # address published
    sync.wait(60)      # prefill wrote
    exp = (np.arange(N_BYTES) % 251).astype(np.uint8)
    ok = bool((buf == exp).all())
    buf[:16] = 7       # something for the peer to read back
    sync.wait(60)
    sync.wait(60)      # prefill read
    eng.destroy()
    eng.unInitialize()
    return ok


def _prefill(session, tmp, sync):
    from memfabric_hybrid_b200.api import TransferEngine
    eng = TransferEngine()
    mine = f"127.0.0.1:{free_port()}"
    assert eng.initialize(f"tcp://{session}", mine, "Prefill", 0) == 0
    down, ev = [], threading.Event()
    eng.set_peer_down_callback(lambda uid: (down.append(uid), ev.set()))
    src = (np.arange(N_BYTES) % 251).astype(np.uint8)
    assert eng.register_memory(src.ctypes.data, N_BYTES) == 0
    sync.wait(60)
    peer = int(open(os.path.join(tmp, "addr")).read())
    half = N_BYTES // 2
    assert eng.transfer_sync_write(session, src.ctypes.data, peer, half) == 0
    # the second half as a batch of four pieces
    q = half // 4
    assert eng.batch_transfer_sync_write(session, [src.ctypes.data + half + i * q for i in range(4)],
                                         [peer + half + i * q for i in range(4)], [q] * 4) == 0
    # outside the registered range: refused
    assert eng.transfer_sync_write(session, src.ctypes.data, peer + N_BYTES - 8, 64) != 0
    sync.wait(60)
    sync.wait(60)
    back = np.zeros(32, dtype=np.uint8)
    assert eng.register_memory(back.ctypes.data, 32) == 0
    assert eng.transfer_sync_read(session, back.ctypes.data, peer, 32) == 0
    ok = bool((back[:16] == 7).all()) and bool((back[16:] == src[16:32]).all())
    sync.wait(60)
    got_down = ev.wait(15)          # the Decode side tears down after the last barrier
    eng.destroy()
    eng.unInitialize()
    return ok and got_down and len(down) == 1


def _role(rank, world, session, tmp, sync):
    os.environ["MF_DEVICE_BACKEND"] = "none"
    return _decode(session, tmp, sync) if rank == 0 else _prefill(session, tmp, sync)


def test_prefill_writes_into_decode(tmp_path):
    session = f"127.0.0.1:{free_port()}"
    assert run_ranks(_role, 2, (session, str(tmp_path)), timeout=120, with_barrier=True) == [True, True]


def _decode_external(session_store, tmp):
    """Decode side against a store that somebody else hosts; stays until told to go."""
    os.environ["MF_DEVICE_BACKEND"] = "none"
    from memfabric_hybrid_b200.api import TransferEngine
    eng = TransferEngine()
    me = f"127.0.0.1:{free_port()}"
    assert eng.initialize(f"tcp://{session_store}", me, "Decode", 0, store_server_role=None) == 0
    buf = np.zeros(4096, dtype=np.uint8)
    assert eng.register_memory(buf.ctypes.data, 4096) == 0
    with open(os.path.join(tmp, "addr"), "w") as f:
        f.write(f"{me} {buf.ctypes.data}")
    end = time.time() + 90
    while not os.path.exists(os.path.join(tmp, "done")) and time.time() < end:
        time.sleep(0.05)
    ok = bool((buf == 0x6B).all())
    eng.destroy()
    eng.unInitialize()
    return ok


def _prefill_external(session_store, tmp):
    os.environ["MF_DEVICE_BACKEND"] = "none"
    from memfabric_hybrid_b200.api import TransferEngine
    eng = TransferEngine()
    assert eng.initialize(f"tcp://{session_store}", f"127.0.0.1:{free_port()}", "Prefill", 0, store_server_role=None) == 0
    peer_id, peer_addr = open(os.path.join(tmp, "addr")).read().split()
    src = np.full(4096, 0x6B, dtype=np.uint8)
    assert eng.register_memory(src.ctypes.data, 4096) == 0
    rc = eng.transfer_sync_write(peer_id, src.ctypes.data, int(peer_addr), 4096)
    eng.destroy()
    eng.unInitialize()
    return rc


def test_endpoint_is_found_again_after_the_store_restarted(tmp_path):
    """The store's server goes away and comes back empty while a Decode endpoint is up. The endpoint reconnects and puts
    its identity and buffer records back, so a Prefill process that starts afterwards still finds and reaches it."""
    import multiprocessing as mp
    import hooks as H
    ctx = mp.get_context("spawn")
    port = free_port()
    srv = H.start_server(port, world=512)
    store = f"127.0.0.1:{port}"
    q = ctx.Queue()
    from mp_util import _child
    dec = ctx.Process(target=_child, args=(_decode_wrapper, 0, 1, (store, str(tmp_path)), q, {}, None))
    dec.start()
    try:
        end = time.time() + 60
        while not os.path.exists(tmp_path / "addr") and time.time() < end:
            time.sleep(0.05)
        assert os.path.exists(tmp_path / "addr")
        H.lib().mf_t_server_stop(srv)                    # every key is gone with it
        time.sleep(0.5)
        srv = H.start_server(port, world=512)
        time.sleep(3.0)                                   # the endpoint's client re-dials once a second
        pre = ctx.Process(target=_child, args=(_prefill_wrapper, 1, 1, (store, str(tmp_path)), q, {}, None))
        pre.start()
        results = {}
        end = time.time() + 90
        while 1 not in results and time.time() < end:
            try:
                r, st, val = q.get(timeout=0.5)
                results[r] = (st, val)
            except Exception:  # noqa: BLE001
                pass
        (tmp_path / "done").write_text("1")
        while 0 not in results and time.time() < end:
            try:
                r, st, val = q.get(timeout=0.5)
                results[r] = (st, val)
            except Exception:  # noqa: BLE001
                pass
        for p in (dec, pre):
            p.join(10)
        assert results.get(1) == ("ok", 0), results
        assert results.get(0) == ("ok", True), results
    finally:
        for p in (dec,):
            if p.is_alive():
                p.kill()
        H.lib().mf_t_server_stop(srv)


def _decode_wrapper(rank, world, store, tmp):
    return _decode_external(store, tmp)


def _prefill_wrapper(rank, world, store, tmp):
    return _prefill_external(store, tmp)
