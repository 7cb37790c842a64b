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
