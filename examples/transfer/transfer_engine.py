"""PD-style transfer: a Decode process registers a buffer, a Prefill process writes into it and reads it back
(examples/transfer/test_transfer_engine.py of the reference). Host buffers here, so it runs without a GPU; with
CUDA tensors' ``data_ptr()`` the same calls move HBM over NVLink.

    python examples/transfer/transfer_engine.py
"""
import os
import sys
import tempfile
import time

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import _launch  # noqa: E402

N = 4 << 20


def main(rank: int, world: int, session: str, tmp: str) -> str:
    from memfabric_hybrid import TransferEngine
    eng = TransferEngine()
    addr_file, done_file = os.path.join(tmp, "addr"), os.path.join(tmp, "done")
    if rank == 0:                                                   # Decode: owns the store and the destination
        assert eng.initialize(f"tcp://{session}", session, "Decode", 0) == 0
        buf = np.zeros(N, dtype=np.uint8)
        assert eng.register_memory(buf.ctypes.data, N) == 0
        open(addr_file, "w").write(str(buf.ctypes.data))
        while not os.path.exists(done_file):
            time.sleep(0.02)
        ok = bool((buf == 0x5A).all())
    else:                                                           # Prefill: pushes its KV bytes
        me = f"127.0.0.1:{_launch.free_port()}"
        assert eng.initialize(f"tcp://{session}", me, "Prefill", 0) == 0
        src = np.full(N, 0x5A, dtype=np.uint8)
        assert eng.register_memory(src.ctypes.data, N) == 0
        while not os.path.exists(addr_file) or not open(addr_file).read():
            time.sleep(0.02)
        peer = int(open(addr_file).read())
        assert eng.transfer_sync_write(session, src.ctypes.data, peer, N) == 0
        check = np.zeros(64, dtype=np.uint8)
        assert eng.register_memory(check.ctypes.data, 64) == 0
        assert eng.transfer_sync_read(session, check.ctypes.data, peer + 1000, 64) == 0
        ok = bool((check == 0x5A).all())
        open(done_file, "w").write("1")
        time.sleep(0.2)
    eng.destroy()
    eng.unInitialize()
    return "ok" if ok else "mismatch"


if __name__ == "__main__":
    with tempfile.TemporaryDirectory() as d:
        res = _launch.run(main, 2, f"127.0.0.1:{_launch.free_port()}", d)
    print(res)
    sys.exit(0 if all(r == "ok" for r in res) else 1)
