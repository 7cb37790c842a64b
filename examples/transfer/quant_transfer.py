"""PD-style transfer with quantisation on the way: the Prefill process holds bf16 KV rows in HBM and writes them into
the Decode process's HBM as int8 plus one fp32 dequantisation factor per unit of 512 elements, in ONE call
(``batch_transfer_write_with_quant``; the kernel quantises while it pushes over NVLink). Needs a GPU; with one GPU
both processes share it. Counterpart of examples/transfer/test_quant_trans.py of the reference.

    python examples/transfer/quant_transfer.py
"""
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import _launch  # noqa: E402

ROWS, UNITS, UNIT = 32, 16, 512


def _wait_for(path):
    while not os.path.exists(path) or not open(path).read():
        time.sleep(0.02)
    return open(path).read()


def main(rank: int, world: int, session: str, tmp: str) -> str:
    import torch
    from memfabric_hybrid import TransferEngine
    dev = rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    eng = TransferEngine()
    x = (torch.randn(ROWS, UNITS * UNIT, device="cuda", generator=torch.Generator("cuda").manual_seed(7)) * 2).to(torch.bfloat16)
    addr, done = os.path.join(tmp, "addr"), os.path.join(tmp, "done")
    if rank == 0:                                                    # Decode: owns the store and the destination
        assert eng.initialize(f"tcp://{session}", session, "Decode", dev) == 0
        q = torch.zeros(ROWS, UNITS * UNIT, dtype=torch.int8, device="cuda")
        factor = torch.zeros(ROWS, UNITS, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()                                     # registered buffers must be complete first
        assert eng.register_memory(q.data_ptr(), q.numel()) == 0
        assert eng.register_memory(factor.data_ptr(), factor.numel() * 4) == 0
        open(addr, "w").write(f"{q.data_ptr()} {factor.data_ptr()}")
        _wait_for(done)
        torch.cuda.synchronize()
        back = q.view(ROWS, UNITS, UNIT).float() * factor[..., None]  # dequantise and compare with what was sent
        err = float((back - x.float().view(ROWS, UNITS, UNIT)).abs().max())
        ok = err <= float(x.float().abs().max()) / 127.0
        print(f"decode: max abs error after dequantisation {err:.4f}")
    else:                                                            # Prefill: quantise-and-push
        assert eng.initialize(f"tcp://{session}", f"127.0.0.1:{_launch.free_port()}", "Prefill", dev) == 0
        torch.cuda.synchronize()
        assert eng.register_memory(x.data_ptr(), x.numel() * 2) == 0
        q_ptr, f_ptr = (int(v) for v in _wait_for(addr).split())
        row = UNITS * UNIT
        rc = eng.batch_transfer_write_with_quant(session, [x[i].data_ptr() for i in range(ROWS)], [q_ptr + i * row for i in range(ROWS)],
                                                 [row * 2] * ROWS, [f_ptr + i * UNITS * 4 for i in range(ROWS)], None, UNIT)
        ok = rc == 0
        open(done, "w").write("1")
        time.sleep(0.5)
    eng.destroy()
    eng.unInitialize()
    return "ok" if ok else "mismatch"


if __name__ == "__main__":
    with tempfile.TemporaryDirectory() as d:
        res = _launch.run(main, 2, f"127.0.0.1:{_launch.free_port()}", d)
    print(res)
    sys.exit(0 if all(r == "ok" for r in res) else 1)
