"""PD-style transfer of HBM buffers between two processes: plain write / read of registered CUDA buffers, and the
quantising write (bf16 -> int8 per unit with its fp32 dequantisation factor) against a PyTorch restatement.

The two processes share one GPU when only one is visible; the copy and quantisation kernels never wait on one
another, so that is a valid test of the inter-process mapping (CUDA IPC handles of user-registered buffers)."""
import os
import time

import pytest

from conftest import free_port
from mp_util import run_ranks

pytestmark = pytest.mark.gpu
B, UNITS, UNIT = 6, 5, 512


def _wait_file(path, secs=60):
    end = time.time() + secs
    while time.time() < end:
        if os.path.exists(path) and os.path.getsize(path) > 0:
            return open(path).read()
        time.sleep(0.02)
    raise AssertionError(f"timed out waiting for {path}")


def _pd(rank, world, session, tmp, sync):
    import torch
    from memfabric_hybrid import TransferEngine
    dev = rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    eng = TransferEngine()
    g = torch.Generator("cuda").manual_seed(4242)
    x = (torch.randn(B, UNITS * UNIT, device="cuda", generator=g) * 3).to(torch.bfloat16)   # both sides draw the same data
    x[2, :UNIT] = 0                                                                          # an all-zero unit
    if rank == 0:                                                                            # Decode: the destination
        assert eng.initialize(f"tcp://{session}", session, "Decode", dev) == 0
        q = torch.zeros(B, UNITS * UNIT, dtype=torch.int8, device="cuda")
        sc = torch.zeros(B, UNITS, dtype=torch.float32, device="cuda")
        raw = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
        q8 = torch.zeros(B, UNITS * UNIT, dtype=torch.uint8, device="cuda")          # fp8 e4m3 bits, one factor per 128
        sc8 = torch.zeros(B, UNITS * UNIT // 128, dtype=torch.float32, device="cuda")
        qodd = torch.zeros(1003 + 5, dtype=torch.int8, device="cuda")                 # odd length at an odd address
        scodd = torch.zeros(2, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        for t in (q, sc, raw, q8, sc8, qodd, scodd):
            assert eng.register_memory(t.data_ptr(), t.numel() * t.element_size()) == 0
        open(os.path.join(tmp, "addr"), "w").write(" ".join(str(t.data_ptr()) for t in (q, sc, raw, q8, sc8, qodd, scodd)))
        sync.wait(45)                                                                       # the peer has written
        torch.cuda.synchronize()
        xf = x.float().view(B, UNITS, UNIT)
        amax = xf.abs().amax(-1)
        want_sc = amax / 127.0
        want_q = torch.where(amax[..., None] > 0, xf * (127.0 / amax.clamp_min(1e-30))[..., None], torch.zeros_like(xf)).round()
        assert (q.view(B, UNITS, UNIT).float() - want_q).abs().max().item() <= 1.0           # rounding of a tie may differ
        assert (q.view(B, UNITS, UNIT).float() - want_q).abs().mean().item() < 0.01
        live = amax > 0                                                                      # an all-zero unit: any finite factor will do
        torch.testing.assert_close(sc[live], want_sc[live], rtol=1e-3, atol=1e-12)
        assert bool(torch.isfinite(sc).all()) and bool((q.view(B, UNITS, UNIT)[~live] == 0).all())
        deq = q.view(B, UNITS, UNIT).float() * sc[..., None]
        assert (deq - xf).abs().max().item() <= (amax.max().item() / 127.0) * 0.51 + 1e-6
        assert bool((raw[:4096] == 0x5A).all()) and int(raw[4096]) == 0
        # fp8 e4m3, 1 x 128 factors: dequantised values within one fp8 step (2^-3 relative) of the input
        x8 = x.float().view(B, -1, 128)
        a8 = x8.abs().amax(-1)
        live8 = a8 > 0
        torch.testing.assert_close(sc8[live8], (a8 / 448.0)[live8], rtol=1e-3, atol=1e-12)
        d8 = q8.view(torch.float8_e4m3fn).float().view(B, -1, 128) * sc8[..., None]
        assert float(((d8 - x8).abs() - 0.0625 * x8.abs() - a8[..., None] * 2e-3).max()) <= 0.0
        # the odd-sized row went through the element-wise path: 1003 elements in units of 512 (512 + 491), offset 5
        xo = x.reshape(-1)[:1003].float()
        for u, (b, e) in enumerate(((0, 512), (512, 1003))):
            am = xo[b:e].abs().max()
            wq = (xo[b:e] * (127.0 / am)).round()
            assert float((qodd[5 + b:5 + e].float() - wq).abs().max()) <= 1.0
            assert abs(float(scodd[u]) - float(am) / 127.0) < 1e-6
        assert int(qodd[:5].abs().sum()) == 0
        ok = True
    else:                                                                                    # Prefill: the source
        me = f"127.0.0.1:{free_port()}"
        assert eng.initialize(f"tcp://{session}", me, "Prefill", dev) == 0
        src = torch.full((4096,), 0x5A, dtype=torch.uint8, device="cuda")
        back = torch.zeros(4096, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        for t in (x, src, back):
            assert eng.register_memory(t.data_ptr(), t.numel() * t.element_size()) == 0
        q_ptr, sc_ptr, raw_ptr, q8_ptr, sc8_ptr, qodd_ptr, scodd_ptr = (int(v) for v in _wait_file(os.path.join(tmp, "addr")).split())
        row = UNITS * UNIT
        rc = eng.batch_transfer_write_with_quant(session, [x[i].data_ptr() for i in range(B)], [q_ptr + i * row for i in range(B)],
                                                 [row * 2] * B, [sc_ptr + i * UNITS * 4 for i in range(B)], None, UNIT)
        assert rc == 0
        rc = eng.batch_transfer_write_with_quant(session, [x[i].data_ptr() for i in range(B)], [q8_ptr + i * row for i in range(B)],
                                                 [row * 2] * B, [sc8_ptr + i * (row // 128) * 4 for i in range(B)], None, 128, flags=1)
        assert rc == 0                                                              # flags=1: fp8 e4m3 output
        assert eng.batch_transfer_write_with_quant(session, [x.data_ptr()], [qodd_ptr + 5], [1003 * 2], [scodd_ptr], None, UNIT) == 0
        assert eng.transfer_sync_write(session, src.data_ptr(), raw_ptr, 4096) == 0
        assert eng.transfer_sync_read(session, back.data_ptr(), raw_ptr, 4096) == 0
        torch.cuda.synchronize()
        ok = bool((back == 0x5A).all())
        sync.wait(45)
    sync.wait(45)                                                                           # nobody tears down early
    eng.destroy()
    eng.unInitialize()
    return ok


def test_pd_transfer_of_hbm_with_quantising_write(tmp_path):
    session = f"127.0.0.1:{free_port()}"
    assert run_ranks(_pd, 2, (session, str(tmp_path)), timeout=300, with_barrier=True) == [True, True]
