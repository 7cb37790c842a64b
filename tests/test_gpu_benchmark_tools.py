"""The native benchmark tools on GPUs: all twelve BigMemory copy directions and the TRANS sweep, data verified."""
import os
import subprocess

import pytest
import torch

from conftest import free_port

pytestmark = pytest.mark.gpu
BIN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "memfabric_hybrid_b200", "bin")


def _tool(name):
    p = os.path.join(BIN, name)
    if not os.path.exists(p):
        from memfabric_hybrid_b200 import _build
        assert _build.build_bench(), "the benchmark tools could not be built"
    return p


def test_bm_perf_benchmark_all_directions():
    out = subprocess.run([_tool("bm_perf_benchmark"), "-bw", "-t", "all", "-s", str(2 << 20), "-bs", "8", "-cc", "20", "-ws", "2", "-lrs", "2",
                          "-ip", f"tcp://127.0.0.1:{free_port()}"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    rows = [l.split() for l in out.stdout.splitlines()[1:] if l and not l.startswith(("ALL", "FAILED"))]
    assert len(rows) == 24 and all(r[-1] == "0" for r in rows), out.stdout     # 12 directions x 2 ranks
    assert "ALL DIRECTIONS VERIFIED" in out.stdout
    print(out.stdout)


def test_transfer_perf_sweep():
    second = 1 if torch.cuda.device_count() > 1 else 0
    out = subprocess.run([_tool("transfer_perf"), "fork", "0", str(second), f"tcp://127.0.0.1:{free_port()}"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    lines = [l for l in out.stdout.splitlines() if l.startswith("Test completed")]
    assert len(lines) == 10 and all("verified yes" in l for l in lines), out.stdout   # 32 KiB .. 16 MiB
    print(out.stdout)
