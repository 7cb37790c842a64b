"""The native benchmark tools (benchmark/bm, benchmark/transfer): built, run on the host-only paths, every row verified."""
import os
import subprocess

import pytest

from conftest import free_port

BIN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "memfabric_hybrid_b200", "bin")


@pytest.fixture(scope="module")
def tools():
    from memfabric_hybrid_b200 import _build, _native
    _native.lib()   # the host library is built on first use
    if not (os.path.exists(os.path.join(BIN, "bm_perf_benchmark")) and os.path.exists(os.path.join(BIN, "transfer_perf"))):
        if not _build.build_bench():
            pytest.skip("nvcc is not available to build the tools")
    return BIN


def _env():
    e = dict(os.environ)
    e["CUDA_VISIBLE_DEVICES"] = ""   # host paths only, also on a GPU box
    return e


def test_bm_perf_benchmark_host_directions(tools):
    out = subprocess.run([os.path.join(tools, "bm_perf_benchmark"), "-bw", "-t", "all", "-ot", "host_shm", "-s", "262144", "-bs", "4",
                          "-cc", "10", "-ws", "2", "-lrs", "2", "-ip", f"tcp://127.0.0.1:{free_port()}"],
                         capture_output=True, text=True, timeout=120, env=_env())
    assert out.returncode == 0, out.stdout + out.stderr
    rows = [l.split() for l in out.stdout.splitlines() if l.startswith(("h2rh", "rh2h"))]
    assert len(rows) == 4 and all(r[-1] == "0" for r in rows), out.stdout
    assert "ALL DIRECTIONS VERIFIED" in out.stdout


def test_bm_perf_benchmark_rejects_bad_arguments(tools):
    out = subprocess.run([os.path.join(tools, "bm_perf_benchmark"), "-t", "sideways"], capture_output=True, text=True, timeout=30)
    assert out.returncode == 2 and "unknown direction" in out.stderr


def test_transfer_perf_fork_mode(tools):
    e = _env()
    e["MF_PERF_MAX_BLOCK_KB"] = "128"
    out = subprocess.run([os.path.join(tools, "transfer_perf"), "fork", "0", "1", f"tcp://127.0.0.1:{free_port()}"],
                         capture_output=True, text=True, timeout=120, env=e)
    assert out.returncode == 0, out.stdout + out.stderr
    lines = [l for l in out.stdout.splitlines() if l.startswith("Test completed")]
    assert len(lines) == 3 and all("verified yes" in l for l in lines), out.stdout


def test_transfer_performance_python_tool():
    """The Python twin (benchmark/transfer/transfer_performance.py): both ranks from one command, host buffers."""
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    e = _env()
    e["MF_DEVICE_BACKEND"] = "none"
    out = subprocess.run([sys.executable, os.path.join(root, "benchmark", "transfer", "transfer_performance.py"), "--both",
                          "--store-url", f"tcp://127.0.0.1:{free_port()}", "--max-block-kb", "64", "--num-threads", "2"],
                         capture_output=True, text=True, timeout=180, env=e)
    assert out.returncode == 0, out.stdout + out.stderr
    lines = [l for l in out.stdout.splitlines() if l.startswith("Test completed")]
    assert len(lines) == 2 and all("verified yes" in l for l in lines), out.stdout
