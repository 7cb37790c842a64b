"""The host library under AddressSanitizer + UndefinedBehaviorSanitizer: the control-plane and host-pool tests run
once more against ``lib_asan/libmf_smem.so`` (the reference runs its unit tests under the same sanitizers)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FILES = ["test_config_store.py", "test_group_engine.py", "test_ha_store.py", "test_trace_failpoints.py", "test_transfer_cpu.py",
         "test_shm_api_cpu.py", "test_bm_host_pool.py", "test_fake_device_pool.py", "test_zbal_cpu.py", "test_store_tls.py", "test_etcd_backend.py", "test_fuzz_cpu.py"]


def test_host_tests_are_clean_under_asan_and_ubsan():
    from memfabric_hybrid_b200 import _build
    rt = _build.asan_runtime()
    if rt is None:
        pytest.skip("the compiler ships no libasan.so")
    lib = _build.build_host(asan=True)
    env = dict(os.environ, LD_PRELOAD=rt, MF_NATIVE_LIB_DIR=os.path.dirname(str(lib)),
               ASAN_OPTIONS="detect_leaks=0:halt_on_error=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    # -s: a sanitizer report must reach this process's pipe; the c10d extension is not part of the sanitizer build
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-s", "-p", "no:cacheprovider", "-k", "not native"] +
                       [os.path.join(ROOT, "tests", f) for f in FILES], env=env, capture_output=True, text=True, errors="replace", timeout=1500, cwd=ROOT)   # log lines may quote fuzzed bytes
    out = r.stdout + r.stderr
    assert "runtime error:" not in out and "ERROR: AddressSanitizer" not in out, out[-4000:]
    assert r.returncode == 0, out[-4000:]


TSAN_FILES = ["test_config_store.py", "test_ha_store.py", "test_group_engine.py", "test_etcd_backend.py", "test_fuzz_cpu.py", "test_store_tls.py",
              "test_trace_failpoints.py", "test_bm_host_pool.py", "test_transfer_cpu.py"]


def test_control_plane_is_free_of_data_races_under_tsan():
    """The threaded part of the host library (RPC endpoints, store client / server, the highly available store, the etcd
    backend, the group engine, tracer and fault points, the DRAM pool and the transfer engine with their copy threads and the
    descriptor channel) once more against ``lib_tsan/libmf_smem.so``. The pools' address windows lie where ThreadSanitizer
    keeps its shadow memory: MF_GVA_DRAM_BASE moves the DRAM space into the 5 TiB the sanitizer leaves to the program; the
    symmetric-memory and device windows (further up in their space) and the 16 TiB of a 56-bit pool do not fit there."""
    from memfabric_hybrid_b200 import _build
    rt = _build.tsan_runtime()
    if rt is None:
        pytest.skip("the compiler ships no libtsan.so")
    # some kernels' address-space randomisation leaves the sanitizer no room for its shadow memory: it then dies at start-up
    probe = subprocess.run([sys.executable, "-c", "pass"], env=dict(os.environ, LD_PRELOAD=rt), capture_output=True, text=True, timeout=120)
    if probe.returncode != 0:
        pytest.skip("ThreadSanitizer cannot start in this environment: " + (probe.stderr.strip().splitlines() or ["?"])[-1][:200])
    lib = _build.build_host(tsan=True)
    env = dict(os.environ, LD_PRELOAD=rt, MF_NATIVE_LIB_DIR=os.path.dirname(str(lib)), MF_FUZZ_LIGHT="1",
               OPENBLAS_NUM_THREADS="1", OMP_NUM_THREADS="1",       # no library threads around when a test forks
               MF_GVA_DRAM_BASE=str(0x560000000000),
               TSAN_OPTIONS="halt_on_error=0:report_signal_unsafe=0:history_size=4:exitcode=0")
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-s", "-p", "no:cacheprovider", "-k", "not native and not exchange_records and not 56_bit and not survives_the_death"] +   # (the four-process failover scenario runs on lease and recovery timers: too slow under this sanitizer)
                       [os.path.join(ROOT, "tests", f) for f in TSAN_FILES], env=env, capture_output=True, text=True, errors="replace",
                       timeout=2400, cwd=ROOT)
    out = r.stdout + r.stderr
    assert "WARNING: ThreadSanitizer" not in out, out[out.find("WARNING: ThreadSanitizer"):][:6000]
    assert r.returncode == 0, out[-4000:]
