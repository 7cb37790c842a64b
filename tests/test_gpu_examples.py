"""The shipped examples run as written (each in child processes)."""
import importlib.util
import os

import pytest
import torch

from conftest import free_port
from mp_util import run_ranks

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(path):
    spec = importlib.util.spec_from_file_location("example_" + os.path.basename(path)[:-3], os.path.join(ROOT, path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _shm_allreduce(rank, world, url):
    return _load("examples/hbm_share_memory/allreduce.py").run(rank, world, rank % torch.cuda.device_count(), url, n=300_000)


def test_shm_user_kernel_single_gpu():
    assert run_ranks(_shm_allreduce, 1, (f"tcp://127.0.0.1:{free_port()}",), timeout=180) == [0.0]


@pytest.mark.multigpu
def test_shm_user_kernel_multi_gpu():
    n = min(torch.cuda.device_count(), 4)
    assert run_ranks(_shm_allreduce, n, (f"tcp://127.0.0.1:{free_port()}",), timeout=240) == [0.0] * n


def _shm_shift(rank, world, url):
    return _load("examples/hbm_share_memory/shift_put_get.py").run(rank, world, rank % torch.cuda.device_count(), url, n=300_000)


def test_shm_shift_single_gpu():
    assert run_ranks(_shm_shift, 1, (f"tcp://127.0.0.1:{free_port()}",), timeout=180) == [0.0]


@pytest.mark.multigpu
def test_shm_shift_multi_gpu():
    n = min(torch.cuda.device_count(), 4)
    assert run_ranks(_shm_shift, n, (f"tcp://127.0.0.1:{free_port()}",), timeout=240) == [0.0] * n


def test_hbm_pool_example():
    import subprocess
    import sys
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples/memory_pool/03_hbm_pool_external_stream.py")], capture_output=True, text=True,
                       timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def test_quant_transfer_example():
    import subprocess
    import sys
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE")}
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples/transfer/quant_transfer.py")], env=env, capture_output=True, text=True,
                       timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def test_zbal_backend_example_single_process():
    import subprocess
    import sys
    env = dict(os.environ, RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples/zbal/allreduce_backend.py")], env=env, capture_output=True, text=True,
                       timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
