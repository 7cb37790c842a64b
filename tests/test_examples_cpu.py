"""The examples that need no GPU run as written and exit 0."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script", ["examples/memory_pool/01_two_rank_dram_pool.py", "examples/memory_pool/02_copy_data_batch_and_register.py",
                                    "examples/memory_pool/04_extend_local_mem.py",
                                    "examples/transfer/transfer_engine.py", "examples/tensor_rtl/reshard_tp4_to_tp2.py",
                                    "examples/tensor_rtl/eplb_expert_migration.py", "examples/tensor_rtl/rl_train_to_infer_reshard.py"])
def test_example_runs(script):
    env = dict(os.environ, MF_DEVICE_BACKEND="none")
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    r = subprocess.run([sys.executable, os.path.join(ROOT, script)], env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
