"""Drop-in compatibility: example scripts written against the reference's ``memfabric_hybrid`` Python API run UNCHANGED
against this repository's module (they import only ``torch`` and ``memfabric_hybrid``). The scripts are read from the
reference tree when it is present on the machine (it is not shipped with this repository); command-line options that a
script offers are used to keep its memory footprint small, its source is not touched.

Not run here, with the reason:
  * 01_basic/03_single_device_hbm_pool, 06_single_card_external_stream, examples/transfer/*.py: they import ``torch_npu`` /
    need an HBM pool (a GPU); the HBM pool and the transfer engine are covered by tests/test_gpu_*.py;
  * 02_scale_out/02_multi_node_multi_device_dram: wants two hosts;
  * 04_features/03_enable_56bits_gva: asks for a 1 PiB global address range (1024 ranks x 1 TiB); this implementation maps
    global addresses 1:1 into the process's 47-bit address space and refuses that range;
  * 01_basic/04, 05 (host RDMA / URMA pools): need the hcom transport library of the reference.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REF = Path(os.environ.get("MF_REFERENCE_TREE") or Path(__file__).resolve().parents[2] / "reference") / "examples" / "memory_pool"

CASES = [
    ("01_basic/01_single_device_dram_pool/01_single_device_dram_pool.py", [], "01_single_device_dram_pool ok"),
    ("01_basic/02_single_device_dram_configurable_pool/02_single_device_dram_configurable_pool.py", [], "PASSED"),
    ("02_scale_out/01_single_node_multi_device_dram/01_single_node_multi_device_dram.py", [], "all ranks OK"),
    ("03_optimization/01_copy_data_batch/01_copy_data_batch.py", [], "01_copy_data_batch ok"),
    ("03_optimization/02_register/02_register.py", [], "02_register ok"),
    ("03_optimization/03_device_sdma/03_device_sdma.py", [], "03_device_sdma ok"),
    ("04_features/02_extend_local_mem/02_extend_local_mem.py", ["--world_size", "2", "--local_ranks", "2"], "alloc extend memory test ok"),
    # 2 of 1 024 ranks of a pool with 1 TiB per rank: a 1 PiB window of 56-bit addresses
    ("04_features/03_enable_56bits_gva/03_enable_56bits_gva.py",
     ["--world_size", "1024", "--local_ranks", "2", "--rank_start", "0", "--protocol", "device_sdma", "--url", "tcp://127.0.0.1:{port}"],
     "rank:1, 56-bit GVA test ok."),
]


@pytest.mark.skipif(not REF.is_dir(), reason="the reference tree is not on this machine")
@pytest.mark.parametrize("script,args,marker", CASES, ids=[c[0].split("/")[-1] for c in CASES])
def test_reference_example_runs_unchanged(script, args, marker, tmp_path):
    path = REF / script
    if not path.is_file():
        pytest.skip(f"{script} is not in this version of the reference")
    env = dict(os.environ)
    env["PYTHONPATH"] = str(ROOT) + os.pathsep + env.get("PYTHONPATH", "")
    env["MF_DEVICE_BACKEND"] = "none"     # CPU tier: DRAM pools only
    if any("{port}" in a for a in args):
        import socket
        sk = socket.socket()
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
        sk.close()
        args = [a.replace("{port}", str(port)) for a in args]
    p = subprocess.run([sys.executable, str(path)] + args, cwd=tmp_path, env=env, capture_output=True, text=True, timeout=300)
    out = p.stdout + p.stderr
    assert p.returncode == 0, out[-3000:]
    assert marker in out, out[-3000:]
