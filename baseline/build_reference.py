#!/usr/bin/env python
"""Builds the UNMODIFIED reference (CPU-only flavour, -DXPU_TYPE=NONE: config store, group engine, HOST_SHM DRAM pool and
its Python bindings) from a copy under /tmp and lays its Python package out under baseline/_ref/memfabric_hybrid, the way
the reference's own wheel does (package sources + the two extension modules + lib/*.so).

    python baseline/build_reference.py [path of the reference tree; default: $MF_REFERENCE_TREE, else the tree beside this repository]

`pip install <reference>` does not work (the tree has no setup.py / pyproject.toml at its root); the CMake build needs no
network with these options. Returns 0 when baseline/_ref is usable afterwards.
"""
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref" / "memfabric_hybrid"


def usable() -> bool:
    tag = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return (DEST / "__init__.py").is_file() and (DEST / ("_pymf_hybrid" + tag)).is_file() and (DEST / "lib" / "libmf_smem.so").is_file()


DEFAULT_REF = os.environ.get("MF_REFERENCE_TREE") or str(Path(__file__).resolve().parents[2] / "reference")


def build(ref: str = DEFAULT_REF, jobs: int | None = None, log=None) -> bool:
    if usable():
        return True
    ref_path = Path(ref)
    if not (ref_path / "CMakeLists.txt").is_file() or shutil.which("cmake") is None:
        return False
    work = Path("/tmp") / f"mf_ref_build_{os.getuid()}"
    shutil.rmtree(work, ignore_errors=True)
    shutil.copytree(ref_path, work, symlinks=True)
    out = open(log, "w") if log else subprocess.DEVNULL
    try:
        cfg = ["cmake", "-S", str(work), "-B", str(work / "build"), "-DCMAKE_BUILD_TYPE=RELEASE", "-DXPU_TYPE=NONE", "-DBUILD_PYTHON=ON",
               "-DBUILD_GIT_COMMIT=OFF", "-DBUILD_OPEN_ABI=ON", f"-DPython3_EXECUTABLE={sys.executable}"]
        if subprocess.run(cfg, stdout=out, stderr=subprocess.STDOUT).returncode != 0:
            return False
        if subprocess.run(["make", "-C", str(work / "build"), f"-j{jobs or os.cpu_count() or 8}"], stdout=out, stderr=subprocess.STDOUT).returncode != 0:
            return False
    finally:
        if log:
            out.close()
    b = work / "build" / "src"
    shutil.rmtree(DEST.parent, ignore_errors=True)
    (DEST / "lib").mkdir(parents=True)
    for f in (work / "src" / "smem" / "python" / "memfabric_hybrid" / "memfabric_hybrid").glob("*.py"):
        shutil.copy(f, DEST / f.name)
    for pat, sub in (("smem/csrc/python_wrapper/memfabric_hybrid/_pymf_hybrid*.so", ""), ("smem/csrc/python_wrapper/mk_transfer_adapter/_pymf_transfer*.so", ""),
                     ("smem/csrc/libmf_smem.so", "lib"), ("hybm/csrc/libmf_hybm_core.so", "lib"), ("acc_links/csrc/libacc_tcp_net.so", "lib")):
        for f in b.glob(pat):
            shutil.copy(f, DEST / sub / f.name)
    shutil.rmtree(work, ignore_errors=True)
    return usable()


if __name__ == "__main__":
    ok = build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REF, log=str(HERE / "_ref_build.log"))
    print("baseline/_ref is", "ready" if ok else "NOT available")
    sys.exit(0 if ok else 1)
