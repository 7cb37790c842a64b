"""In-tree build of the native libraries.

    libmf_smem.so   host core (g++): util, RPC, config store, group engine, hybm, smem/zbal C APIs
    libmf_cuda.so   device backend and every sm_100a kernel (nvcc, static cudart)
    _zbal_c10d.so   the torch.distributed backend "zbal" as a c10d::Backend (g++ against libtorch, links libmf_smem)

Objects are cached under ``build/`` keyed by a hash of the source, its local includes and the
flags, so a rebuild only recompiles what changed.  ``python -m memfabric_hybrid_b200._build``
builds everything; ``--host`` / ``--cuda`` restrict it.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
BUILD = PKG.parent / "build"

HOST_DIRS = ["util", "net", "store", "group", "hybm", "smem", "zbal"]
CXXFLAGS = ["-std=c++17", "-O2", "-g", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter", "-pthread",
            "-fvisibility=default", "-fstack-protector-strong", "-D_FORTIFY_SOURCE=2"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _hash(src: Path, flags: list[str]) -> str:
    h = hashlib.sha1()
    h.update(" ".join(flags).encode())
    h.update(src.read_bytes())
    # every header of the tree participates: cheap and always correct
    for hdr in sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh"))):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _compile(cmd: list[str], src: Path, obj: Path, log: Path) -> tuple[Path, int, str]:
    # compile to a name of this process and move it into place: a second builder never sees a half-written object
    tmp = obj.with_name(f"{obj.name}.{os.getpid()}.tmp")
    p = subprocess.run(cmd + ["-c", str(src), "-o", str(tmp)], capture_output=True, text=True)
    log.write_text(p.stdout + p.stderr)
    if p.returncode == 0:
        tmp.replace(obj)
    elif tmp.exists():
        tmp.unlink()
    return src, p.returncode, p.stdout + p.stderr


def _build_objs(srcs: list[Path], cmd: list[str], flags: list[str], tag: str, jobs: int) -> list[Path]:
    BUILD.mkdir(exist_ok=True)
    objs, todo = [], []
    for s in srcs:
        obj = BUILD / f"{tag}_{s.stem}_{_hash(s, flags)}.o"
        objs.append(obj)
        if not obj.exists():
            todo.append((s, obj))
    if todo:
        with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
            futs = [ex.submit(_compile, cmd + flags, s, o, BUILD / f"{tag}_{s.stem}.log") for s, o in todo]
            failed = False
            for f in futs:
                src, rc, out = f.result()
                if rc != 0:
                    failed = True
                    sys.stderr.write(f"--- {src}\n{out}\n")
            if failed:
                raise RuntimeError(f"{tag}: compilation failed")
    return objs


SAN_FLAGS = ["-fsanitize=address,undefined,pointer-compare,pointer-subtract", "-fno-omit-frame-pointer", "-fno-sanitize-recover=undefined"]


TSAN_FLAGS = ["-fsanitize=thread", "-fno-omit-frame-pointer"]


def build_host(jobs: int | None = None, asan: bool = False, tsan: bool = False) -> Path:
    """``asan=True``: the same sources under AddressSanitizer + UndefinedBehaviorSanitizer into ``lib_asan/``
    (load it with MF_NATIVE_LIB_DIR and LD_PRELOAD of the compiler's libasan.so). ``tsan=True``: under ThreadSanitizer
    into ``lib_tsan/`` (LD_PRELOAD of libtsan.so)."""
    jobs = jobs or os.cpu_count() or 4
    srcs = [p for d in HOST_DIRS for p in sorted((CSRC / d).glob("*.cpp"))]
    flags = CXXFLAGS + [f"-I{CSRC / 'include'}", f"-I{CSRC}"]
    libdir, san, tag = LIB, [], "host"
    if asan or tsan:
        san = SAN_FLAGS if asan else TSAN_FLAGS
        flags = [f for f in flags if f not in ("-O2", "-D_FORTIFY_SOURCE=2")] + ["-O1"] + san
        libdir, tag = (PKG / "lib_asan", "asan") if asan else (PKG / "lib_tsan", "tsan")
    objs = _build_objs(srcs, ["g++"], flags, tag, jobs)
    libdir.mkdir(exist_ok=True)
    out = libdir / "libmf_smem.so"
    tmp = out.with_suffix(f".so.{os.getpid()}.tmp")
    subprocess.run(["g++", "-shared", "-o", str(tmp)] + [str(o) for o in objs] + san +
                   ["-pthread", "-ldl", "-lrt", "-Wl,-z,relro,-z,now"], check=True)
    tmp.replace(out)
    return out


def tsan_runtime() -> str | None:
    """Path of the compiler's libtsan.so (to LD_PRELOAD under Python), or None."""
    p = subprocess.run(["gcc", "-print-file-name=libtsan.so"], capture_output=True, text=True).stdout.strip()
    return p if os.path.isabs(p) and os.path.exists(p) else None


def asan_runtime() -> str | None:
    """Path of the compiler's libasan.so (to LD_PRELOAD under Python), or None."""
    p = subprocess.run(["gcc", "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    return p if p and os.path.isabs(p) and os.path.exists(p) else None


def build_cuda(jobs: int | None = None) -> Path | None:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        return None
    jobs = jobs or os.cpu_count() or 4
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    if not srcs:
        return None
    flags = NVCC_FLAGS + [f"-I{CSRC / 'include'}", f"-I{CSRC}"]
    objs = _build_objs(srcs, [nvcc], flags, "cuda", jobs)
    LIB.mkdir(exist_ok=True)
    out = LIB / "libmf_cuda.so"
    tmp = out.with_suffix(f".so.{os.getpid()}.tmp")
    subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(tmp)] + [str(o) for o in objs] +
                   ["-cudart", "static", f"-L{LIB}", "-lmf_smem", "-Xlinker", "-rpath=$ORIGIN", "-Xlinker", "-z,relro",
                    "-lpthread", "-ldl", "-lrt"], check=True)
    tmp.replace(out)
    return out


def build_bench() -> list[Path]:
    """The native benchmark tools (benchmark/bm, benchmark/transfer) into memfabric_hybrid_b200/bin/. They use the public C
    API of libmf_smem.so plus the CUDA runtime for their private buffers."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    bench = PKG.parent / "benchmark"
    if not Path(nvcc).exists() or not bench.exists():
        return []
    bindir = PKG / "bin"
    bindir.mkdir(exist_ok=True)
    outs = []
    for src in (bench / "bm" / "bm_perf_benchmark.cpp", bench / "transfer" / "transfer_perf.cpp"):
        out = bindir / src.stem
        tmp = out.with_suffix(f".{os.getpid()}.tmp")
        subprocess.run([nvcc, "-O2", "-std=c++17", "-x", "cu", "-gencode", "arch=compute_100a,code=sm_100a", f"-I{CSRC / 'include'}", "-o", str(tmp), str(src), "-cudart", "static",
                        f"-L{LIB}", "-lmf_smem", "-Xlinker", "-rpath=$ORIGIN/../lib", "-lpthread", "-ldl", "-lrt"], check=True)
        tmp.replace(out)
        outs.append(out)
    return outs


def build_c10d() -> Path | None:
    """The c10d extension module. Needs PyTorch's headers and a CUDA include tree; returns None without them."""
    try:
        import torch
        from torch.utils import cpp_extension as ce
    except Exception:
        return None
    cuda_inc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
    if not (cuda_inc / "cuda_runtime_api.h").exists():
        return None
    import sysconfig
    tdir = Path(torch.__file__).resolve().parent
    srcs = sorted((CSRC / "c10d").glob("*.cpp"))
    incs = [str(tdir / "include"), str(tdir / "include" / "torch" / "csrc" / "api" / "include"), str(cuda_inc),
            sysconfig.get_paths()["include"], str(CSRC / "include"), str(CSRC)]
    abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    flags = ["-std=c++17", "-O2", "-fPIC", "-pthread", "-fvisibility=hidden", "-Wall", "-Wno-unused-parameter", "-Wno-interference-size",
             f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_zbal_c10d", "-DTORCH_API_INCLUDE_EXTENSION_H",
             "-DUSE_C10D", "-DUSE_CUDA", f"-DTORCH_VERSION_TAG={torch.__version__.replace('+', '_').replace('.', '_')}"] + \
            [f"-I{i}" for i in incs]
    objs = _build_objs(srcs, ["g++"], flags, "c10d", os.cpu_count() or 4)
    LIB.mkdir(exist_ok=True)
    build_host()
    out = LIB / "_zbal_c10d.so"
    tmp = out.with_suffix(f".so.{os.getpid()}.tmp")
    tlib = tdir / "lib"
    subprocess.run(["g++", "-shared", "-o", str(tmp)] + [str(o) for o in objs] +
                   [f"-L{tlib}", "-ltorch_python", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
                    f"-L{LIB}", "-lmf_smem", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}", "-pthread"], check=True)
    tmp.replace(out)
    return out


def build_all() -> None:
    build_host()
    build_cuda()
    build_c10d()
    build_bench()


if __name__ == "__main__":
    args = set(sys.argv[1:])
    if "--asan" in args:
        print(build_host(asan=True))
        args.discard("--asan")
    if "--tsan" in args:
        print(build_host(tsan=True))
        args.discard("--tsan")
        if not args:
            sys.exit(0)
    if not args or "--host" in args:
        print(build_host())
    if not args or "--cuda" in args:
        print(build_cuda())
    if not args or "--c10d" in args:
        print(build_c10d())
    if not args or "--bench" in args:
        print(build_bench())
