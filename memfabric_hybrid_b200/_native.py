"""ctypes bindings of the native libraries.

``lib()`` returns libmf_smem.so (host core; always loadable), ``cuda()`` returns libmf_cuda.so
(device backend and kernels; needs only the CUDA runtime that is linked statically, so it loads on
a machine without a GPU too, where its calls report "no device").  Both are built in-tree by
``memfabric_hybrid_b200._build`` on first use when missing.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent
# MF_NATIVE_LIB_DIR selects another build of the libraries (the ASAN + UBSAN build lives in lib_asan/)
_LIB_DIR = Path(os.environ["MF_NATIVE_LIB_DIR"]).resolve() if os.environ.get("MF_NATIVE_LIB_DIR") else _PKG / "lib"
_lock = threading.Lock()
_host = None
_cuda = None

u64, u32, u16, i32, i64 = C.c_uint64, C.c_uint32, C.c_uint16, C.c_int32, C.c_int64
vp, cp = C.c_void_p, C.c_char_p


class TlsConfig(C.Structure):
    _fields_ = [("tlsEnable", C.c_bool)] + [(n, C.c_char * 256) for n in (
        "caPath", "crlPath", "certPath", "keyPath", "keyPassPath", "packagePath", "decrypterLibPath")]


class BmConfigC(C.Structure):
    _fields_ = [("initTimeout", u32), ("createTimeout", u32), ("controlOperationTimeout", u32),
                ("startConfigStoreServer", C.c_bool), ("startConfigStoreOnly", C.c_bool),
                ("dynamicWorldSize", C.c_bool), ("unifiedAddressSpace", C.c_bool), ("autoRanking", C.c_bool),
                ("rankId", u32), ("flags", u32), ("hcomUrl", C.c_char * 64),
                ("hcomTlsConfig", TlsConfig), ("storeTlsConfig", TlsConfig)]


class BmCreateOptionC(C.Structure):
    _fields_ = [("maxDramSize", u64), ("maxHbmSize", u64), ("localDRAMSize", u64), ("localHBMSize", u64),
                ("dataOpType", C.c_int), ("enable56BitsGva", C.c_bool), ("flags", u32), ("tag", C.c_char * 32),
                ("tagOpInfo", C.c_char * 256), ("dramShmFd", C.c_int)]


class CopyParamsC(C.Structure):
    _fields_ = [("src", vp), ("dest", vp), ("dataSize", C.c_size_t), ("stream", vp)]


class BatchCopyParamsC(C.Structure):
    _fields_ = [("sources", C.POINTER(vp)), ("destinations", C.POINTER(vp)), ("dataSizes", C.POINTER(u64)),
                ("batchSize", u32), ("stream", vp)]


class BatchCopyResultC(C.Structure):
    _fields_ = [("results", C.POINTER(i32)), ("batchSize", u32)]


class ShmConfigC(C.Structure):
    _fields_ = [("shmInitTimeout", u32), ("shmCreateTimeout", u32), ("controlOperationTimeout", u32),
                ("startConfigStoreServer", C.c_bool), ("flags", u32)]


class TransConfigC(C.Structure):
    _fields_ = [("role", C.c_int), ("initTimeout", u32), ("deviceId", u32), ("flags", u32), ("dataOpType", C.c_int)]


class TransQuantParamC(C.Structure):
    _fields_ = [("remoteUniqueId", cp), ("localAddrs", C.POINTER(vp)), ("remoteAddrs", C.POINTER(vp)),
                ("dataSizes", C.POINTER(C.c_size_t)), ("scale", C.POINTER(vp)), ("offset", C.POINTER(vp)),
                ("batchSize", u32), ("unitNum", u32), ("stream", vp), ("inputType", u32), ("flags", u32)]


LOG_FN = C.CFUNCTYPE(None, C.c_int, cp)
BM_EVENT_FN = C.CFUNCTYPE(None, vp, u32, C.c_int, vp)
PEER_DOWN_FN = C.CFUNCTYPE(None, cp, vp)
EXIT_FN = C.CFUNCTYPE(None, C.c_int)


def _sig(lib, name, res, *args):
    f = getattr(lib, name)
    f.restype = res
    f.argtypes = list(args)
    return f


def _declare_host(l):
    P = C.POINTER
    _sig(l, "smem_init", i32, u32)
    _sig(l, "smem_uninit", None)
    _sig(l, "smem_create_config_store", i32, cp, u64)
    _sig(l, "smem_destroy_config_store", None, cp)
    _sig(l, "smem_set_extern_logger", i32, LOG_FN)
    _sig(l, "smem_set_log_level", i32, C.c_int)
    _sig(l, "smem_set_conf_store_tls", i32, C.c_bool, cp, u32)
    _sig(l, "smem_set_config_store_tls_key", i32, cp, u32, cp, u32, C.c_void_p)
    _sig(l, "smem_get_last_err_msg", cp)
    _sig(l, "smem_get_last_err_code", i32)
    _sig(l, "smem_get_and_clear_last_err_msg", cp)
    # bm
    _sig(l, "smem_bm_config_init", i32, P(BmConfigC))
    _sig(l, "smem_bm_init", i32, cp, u32, u16, P(BmConfigC))
    _sig(l, "smem_bm_uninit", None, u32)
    _sig(l, "smem_bm_get_rank_id", u32)
    _sig(l, "smem_bm_create", vp, u32, u32, C.c_int, u64, u64, u32)
    _sig(l, "smem_bm_create2", vp, u32, P(BmCreateOptionC))
    _sig(l, "smem_bm_destroy", None, vp)
    _sig(l, "smem_bm_join", i32, vp, u32)
    _sig(l, "smem_bm_leave", i32, vp, u32)
    _sig(l, "smem_bm_extend_local_mem", i32, vp, C.c_int, u64)
    _sig(l, "smem_bm_set_group_event_handler", i32, vp, BM_EVENT_FN, vp)
    _sig(l, "smem_bm_get_local_mem_size_by_mem_type", u64, vp, C.c_int)
    _sig(l, "smem_bm_ptr_by_mem_type", vp, vp, C.c_int, u16)
    _sig(l, "smem_bm_gva_to_va", i32, vp, vp, C.c_int, P(vp))
    _sig(l, "smem_bm_copy", i32, vp, P(CopyParamsC), C.c_int, u32)
    _sig(l, "smem_bm_copy_batch", i32, vp, P(BatchCopyParamsC), C.c_int, u32)
    _sig(l, "smem_bm_copy_batch_partial_succeed", i32, vp, P(BatchCopyParamsC), C.c_int, u32, P(BatchCopyResultC))
    _sig(l, "smem_bm_wait", i32, vp)
    _sig(l, "smem_bm_register_user_mem", i32, vp, u64, u64)
    _sig(l, "smem_bm_unregister_user_mem", i32, vp, u64)
    _sig(l, "smem_bm_get_rank_id_by_gva", u32, vp, vp)


_OPTIONAL_DECLS = []  # filled by modules that bind further symbol groups (shm, trans, zbal, test hooks)


def register_decls(fn):
    """Registers a function(lib) that declares more signatures; applied at load and immediately if loaded."""
    _OPTIONAL_DECLS.append(fn)
    if _host is not None:
        fn(_host)
    return fn


def _ensure_built(which: str) -> None:
    target = _LIB_DIR / ("libmf_smem.so" if which == "host" else "libmf_cuda.so")
    if target.exists():
        return
    if _LIB_DIR != _PKG / "lib":
        raise RuntimeError(f"{target} is missing (MF_NATIVE_LIB_DIR points at a build that does not exist)")
    # Several ranks of one job may arrive here at the same moment on a fresh checkout: one of them builds, the
    # others wait on the file lock and find the library in place.
    import fcntl
    _LIB_DIR.mkdir(exist_ok=True)
    with open(_LIB_DIR / ".build.lock", "w") as lk:
        fcntl.flock(lk, fcntl.LOCK_EX)
        try:
            if not target.exists():
                from . import _build
                (_build.build_host if which == "host" else _build.build_cuda)()
        finally:
            fcntl.flock(lk, fcntl.LOCK_UN)


def lib():
    global _host
    with _lock:
        if _host is None:
            _ensure_built("host")
            l = C.CDLL(str(_LIB_DIR / "libmf_smem.so"), mode=C.RTLD_GLOBAL)
            _declare_host(l)
            for fn in _OPTIONAL_DECLS:
                fn(l)
            _host = l
        return _host


def cuda():
    """libmf_cuda.so, or raises RuntimeError when it cannot be built or loaded."""
    global _cuda
    with _lock:
        if _cuda is None:
            _ensure_built("cuda")
            path = _LIB_DIR / "libmf_cuda.so"
            if not path.exists():
                raise RuntimeError("libmf_cuda.so is missing and nvcc is not available to build it")
            _cuda = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
        return _cuda


def last_error() -> str:
    return (lib().smem_get_last_err_msg() or b"").decode(errors="replace")
