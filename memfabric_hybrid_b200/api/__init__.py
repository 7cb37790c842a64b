"""Python surface with the names of the reference's ``memfabric_hybrid`` wheel.

    import memfabric_hybrid as mf           # or: from memfabric_hybrid_b200 import api as mf
    mf.initialize(); mf.bm.initialize(url, world, dev, cfg); h = mf.bm.create2(...); h.join(); ...

Every call forwards to the C ABI in libmf_smem.so through ctypes, which releases the GIL for the
duration of the call (the reference's pybind11 module does the same with ``gil_scoped_release``).
Parity: src/smem/csrc/python_wrapper/memfabric_hybrid/pymf_hybrid.cpp:444-861, doc/pythonAPI.md.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable

from .. import _native as N

_keep = {}  # callbacks handed to C must stay referenced


def initialize(flags: int = 0) -> int:
    return N.lib().smem_init(flags)


def uninitialize() -> None:
    N.lib().smem_uninit()


def create_config_store(store_url: str, flags: int = 0) -> int:
    return N.lib().smem_create_config_store(store_url.encode(), flags)


def destroy_config_store(store_url: str) -> None:
    N.lib().smem_destroy_config_store(store_url.encode())


def set_log_level(level: int) -> int:
    return N.lib().smem_set_log_level(int(level))


def set_extern_logger(log_fn: Callable[[int, str], None]) -> int:
    if log_fn is None:
        _keep.pop("logger", None)
        return N.lib().smem_set_extern_logger(C.cast(None, N.LOG_FN))
    cb = N.LOG_FN(lambda lv, msg: log_fn(lv, (msg or b"").decode(errors="replace")))
    _keep["logger"] = cb
    return N.lib().smem_set_extern_logger(cb)


def set_conf_store_tls(enable: bool, tls_info: str = "") -> int:
    b = tls_info.encode()
    return N.lib().smem_set_conf_store_tls(bool(enable), b, len(b))


def set_conf_store_tls_key(tls_pk: str, tls_pk_pw: str = "", py_decrypt_func: Callable[[str], str] | None = None) -> int:
    """Private key of this process's store links: PEM text or the path of a PEM file; tls_pk_pw is its pass phrase, turned
    into plain text by py_decrypt_func when one is given. Applies to stores created afterwards."""
    if not tls_pk:
        return -2000
    pw = tls_pk_pw or ""
    if pw and py_decrypt_func is not None:
        pw = py_decrypt_func(pw)
    k, w = tls_pk.encode(), pw.encode()
    return N.lib().smem_set_config_store_tls_key(k, len(k), w if w else None, len(w), None)


def get_last_err_msg() -> str:
    return N.last_error()


def get_last_err_code() -> int:
    return N.lib().smem_get_last_err_code()


def get_and_clear_last_err_msg() -> str:
    return (N.lib().smem_get_and_clear_last_err_msg() or b"").decode(errors="replace")


from . import bm, shm  # noqa: E402
from .transfer import TransferEngine, TransDataOpType, TransferOpcode  # noqa: E402

__all__ = ["initialize", "uninitialize", "create_config_store", "destroy_config_store", "set_log_level",
           "set_extern_logger", "set_conf_store_tls", "set_conf_store_tls_key", "get_last_err_msg",
           "get_last_err_code", "get_and_clear_last_err_msg", "bm", "shm", "TransferEngine",
           "TransDataOpType", "TransferOpcode"]
