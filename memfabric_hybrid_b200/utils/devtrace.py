"""Device timeline of the communication kernels as a Chrome-trace file (open it in chrome://tracing or Perfetto).

    from memfabric_hybrid_b200.utils import devtrace
    devtrace.enable()                     # or set ZBAL_PROF_ENABLE=1 before importing zbal / ops
    ... run collectives / MoE dispatch ...
    devtrace.dump("trace.json")           # also written at exit and on SIGUSR1 when enabled from the environment

Environment (names of the reference, app/zbal/doc/performance/npu/prof_npu_profiling_tool.md:15-44):
ZBAL_PROF_ENABLE=1, ZBAL_PROF_MAX_TRACING_COUNT (records per CTA lane, default 20480), ZBAL_PROF_DIR (default ".").
Kernels mark phases with MF_PROF_START/STOP (csrc/kernels/mf_devtrace.cuh); one lane per CTA index, 8 bytes a record.
"""
from __future__ import annotations

import atexit
import ctypes as C
import os
import signal

from .. import _native as N

_enabled = False


def _cu():
    l = N.cuda()
    l.mf_devtrace_enable.restype = C.c_int
    l.mf_devtrace_enable.argtypes = [C.c_uint32, C.c_uint32]
    l.mf_devtrace_disable.restype = C.c_int
    l.mf_devtrace_count.restype = C.c_longlong
    l.mf_devtrace_dump.restype = C.c_longlong
    l.mf_devtrace_dump.argtypes = [C.c_char_p, C.c_int, C.c_int]
    return l


def enable(lanes: int = 512, per_lane: int | None = None) -> None:
    global _enabled
    per = per_lane or int(os.environ.get("ZBAL_PROF_MAX_TRACING_COUNT", "20480"))
    rc = _cu().mf_devtrace_enable(lanes, per)
    if rc != 0:
        raise RuntimeError(f"device trace could not be enabled ({rc})")
    _enabled = True


def disable() -> None:
    global _enabled
    if _enabled:
        _cu().mf_devtrace_disable()
        _enabled = False


def count() -> int:
    return int(_cu().mf_devtrace_count()) if _enabled else 0


def default_path() -> str:
    return os.path.join(os.environ.get("ZBAL_PROF_DIR", "."), f"zbal_trace_{os.getpid()}.json")


def dump(path: str | None = None, rank: int | None = None, reset: bool = True) -> int:
    """Writes the events recorded so far; returns how many."""
    if not _enabled:
        return 0
    r = int(os.environ.get("RANK", "0")) if rank is None else rank
    n = _cu().mf_devtrace_dump((path or default_path()).encode(), r, 1 if reset else 0)
    if n < 0:
        raise RuntimeError(f"device trace dump failed ({n})")
    return int(n)


def enable_from_env() -> bool:
    """Turns tracing on when ZBAL_PROF_ENABLE=1; the file is then written at exit and on SIGUSR1."""
    if os.environ.get("ZBAL_PROF_ENABLE", "0") != "1" or _enabled:
        return _enabled
    enable()
    atexit.register(lambda: dump(reset=False))
    try:
        signal.signal(signal.SIGUSR1, lambda *_: dump(reset=False))
    except ValueError:  # not the main thread
        pass
    return True
