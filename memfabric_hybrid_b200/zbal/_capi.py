"""ctypes view of the zbal C entry points in libmf_smem.so (headers: csrc/include/zbal*.h)."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N

u64, u32, i32, i64, vp = C.c_uint64, C.c_uint32, C.c_int32, C.c_int64, C.c_void_p

Z_OK = 0
Z_NOT_SUPPORTED = -6

# zbal_datatype_t
DT = {torch.int8: 0, torch.int16: 1, torch.int32: 2, torch.int64: 3, torch.float64: 5, torch.float16: 6, torch.float32: 7,
      torch.bfloat16: 8, torch.uint8: 9, torch.bool: 9, torch.float8_e4m3fn: 9, torch.float8_e5m2: 9}
REDUCIBLE = (torch.bfloat16, torch.float16, torch.float32, torch.int32)
# zbal_reduce_op_t
OP_PROD, OP_SUM, OP_MAX, OP_MIN = 0, 1, 2, 3


class BootstrapOptionsC(C.Structure):
    _fields_ = [("flags", u32), ("btType", C.c_int), ("ipPort", C.c_char * 128), ("worldSize", u32), ("rankId", u32),
                ("deviceId", i32), ("startConfigServer", C.c_bool), ("deviceMemorySize", u64), ("dataOperationType", C.c_int),
                ("commMetaSpaceSize", u64), ("commGroupCap", u32)]


class BootstrapOutputC(C.Structure):
    _fields_ = [("baseGva", u64), ("localGva", u64), ("symmetricSize", u64), ("commAreaSize", u64), ("heapGva", u64),
                ("heapSize", u64), ("worldSize", u32), ("rankId", u32)]


class AllocatorOptionsC(C.Structure):
    _fields_ = [("baseAddress", u64), ("size", u64), ("smallThreshold", u64), ("deviceId", i32), ("flags", u32)]


class CommOptionsC(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("firstRank", u32), ("rankStep", u32), ("groupSize", u32), ("flags", u32)]


class CommPropertyC(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("groupId", u32), ("groupSize", u32), ("groupRank", u32), ("firstRank", u32),
                ("rankStep", u32), ("signalGva", u64), ("stageBytes", u64), ("epoch", u64)]


class MoeOptionsC(C.Structure):
    _fields_ = [("maxTokens", u32), ("hidden", u32), ("experts", u32), ("topk", u32), ("maxRecv", u32), ("rawBf16", u32)]


class MoeBuffersC(C.Structure):
    _fields_ = [("recvTokens", vp), ("recvScales", vp), ("recvInfo", vp), ("maxRecv", u32), ("localExperts", u32)]


class SmaStatsC(C.Structure):
    _fields_ = [(n, u64) for n in ("heapSize", "inUseBytes", "cachedBytes", "peakInUseBytes", "largestFreeBlock", "mallocCalls",
                                   "freeCalls", "cacheHits", "heapCarves", "failedMallocs", "poolCount", "poolCachedBytes", "segments",
                                   "segmentsAdded")]


_declared = False


def _declare(l):
    P = C.POINTER
    s = N._sig
    s(l, "zbal_version", C.c_char_p)
    s(l, "zbal_set_logger_level", i32, C.c_int)
    s(l, "zbal_get_last_error_msg", C.c_char_p)
    s(l, "zbal_get_and_clear_last_error_msg", C.c_char_p)
    s(l, "zbal_bootstrap_options_init", i32, P(BootstrapOptionsC))
    s(l, "zbal_bootstrap", i32, P(BootstrapOptionsC), P(BootstrapOutputC))
    s(l, "zbal_unbootstrap", i32, u32)
    s(l, "zbal_is_bootstrapped", i32)
    s(l, "zbal_bootstrap_get_output", i32, P(BootstrapOutputC))
    s(l, "zbal_sma_init", i32, P(AllocatorOptionsC), i32)
    s(l, "zbal_sma_uninit", None, i32)
    s(l, "zbal_pluggable_init", None, i32)
    s(l, "zbal_pluggable_malloc", vp, C.c_size_t, i32, vp)
    s(l, "zbal_pluggable_free", None, vp, C.c_size_t, i32, vp)
    s(l, "zbal_pluggable_empty_cache", None, C.c_bool)
    s(l, "zbal_simulate_init", None, i64, i64)
    s(l, "zbal_sma_begin_pool", i32, u64, u64, vp, vp)
    s(l, "zbal_sma_end_pool", i32, u64, u64)
    s(l, "zbal_sma_release_pool", i32, u64, u64)
    s(l, "zbal_sma_get_stats", i32, P(SmaStatsC))
    s(l, "zbal_sma_add_segment", i32, u64, u64)
    s(l, "zbal_heap_expand", i32, P(u64), P(u64))
    s(l, "zbal_is_symmetric", i32, C.c_void_p, u64)
    s(l, "zbal_sma_reset_peak", None)
    s(l, "zbal_sma_record_history", None, C.c_bool, u32)
    s(l, "zbal_sma_snapshot", i64, C.c_char_p, i64)
    s(l, "zbal_comm_create", i32, P(CommOptionsC), P(vp))
    s(l, "zbal_comm_get_property", i32, vp, P(CommPropertyC))
    s(l, "zbal_comm_get_global", vp)
    s(l, "zbal_comm_get_by_name", vp, C.c_char_p)
    s(l, "zbal_comm_destroy", i32, vp, u32)
    s(l, "zbal_comm_destroy_all", None, u32)
    s(l, "zbal_comm_get_device_status", i32, vp, P(u32 * 4))
    s(l, "zbal_all_reduce", i32, vp, vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp)
    s(l, "zbal_all_reduce_scaled", i32, vp, vp, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_float, vp, vp)
    s(l, "zbal_reduce_scatter", i32, vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp)
    s(l, "zbal_all_gather", i32, vp, vp, C.c_size_t, C.c_int, vp, vp)
    s(l, "zbal_all_to_all_v", i32, vp, vp, vp, u64, vp, vp)
    s(l, "zbal_broadcast", i32, vp, u64, C.c_int, C.c_uint16, vp, vp)
    s(l, "zbal_scatter", i32, vp, vp, u64, C.c_int, C.c_uint16, vp, vp)
    s(l, "zbal_gather", i32, vp, vp, u64, C.c_int, C.c_uint16, vp, vp)
    s(l, "zbal_barrier", i32, vp, vp)
    s(l, "zbal_send", i32, vp, C.c_size_t, C.c_int, u32, vp, vp)
    s(l, "zbal_moe_create", i32, vp, P(MoeOptionsC), P(vp))
    s(l, "zbal_moe_destroy", i32, vp)
    s(l, "zbal_moe_get_buffers", i32, vp, P(MoeBuffersC))
    s(l, "zbal_moe_get_status", i32, vp, P(i32))
    s(l, "zbal_dispatch_normal_layout", i32, vp, vp, i64, vp, vp, vp, vp, vp)
    s(l, "zbal_dispatch_normal_notify", i32, vp, vp, vp, vp, vp, vp, vp)
    s(l, "zbal_dispatch_normal", i32, vp, vp, i64, vp, vp, vp, vp, vp)
    s(l, "zbal_combine_normal", i32, vp, vp, i64, vp, i32, vp, i64, vp, vp)
    s(l, "zbal_dispatch_low_latency", i32, vp, vp, i64, vp, vp, vp, vp, vp, vp, vp, vp, vp)
    s(l, "zbal_combine_low_latency", i32, vp, vp, i64, vp, i32, vp, vp, i64, vp, vp)
    s(l, "zbal_fused_deep_moe_workspace", u64, vp, u32)
    s(l, "zbal_fused_deep_moe", i32, vp, vp, i64, vp, vp, vp, vp, vp, vp, u32, vp, vp, vp)
    s(l, "zbal_recv", i32, vp, C.c_size_t, C.c_int, u32, vp, vp)


def lib():
    global _declared
    l = N.lib()
    if not _declared:
        _declare(l)
        _declared = True
    return l


def last_error() -> str:
    return (lib().zbal_get_last_error_msg() or b"").decode(errors="replace")


class ZbalError(RuntimeError):
    def __init__(self, what: str, code: int):
        super().__init__(f"{what} failed ({code}): {last_error()}")
        self.code = code


def check(rc: int, what: str) -> None:
    if rc != Z_OK:
        raise ZbalError(what, rc)
