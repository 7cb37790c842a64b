"""``memfabric_hybrid.bm``: Big Memory pools (see csrc/include/smem_bm.h for the C contract)."""
from __future__ import annotations

import ctypes as C
import enum
import threading
from typing import Callable, Sequence

from .. import _native as N


class BmMemType(enum.IntEnum):
    LOCAL_DEVICE = 0
    LOCAL_HOST = 1
    DEVICE = 2
    HOST = 3


class BmCopyType(enum.IntEnum):
    L2G = 0
    G2L = 1
    G2H = 2
    H2G = 3
    L2GH = 4
    GH2L = 5
    GH2H = 6
    H2GH = 7
    G2G = 8
    AUTO = 9


class BmDataOpType(enum.IntFlag):
    SDMA = 1 << 0
    HOST_RDMA = 1 << 1
    HOST_TCP = 1 << 2
    DEVICE_RDMA = 1 << 3
    HOST_URMA = 1 << 4
    HOST_SHM = 1 << 5
    DEVICE_URMA = 1 << 6


class BmGroupEvent(enum.IntEnum):
    JOIN_EVENT = 0
    LEAVE_EVENT = 1


_TLS = threading.local()

ASYNC_COPY_FLAG = 1 << 0
COPY_EXTEND_FLAG = 1 << 1
FLAG_USE_EXTERNAL_STREAM = 1 << 2


class BmConfig:
    """Mirror of ``smem_bm_config_t`` with the reference's Python attribute names."""

    _MAP = {"init_timeout": "initTimeout", "create_timeout": "createTimeout",
            "operation_timeout": "controlOperationTimeout", "start_store": "startConfigStoreServer",
            "start_store_only": "startConfigStoreOnly", "dynamic_world_size": "dynamicWorldSize",
            "unified_address_space": "unifiedAddressSpace", "auto_ranking": "autoRanking", "rank_id": "rankId",
            "flags": "flags"}

    def __init__(self) -> None:
        object.__setattr__(self, "_c", N.BmConfigC())
        N.lib().smem_bm_config_init(C.byref(self._c))

    def __getattr__(self, name):
        if name in BmConfig._MAP:
            return getattr(self._c, BmConfig._MAP[name])
        raise AttributeError(name)

    def __setattr__(self, name, value):
        if name in BmConfig._MAP:
            setattr(self._c, BmConfig._MAP[name], value)
        else:
            raise AttributeError(name)

    def set_nic(self, nic: str) -> None:
        self._c.hcomUrl = nic.encode()[:63]


def initialize(store_url: str, world_size: int, device_id: int, config: BmConfig) -> int:
    return N.lib().smem_bm_init(store_url.encode(), world_size, device_id, C.byref(config._c))


def uninitialize(flags: int = 0) -> None:
    N.lib().smem_bm_uninit(flags)


def bm_rank_id() -> int:
    return N.lib().smem_bm_get_rank_id()


def _ptr_array(values: Sequence[int]):
    return (C.c_void_p * len(values))(*[int(v) for v in values])


def _u64_view(values, n: int, ctype):
    """``values`` as a C array of ``n`` 64-bit words plus the object that keeps it alive. A contiguous numpy array of
    64-bit integers is passed as it is (no copy: the cost of a call on a large descriptor list is then the C call
    alone); any other sequence is converted once."""
    import numpy as np
    a = values if isinstance(values, np.ndarray) else np.asarray(values[:n], dtype=np.uint64)
    if a.dtype not in (np.uint64, np.int64) or not a.flags["C_CONTIGUOUS"]:
        a = np.ascontiguousarray(a, dtype=np.uint64)
    if a.shape[0] < n:
        raise ValueError(f"batch of {n} items but only {a.shape[0]} values")
    return a.ctypes.data_as(C.POINTER(ctype)), a


class _QuantParamsC(C.Structure):   # hybm_quant_copy_params
    _fields_ = [("sources", C.POINTER(C.c_void_p)), ("destinations", C.POINTER(C.c_void_p)), ("dataSizes", C.POINTER(C.c_uint64)),
                ("scale", C.POINTER(C.c_void_p)), ("offset", C.POINTER(C.c_void_p)), ("batchSize", C.c_uint32), ("unitNum", C.c_uint32),
                ("stream", C.c_void_p), ("inputType", C.c_uint32), ("flags", C.c_uint32)]


class BigMemory:
    def __init__(self, handle: int):
        self._h = handle
        self._cb = None

    # -- membership
    def join(self, flags: int = 0) -> int:
        return N.lib().smem_bm_join(self._h, flags)

    def leave(self, flags: int = 0) -> int:
        return N.lib().smem_bm_leave(self._h, flags)

    def extend_local_mem(self, mem_type: BmMemType = BmMemType.HOST, size: int = 0) -> int:
        return N.lib().smem_bm_extend_local_mem(self._h, int(mem_type), size)

    def set_group_event_handler(self, cb: Callable[[int, BmGroupEvent], None]) -> int:
        def tramp(_h, rank, ev, _ctx):
            cb(rank, BmGroupEvent(ev))
        self._cb = N.BM_EVENT_FN(tramp)
        return N.lib().smem_bm_set_group_event_handler(self._h, self._cb, None)

    # -- addressing
    def local_mem_size(self, mem_type: BmMemType = BmMemType.DEVICE) -> int:
        return N.lib().smem_bm_get_local_mem_size_by_mem_type(self._h, int(mem_type))

    def peer_rank_ptr(self, peer_rank: int, mem_type: BmMemType = BmMemType.DEVICE) -> int:
        return N.lib().smem_bm_ptr_by_mem_type(self._h, int(mem_type), peer_rank) or 0

    def gva_to_va(self, gva: int, mem_type: BmMemType = BmMemType.LOCAL_HOST) -> int:
        out = C.c_void_p()
        rc = N.lib().smem_bm_gva_to_va(self._h, gva, int(mem_type), C.byref(out))
        return (out.value or 0) if rc == 0 else 0

    def get_rank_id_by_gva(self, gva: int) -> int:
        return N.lib().smem_bm_get_rank_id_by_gva(self._h, gva)

    def register(self, addr: int, size: int) -> int:
        return N.lib().smem_bm_register_user_mem(self._h, addr, size)

    def unregister(self, addr: int) -> int:
        return N.lib().smem_bm_unregister_user_mem(self._h, addr)

    # -- data
    def copy_data(self, src_ptr: int, dst_ptr: int, size: int, type: BmCopyType, flags: int = 0, stream: int = 0) -> int:
        """One copy. Without ``FLAG_USE_EXTERNAL_STREAM`` it runs on the pool's own non-blocking stream, which is
        not ordered with PyTorch's streams: a tensor that a PyTorch kernel is still filling (``torch.zeros``,
        ``randn``, the output of a layer) must be complete first (synchronise its stream), or pass that stream
        with the flag so that the copy is enqueued behind the producer."""
        tl = _TLS
        p = getattr(tl, "copy_params", None)
        if p is None:     # one parameter block per thread: the call releases the GIL, so threads must not share one
            p = tl.copy_params = N.CopyParamsC()
            tl.copy_ref = C.byref(p)
            tl.copy_fn = N.lib().smem_bm_copy
        p.src, p.dest, p.dataSize, p.stream = src_ptr, dst_ptr, size, stream or None
        return tl.copy_fn(self._h, tl.copy_ref, int(type), flags)

    def _batch(self, src_addrs, dst_addrs, sizes, count, stream):
        n = int(count)
        srcs, k0 = _u64_view(src_addrs, n, C.c_void_p)
        dsts, k1 = _u64_view(dst_addrs, n, C.c_void_p)
        lens, k2 = _u64_view(sizes, n, C.c_uint64)
        p = N.BatchCopyParamsC(srcs, dsts, lens, n, stream or None)
        return p, (k0, k1, k2)

    def copy_data_batch(self, src_addrs, dst_addrs, sizes, count, type: BmCopyType, flags: int = 0, stream: int = 0) -> int:
        """``smem_bm_copy_batch``. The three lists may be any sequences of integers; contiguous numpy arrays of
        uint64 / int64 are handed to the C call without conversion."""
        p, _keep = self._batch(src_addrs, dst_addrs, sizes, count, stream)
        return N.lib().smem_bm_copy_batch(self._h, C.byref(p), int(type), flags)

    def prepare_batch(self, src_addrs, dst_addrs, sizes, count=None):
        """Extension: marshals a batch once so that repeated submissions skip the Python-side conversion (every submission
        still runs the library's validation and descriptor marshalling: see ``create_batch`` for the path that does not)."""
        n = int(count if count is not None else len(sizes))
        return self._batch(src_addrs, dst_addrs, sizes, n, 0)

    def copy_prepared(self, prepared, type: BmCopyType, flags: int = 0, stream: int = 0) -> int:
        p, _keep = prepared
        p.stream = stream or None
        return N.lib().smem_bm_copy_batch(self._h, C.byref(p), int(type), flags)

    def create_batch(self, src_addrs, dst_addrs, sizes, type: BmCopyType, count=None) -> "PreparedBatch":
        """Extension (``mf_bm_batch_create``): a device-to-device batch (L2G, G2L, G2G) validated, merged and cut into work
        chunks ONCE, with its descriptors in pinned memory of its own. ``launch(stream)`` is then a single kernel launch that
        may be recorded into a CUDA graph. Re-create it after a member of the pool leaves."""
        n = int(count if count is not None else len(sizes))
        p, _keep = self._batch(src_addrs, dst_addrs, sizes, n, 0)
        out = C.c_void_p()
        l = N.lib()
        l.mf_bm_batch_create.restype = C.c_int32
        l.mf_bm_batch_create.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_void_p)]
        rc = l.mf_bm_batch_create(self._h, C.byref(p), int(type), C.byref(out))
        if rc != 0:
            raise RuntimeError(f"mf_bm_batch_create failed ({rc}): {N.last_error()}")
        return PreparedBatch(out.value)

    def copy_data_batch_partial_succeed(self, src_addrs, dst_addrs, sizes, count, type: BmCopyType, flags: int = 0,
                                        stream: int = 0):
        """Returns (code, per-item list of codes)."""
        p, _keep = self._batch(src_addrs, dst_addrs, sizes, count, stream)
        res = (C.c_int32 * int(count))()
        r = N.BatchCopyResultC(res, int(count))
        rc = N.lib().smem_bm_copy_batch_partial_succeed(self._h, C.byref(p), int(type), flags, C.byref(r))
        return rc, list(res)

    def wait(self) -> int:
        return N.lib().smem_bm_wait(self._h)

    def prepare_quant_batch(self, src_addrs, dst_addrs, sizes, scale_addrs, unit: int, fp8: bool = False, fp16_input: bool = False):
        """Extension: marshals a quantising batch once (see ``quant_copy_batch``) for repeated submission."""
        n = len(sizes)
        keep = (_ptr_array(src_addrs[:n]), _ptr_array(dst_addrs[:n]), (C.c_uint64 * n)(*[int(v) for v in sizes]), _ptr_array(scale_addrs[:n]),
                _ptr_array([0] * n))
        p = _QuantParamsC(keep[0], keep[1], keep[2], keep[3], keep[4], n, unit, None, 1 if fp16_input else 0, 1 if fp8 else 0)
        return p, keep

    def quant_copy_prepared(self, prepared, stream: int = 0) -> int:
        p, _keep = prepared
        p.stream = stream or None
        f = N.lib().mf_bm_quant_copy
        f.restype, f.argtypes = C.c_int32, [C.c_void_p, C.c_void_p]
        return f(self._h, C.byref(p))

    def quant_copy_batch(self, src_addrs, dst_addrs, sizes, scale_addrs, unit: int, fp8: bool = False, fp16_input: bool = False,
                         stream: int = 0) -> int:
        """Extension: quantise-while-copy. ``sizes`` are the SOURCE bytes (bf16, or fp16 with ``fp16_input``); each item
        writes ``size / 2`` quantised bytes to its destination and one fp32 dequantisation factor per ``unit`` elements
        to its scale address. int8 by default; ``fp8=True``: e4m3 with ``unit`` 128. Destinations may be peer slices.
        Without a stream the call returns when the data has arrived."""
        return self.quant_copy_prepared(self.prepare_quant_batch(src_addrs, dst_addrs, sizes, scale_addrs, unit, fp8, fp16_input), stream)

    def copy_stats(self) -> dict:
        """Counters of the copy paths (extension): kernel launches/chunks, engine, host, process-VM copies."""
        out = (C.c_uint64 * 6)()
        f = N.lib().mf_bm_copy_stats
        f.restype, f.argtypes = C.c_int32, [C.c_void_p, C.POINTER(C.c_uint64)]
        f(self._h, out)
        keys = ("kernel_launches", "kernel_chunks", "engine_copies", "host_copies", "vm_copies", "coalesced")
        return dict(zip(keys, [int(v) for v in out]))

    def destroy(self) -> None:
        if self._h:
            N.lib().smem_bm_destroy(self._h)
            self._h = None

    @property
    def handle(self) -> int:
        return self._h


class PreparedBatch:
    """Handle of ``BigMemory.create_batch``."""

    def __init__(self, handle: int):
        self._b = handle
        l = N.lib()
        l.mf_bm_batch_launch.restype = C.c_int32
        l.mf_bm_batch_launch.argtypes = [C.c_void_p, C.c_void_p]
        l.mf_bm_batch_bytes.restype = C.c_uint64
        l.mf_bm_batch_bytes.argtypes = [C.c_void_p]
        l.mf_bm_batch_destroy.restype = C.c_int32
        l.mf_bm_batch_destroy.argtypes = [C.c_void_p]
        self._launch = l.mf_bm_batch_launch

    def launch(self, stream: int) -> int:
        """Enqueues the batch on ``stream`` (asynchronous; capturable)."""
        return self._launch(self._b, stream or None)

    @property
    def nbytes(self) -> int:
        return int(N.lib().mf_bm_batch_bytes(self._b))

    def destroy(self) -> None:
        if self._b:
            N.lib().mf_bm_batch_destroy(self._b)
            self._b = None


def create(id: int, local_dram_size: int, local_hbm_size: int = 0, data_op_type: BmDataOpType = BmDataOpType.SDMA,
           flags: int = 0) -> BigMemory:
    h = N.lib().smem_bm_create(id, 0, int(data_op_type), local_dram_size, local_hbm_size, flags)
    if not h:
        raise RuntimeError("bm.create failed: " + N.last_error())
    return BigMemory(h)


def create2(id: int, local_dram_size: int, max_dram_size: int, local_hbm_size: int = 0, max_hbm_size: int = 0,
            data_op_type: BmDataOpType = BmDataOpType.SDMA, enable_56bits_gva: bool = False, flags: int = 0,
            shm_fd: int = -1) -> BigMemory:
    o = N.BmCreateOptionC()
    o.maxDramSize, o.maxHbmSize = max_dram_size, max_hbm_size
    o.localDRAMSize, o.localHBMSize = local_dram_size, local_hbm_size
    o.dataOpType = int(data_op_type)
    o.enable56BitsGva = enable_56bits_gva
    o.flags = flags
    o.dramShmFd = shm_fd
    h = N.lib().smem_bm_create2(id, C.byref(o))
    if not h:
        raise RuntimeError("bm.create2 failed: " + N.last_error())
    return BigMemory(h)
