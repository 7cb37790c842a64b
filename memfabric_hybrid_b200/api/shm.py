"""``memfabric_hybrid.shm``: symmetric shared memory (see csrc/include/smem_shm.h for the C contract)."""
from __future__ import annotations

import ctypes as C
import enum

from .. import _native as N


@N.register_decls
def _decls(l):
    P = C.POINTER
    N._sig(l, "smem_shm_config_init", N.i32, P(N.ShmConfigC))
    N._sig(l, "smem_shm_init", N.i32, N.cp, N.u32, N.u32, N.u16, P(N.ShmConfigC))
    N._sig(l, "smem_shm_uninit", None, N.u32)
    N._sig(l, "smem_shm_query_support_data_operation", N.u32)
    N._sig(l, "smem_shm_create", N.vp, N.u32, N.u32, N.u32, N.u64, C.c_int, N.u32, P(N.vp))
    N._sig(l, "smem_shm_get_symmetric_size", N.u64, N.vp)
    N._sig(l, "smem_shm_destroy", N.i32, N.vp, N.u32)
    N._sig(l, "smem_shm_set_extra_context", N.i32, N.vp, N.cp, N.u32)
    N._sig(l, "smem_shm_get_global_rank", N.u32, N.vp)
    N._sig(l, "smem_shm_get_global_rank_size", N.u32, N.vp)
    N._sig(l, "smem_shm_control_barrier", N.i32, N.vp)
    N._sig(l, "smem_shm_control_allgather", N.i32, N.vp, N.cp, N.u32, C.c_char_p, N.u32)
    N._sig(l, "smem_shm_subgroup_barrier", N.i32, N.vp, N.cp, N.u32, N.u32)
    N._sig(l, "smem_shm_subgroup_allgather", N.i32, N.vp, N.cp, N.u32, N.u32, N.cp, N.u32, C.c_char_p, N.u32)
    N._sig(l, "smem_shm_topology_can_reach", N.i32, N.vp, N.u32, P(N.u32))
    N._sig(l, "smem_shm_atomic_alloc_value", N.i32, N.vp, N.u32, P(N.i32))
    N._sig(l, "smem_shm_atomic_release_value", N.i32, N.vp, N.i32)
    N._sig(l, "smem_shm_register_exit", N.i32, N.vp, N.EXIT_FN)
    N._sig(l, "smem_shm_global_exit", None, N.vp, C.c_int)
    N._sig(l, "smem_shm_get_device_context", N.i32, N.vp, N.vp, N.u32)


class ShmDataOpType(enum.IntFlag):
    MTE = 1 << 0
    SDMA = 1 << 1
    RDMA = 1 << 2


class ShmConfig:
    _MAP = {"init_timeout": "shmInitTimeout", "create_timeout": "shmCreateTimeout",
            "operation_timeout": "controlOperationTimeout", "start_store": "startConfigStoreServer", "flags": "flags"}

    def __init__(self) -> None:
        object.__setattr__(self, "_c", N.ShmConfigC())
        N.lib().smem_shm_config_init(C.byref(self._c))

    def __getattr__(self, name):
        if name in ShmConfig._MAP:
            return getattr(self._c, ShmConfig._MAP[name])
        raise AttributeError(name)

    def __setattr__(self, name, value):
        if name not in ShmConfig._MAP:
            raise AttributeError(name)
        setattr(self._c, ShmConfig._MAP[name], value)


def initialize(store_url: str, world_size: int, rank_id: int, device_id: int, config: ShmConfig) -> int:
    return N.lib().smem_shm_init(store_url.encode(), world_size, rank_id, device_id, C.byref(config._c))


def uninitialize(flags: int = 0) -> None:
    N.lib().smem_shm_uninit(flags)


class ShmDeviceContext(C.Structure):
    """Mirror of ``smem_shm_device_ctx_t``."""
    _fields_ = [("base", C.c_uint64), ("symmetric_size", C.c_uint64), ("mc_base", C.c_uint64), ("rank", C.c_uint32),
                ("rank_size", C.c_uint32), ("reserved", C.c_uint32), ("spin_limit", C.c_uint32)]


USER_OFFSET = 1 << 20  # the first MiB of every slice holds the flags of the device API


class ShareMemory:
    def __init__(self, handle: int, gva: int):
        self._h = handle
        self._gva = gva
        self._exit_cb = None

    def set_context(self, context: bytes) -> int:
        return N.lib().smem_shm_set_extra_context(self._h, context, len(context))

    @property
    def local_rank(self) -> int:
        return N.lib().smem_shm_get_global_rank(self._h)

    @property
    def rank_size(self) -> int:
        return N.lib().smem_shm_get_global_rank_size(self._h)

    @property
    def gva(self) -> int:
        """Start of the whole symmetric range; rank r's slice is at gva + r * symmetric_size."""
        return self._gva

    @property
    def symmetric_size(self) -> int:
        return N.lib().smem_shm_get_symmetric_size(self._h)

    def destroy(self, flags: int = 0) -> int:
        if not self._h:
            return 0
        rc = N.lib().smem_shm_destroy(self._h, flags)
        self._h = None
        return rc

    def query_support_data_operation(self) -> int:
        return N.lib().smem_shm_query_support_data_operation()

    def barrier(self) -> int:
        return N.lib().smem_shm_control_barrier(self._h)

    def all_gather(self, local_data: bytes) -> bytes:
        n = len(local_data) * self.rank_size
        out = C.create_string_buffer(n)
        rc = N.lib().smem_shm_control_allgather(self._h, local_data, len(local_data), out, n)
        if rc != 0:
            raise RuntimeError(f"all_gather failed ({rc}): {N.last_error()}")
        return out.raw

    def subgroup_barrier(self, key: str, rank_size: int, rank_id: int) -> int:
        return N.lib().smem_shm_subgroup_barrier(self._h, key.encode(), rank_size, rank_id)

    def subgroup_all_gather(self, key: str, rank_size: int, rank_id: int, local_data: bytes) -> bytes:
        n = len(local_data) * rank_size
        out = C.create_string_buffer(n)
        rc = N.lib().smem_shm_subgroup_allgather(self._h, key.encode(), rank_size, rank_id, local_data, len(local_data), out, n)
        if rc != 0:
            raise RuntimeError(f"subgroup_all_gather failed ({rc}): {N.last_error()}")
        return out.raw

    def topology_can_reach(self, remote_rank: int, reach_info: int = 0) -> int:
        out = N.u32(reach_info)
        rc = N.lib().smem_shm_topology_can_reach(self._h, remote_rank, C.byref(out))
        return rc if rc != 0 else out.value

    def atomic_alloc_value(self, limit: int) -> int:
        v = N.i32(-1)
        rc = N.lib().smem_shm_atomic_alloc_value(self._h, limit, C.byref(v))
        if rc != 0:
            raise RuntimeError(f"atomic_alloc_value failed ({rc}): {N.last_error()}")
        return v.value

    def atomic_release_value(self, value: int) -> int:
        return N.lib().smem_shm_atomic_release_value(self._h, value)

    def device_context(self) -> "ShmDeviceContext":
        """The block a kernel takes by value to use the device API (csrc/include/smem_shm_device.cuh)."""
        ctx = ShmDeviceContext()
        rc = N.lib().smem_shm_get_device_context(self._h, C.byref(ctx), C.sizeof(ctx))
        if rc != 0:
            raise RuntimeError(f"smem_shm_get_device_context failed ({rc}): {N.last_error()}")
        return ctx

    def register_exit(self, fn) -> int:
        self._exit_cb = N.EXIT_FN(fn)
        return N.lib().smem_shm_register_exit(self._h, self._exit_cb)

    def global_exit(self, status: int) -> None:
        N.lib().smem_shm_global_exit(self._h, status)


def create(id: int, rank_size: int, rank_id: int, local_mem_size: int, data_op_type: ShmDataOpType = ShmDataOpType.MTE,
           flags: int = 0) -> ShareMemory:
    gva = C.c_void_p()
    h = N.lib().smem_shm_create(id, rank_size, rank_id, local_mem_size, int(data_op_type), flags, C.byref(gva))
    if not h:
        raise RuntimeError("shm.create failed: " + N.last_error())
    return ShareMemory(h, gva.value or 0)
