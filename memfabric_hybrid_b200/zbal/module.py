"""zbal life cycle and allocator control.

    zbal_init(world_size, device_id, rank_id, device_mem_size, ip_port="127.0.0.1:7000", start_config_server=True)
    with switch_to_allocator():           # tensors created here live in the symmetric heap
        x = torch.empty(...)
    zbal_uninit()

Parity: app/zbal/src/python/zbal/zbal_module.py:19-161 of the reference. Differences: the allocator switch
is a scoped ``torch.cuda.MemPool`` by default (PyTorch's native caching allocator asks zbal for its
segments), because a CUDA process can swap its global allocator only before the first allocation;
``switch_to_allocator(globally=True)`` does that swap and must be called first thing: before PyTorch initialises
CUDA (``torch.cuda.set_device`` already does) and before ``zbal_init``; allocations made before the heap exists fail. Under the
global allocator a ``torch.cuda.graph`` capture allocates from a private pool of the symmetric heap.
"""
from __future__ import annotations

import contextlib
import ctypes as C
import enum
import json
import os
from typing import Optional

import torch

from .. import _native as N
from . import _capi as K

__version__ = "1.0.0"


class ZBALBootstrapType(enum.IntEnum):
    BOOT_BY_MEMFABRIC = 0


_state = {"output": None, "allocator": None, "py_allocator": None, "pool": None, "global": False}


def zbal_set_logger_level(level: int) -> int:
    return K.lib().zbal_set_logger_level(level)


def is_initialized() -> bool:
    return bool(K.lib().zbal_is_bootstrapped())


def zbal_init(world_size: int, device_id: int, rank_id: int, device_mem_size: int,
              bootstrap_type: ZBALBootstrapType = ZBALBootstrapType.BOOT_BY_MEMFABRIC, start_config_server: bool = False,
              data_op_type: int = 0, comm_meta_space_size: int = 0, comm_group_cap: int = 16, flags: int = 0, ip_port: str = "") -> bool:
    """Collective over all ranks. ``comm_meta_space_size`` is in KiB per communicator (0 = derive from the slice).
    ``ip_port`` defaults to $ZBAL_IP_PORT or MASTER_ADDR:(MASTER_PORT + 7); rank 0 hosts the store when
    ``start_config_server`` is set or no address was given. Returns True on success."""
    l = K.lib()
    if torch.cuda.is_available():
        N.cuda()  # kernels and the CUDA device backend
        torch.cuda.set_device(device_id)
        torch.cuda.synchronize()  # a context must exist before the VMM calls (no allocation: the heap may be the allocator)
    auto = False
    if not ip_port:
        ip_port = os.environ.get("ZBAL_IP_PORT", "")
    if not ip_port:
        ip_port = f"{os.environ.get('MASTER_ADDR', '127.0.0.1')}:{int(os.environ.get('MASTER_PORT', '29500')) + 7}"
        auto = True
    if "://" not in ip_port:
        ip_port = "tcp://" + ip_port
    o = K.BootstrapOptionsC()
    l.zbal_bootstrap_options_init(C.byref(o))
    o.flags = flags
    o.btType = int(bootstrap_type)
    o.ipPort = ip_port.encode()
    o.worldSize, o.rankId, o.deviceId = world_size, rank_id, device_id
    o.startConfigServer = bool(start_config_server or auto)
    o.deviceMemorySize = device_mem_size
    o.dataOperationType = data_op_type
    o.commMetaSpaceSize = comm_meta_space_size << 10
    o.commGroupCap = comm_group_cap
    out = K.BootstrapOutputC()
    rc = l.zbal_bootstrap(C.byref(o), C.byref(out))
    if rc != K.Z_OK:
        raise K.ZbalError("zbal_bootstrap", rc)
    _state["output"] = out
    if torch.cuda.is_available():
        from ..utils import devtrace
        devtrace.enable_from_env()  # ZBAL_PROF_ENABLE=1: device timeline, written at exit and on SIGUSR1
    return True


def zbal_uninit(flags: int = 0) -> bool:
    l = K.lib()
    if not l.zbal_is_bootstrapped():
        return False
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    from . import process_group
    process_group._forget_all()
    _state["pool"] = None
    l.zbal_comm_destroy_all(flags)
    l.zbal_unbootstrap(flags)
    _state["output"] = None
    return True


def bootstrap_output() -> K.BootstrapOutputC:
    out = K.BootstrapOutputC()
    K.check(K.lib().zbal_bootstrap_get_output(C.byref(out)), "zbal_bootstrap_get_output")
    return out


def zbal_get_symm_base_addr() -> int:
    """Start of this rank's allocator heap (device address)."""
    return int(bootstrap_output().heapGva)


def _native():
    from . import process_group
    return process_group.native_extension()


def _pluggable():
    """The torch._C allocator object over zbal_pluggable_malloc / free. With the native extension it also carries the
    CUDA-graph hooks (private pools: csrc/c10d/zbal_torch_allocator.cpp); the Python-only fallback has malloc / free."""
    if _state["allocator"] is None:
        K.lib()
        ext = _native()
        if ext is not None:
            _state["allocator"] = ext.allocator()
        else:
            path = str(N._LIB_DIR / "libmf_smem.so")
            _state["py_allocator"] = torch.cuda.memory.CUDAPluggableAllocator(path, "zbal_pluggable_malloc", "zbal_pluggable_free")
            _state["allocator"] = _state["py_allocator"].allocator()
    return _state["allocator"]


def switch_to_allocator(globally: bool = False):
    """Routes tensor allocations to the symmetric heap.

    Default: returns a context manager; allocations made inside come from a ``torch.cuda.MemPool`` whose
    segments zbal provides. ``globally=True`` replaces the process-wide allocator instead (only possible
    before the first CUDA allocation of the process) and returns None."""
    alloc = _pluggable()
    if globally:
        ext = _native()
        if ext is not None:
            ext.install_global_allocator()   # CUDA graphs captured from here on get private pools of the symmetric heap
        else:
            torch.cuda.memory.change_current_allocator(_state["py_allocator"])
        _state["global"] = True
        return None
    if _state["pool"] is None:
        _state["pool"] = torch.cuda.MemPool(alloc)
    return torch.cuda.use_mem_pool(_state["pool"])


@contextlib.contextmanager
def symmetric_tensors():
    """Alias of ``switch_to_allocator()`` that reads better at call sites."""
    with switch_to_allocator():
        yield


def in_symmetric_heap(t: torch.Tensor) -> bool:
    out = _state["output"]
    if out is None or not t.is_cuda:
        return False
    p = t.data_ptr()
    if out.heapGva <= p < out.heapGva + out.heapSize:
        return True
    return bool(K.lib().zbal_is_symmetric(p, max(1, t.numel() * t.element_size())))   # expansion segments


def expand_heap() -> tuple:
    """Collective: one more segment of ``device_memory_size`` bytes per rank for the symmetric heap; every rank calls it
    at the same point. -> (address of this rank's part of the new segment, its size). With
    ``ZBAL_ALLOC_CONF=expandable_segments:True`` the allocator does this by itself when a request does not fit."""
    base, size = C.c_uint64(), C.c_uint64()
    K.check(K.lib().zbal_heap_expand(C.byref(base), C.byref(size)), "zbal_heap_expand")
    return int(base.value), int(size.value)


def get_heap_stats():
    """(bytes in use, heap size)."""
    s = K.SmaStatsC()
    K.check(K.lib().zbal_sma_get_stats(C.byref(s)), "zbal_sma_get_stats")
    return int(s.inUseBytes), int(s.heapSize)


def heap_stats() -> dict:
    s = K.SmaStatsC()
    K.check(K.lib().zbal_sma_get_stats(C.byref(s)), "zbal_sma_get_stats")
    return {n: int(getattr(s, n)) for n, _ in K.SmaStatsC._fields_}


def mem_get_info():
    """(free, total) of the symmetric heap, the shape of ``torch.cuda.mem_get_info``."""
    used, total = get_heap_stats()
    return total - used, total


def empty_cache(check_error: bool = False) -> None:
    K.lib().zbal_pluggable_empty_cache(check_error)


def record_memory_history(enabled=True, max_entries: int = 65536) -> None:
    """Starts (any true value: True, "all", "state") or stops (False / None) recording the allocator's malloc / free history."""
    K.lib().zbal_sma_record_history(bool(enabled), max(0, min(int(max_entries), 0xFFFFFFFF)))


def snapshot() -> dict:
    """The allocator's own snapshot: heap settings, address segments, every block with its state, the recorded history."""
    l = K.lib()
    need = l.zbal_sma_snapshot(None, 0)
    if need <= 0:
        raise K.ZbalError("zbal_sma_snapshot", int(need))
    buf = C.create_string_buffer(int(need) + 64)
    l.zbal_sma_snapshot(buf, len(buf))
    return json.loads(buf.value.decode())


def memviz_snapshot(snap: Optional[dict] = None) -> dict:
    """The snapshot in the layout of PyTorch's memory visualiser (``torch.cuda.memory._snapshot()``): ``segments`` (one per
    address segment of the heap, each with its blocks in address order) and ``device_traces`` (one list per device:
    segment_alloc for every segment, then alloc / free_requested / free_completed / empty_cache / oom from the recorded
    history). Pickle it and open it at pytorch.org/memory_viz, or feed it to ``zbal.snapshot_utils``.
    Parity: app/zbal/src/csrc/sma/zbal_sma_pybind.cpp:21-150 of the reference."""
    snap = snap if snap is not None else snapshot()
    heap = snap["heap"]
    dev = int(heap.get("device", 0))
    regions = snap.get("segments") or [{"base": heap["base"], "size": heap["size"]}]
    state = {"active": "active_allocated", "cached": "inactive", "free": "inactive"}
    segments, trace = [], []
    blocks = sorted(snap["blocks"], key=lambda b: b["addr"])
    for r in sorted(regions, key=lambda r: r["base"]):
        lo, hi = r["base"], r["base"] + r["size"]
        mine = [b for b in blocks if lo <= b["addr"] < hi]
        active = sum(b["size"] for b in mine if b["state"] == "active")
        segments.append({"device": dev, "address": lo, "total_size": r["size"], "allocated_size": active, "active_size": active,
                         "requested_size": active, "stream": 0, "segment_type": "large", "segment_pool_id": 0, "is_expandable": False,
                         "frames": [], "blocks": [{"address": b["addr"], "size": b["size"], "requested_size": b["size"],
                                                   "state": state[b["state"]], "frames": []} for b in mine]})
    for r in regions:   # in the order the heap got them
        trace.append({"action": "segment_alloc", "addr": r["base"], "size": r["size"], "stream": 0})
    for ev in snap.get("history", []):
        op = ev["op"]
        if op in ("malloc_heap", "malloc_cache"):
            trace.append({"action": "alloc", "addr": ev["addr"], "size": ev["size"], "stream": ev["stream"]})
        elif op in ("free_cache", "free_heap"):
            trace.append({"action": "free_requested", "addr": ev["addr"], "size": ev["size"], "stream": ev["stream"]})
            trace.append({"action": "free_completed", "addr": ev["addr"], "size": ev["size"], "stream": ev["stream"]})
        elif op == "empty_cache":
            trace.append({"action": "empty_cache", "addr": 0, "size": 0, "stream": 0})
        elif op == "malloc_failed":
            trace.append({"action": "oom", "device_free": heap["size"] - heap.get("in_use", 0), "size": ev.get("requested", ev["size"]),
                          "stream": ev["stream"]})
    traces = [[] for _ in range(dev)] + [trace]
    return {"segments": segments, "device_traces": traces}


def dump_snapshot(path: Optional[str] = None):
    """Without a path: returns the snapshot in the memory visualiser's layout (the reference's call). With a path: writes
    it there, a ``.pkl`` / ``.pickle`` file in the visualiser's layout, anything else as JSON in the allocator's own layout
    (what ``python -m memfabric_hybrid_b200.zbal.simulator`` reads)."""
    if path is None:
        return memviz_snapshot()
    if path.endswith((".pkl", ".pickle")):
        import pickle
        with open(path, "wb") as f:
            pickle.dump(memviz_snapshot(), f)
        return None
    with open(path, "w") as f:
        json.dump(snapshot(), f)
    return None


def simulate_init(addr: int, size: int) -> None:
    """Runs the allocator over a made-up address range (no device): for replaying traces offline."""
    K.lib().zbal_simulate_init(addr, size)


def is_mix_alloc() -> bool:
    """True when a symmetric pool is in use next to PyTorch's own allocator."""
    return _state["pool"] is not None
