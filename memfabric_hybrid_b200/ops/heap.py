"""Symmetric heaps for the device kernels.

``SymmetricHeap``  — the real thing: one ``smem_shm`` object per process group; every rank's slice is
mapped by all ranks at ``base + r * stride`` (NVLink peer mapping through CUDA VMM).
``EmulatedHeap``   — all "ranks" live in one allocation of one GPU and every kernel is launched once
over all of them (rank = blockIdx.y, cooperative launch). Used to test the multi-rank protocols on a
single device, where ranks must never be separate launches.

Slot layout (both): [signal area, 1 MiB][bump-allocated objects ...]. Allocation is a deterministic
bump pointer, so objects allocated in the same order have the same offset on every rank.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N

SIGNAL_BYTES = 1 << 20


class TeamC(C.Structure):
    _fields_ = [("heap_base", C.c_uint64), ("stride", C.c_uint64), ("mc_base", C.c_uint64), ("rank", C.c_uint32),
                ("world", C.c_uint32), ("emu", C.c_uint32), ("spin_limit", C.c_uint32)]


class _RawCuda:
    """Minimal __cuda_array_interface__ carrier so that torch can wrap a raw device address."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def tensor_at(ptr: int, shape, dtype: torch.dtype, device=None) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    raw = torch.as_tensor(_RawCuda(ptr, max(nbytes, 1)), device=dev)
    return raw[:nbytes].view(dtype).view(*shape)


class _HeapBase:
    base: int
    stride: int
    rank: int
    world: int
    emu: bool

    def __init__(self):
        self._top = SIGNAL_BYTES
        self.spin_limit = 1 << 22  # ~1-2 s of polling before a wait gives up
        self.mc_base = 0

    def alloc(self, nbytes: int, align: int = 256) -> int:
        """Returns the slot offset of a new object (identical on every rank when called in the same order)."""
        off = (self._top + align - 1) // align * align
        if off + nbytes > self.stride:
            raise MemoryError(f"symmetric heap exhausted: need {nbytes} at {off}, slot has {self.stride}")
        self._top = off + nbytes
        return off

    def mark(self) -> int:
        return self._top

    def release_to(self, mark: int) -> None:
        self._top = mark

    def ptr(self, rank: int, off: int = 0) -> int:
        return self.base + rank * self.stride + off

    def view(self, off: int, shape, dtype: torch.dtype, rank: int | None = None) -> torch.Tensor:
        r = self.rank if rank is None else rank
        return tensor_at(self.ptr(r, off), shape, dtype)

    def team(self) -> TeamC:
        return TeamC(self.base, self.stride, self.mc_base, self.rank, self.world, 1 if self.emu else 0, self.spin_limit)

    def status(self, rank: int | None = None):
        """(code, where, epoch, count) from the status words of a slot; code 0 means no wait ever gave up."""
        t = self.view(0, (4,), torch.int32, rank).cpu().tolist()
        return tuple(int(v) & 0xFFFFFFFF for v in t)

    def clear_status(self, rank: int | None = None) -> None:
        self.view(0, (4,), torch.int32, rank).zero_()


class EmulatedHeap(_HeapBase):
    def __init__(self, world: int, slot_bytes: int, device: int = 0):
        super().__init__()
        self.world, self.rank, self.emu = world, 0, True
        self.stride = (slot_bytes + 4095) // 4096 * 4096
        self._buf = torch.zeros(world * self.stride, dtype=torch.uint8, device=f"cuda:{device}")
        self.base = self._buf.data_ptr()


class SymmetricHeap(_HeapBase):
    """Symmetric heap of a process group, bootstrapped through the config store (``smem_shm``)."""

    _inited = False

    def __init__(self, store_url: str, world: int, rank: int, device: int, slot_bytes: int, shm_id: int = 0,
                 timeout_s: int = 120):
        super().__init__()
        from ..api import shm
        import memfabric_hybrid_b200.api as mf
        N.cuda()
        torch.cuda.set_device(device)
        torch.zeros(1, device="cuda")  # context
        mf.initialize()
        if not SymmetricHeap._inited:
            cfg = shm.ShmConfig()
            cfg.start_store = rank == 0
            cfg.init_timeout = timeout_s
            cfg.create_timeout = timeout_s
            cfg.operation_timeout = timeout_s
            rc = shm.initialize(store_url, world, rank, device, cfg)
            if rc != 0:
                raise RuntimeError(f"shm.initialize failed ({rc}): {mf.get_last_err_msg()}")
            SymmetricHeap._inited = True
        self._shm = shm.create(shm_id, world, rank, slot_bytes)
        self.world, self.rank, self.emu = world, rank, False
        self.base = self._shm.gva
        self.stride = self._shm.symmetric_size
        self.usable = slot_bytes
        self.mc_base = int(self._shm.device_context().mc_base)  # multicast alias of a slice, 0 unless MF_SHM_MULTICAST=1 took effect
        # the signal area must start at zero on every rank before anybody signals
        self.view(0, (SIGNAL_BYTES,), torch.uint8).zero_()
        torch.cuda.synchronize()
        self._shm.barrier()

    def alloc(self, nbytes: int, align: int = 256) -> int:
        off = (self._top + align - 1) // align * align
        if off + nbytes > self.usable:
            raise MemoryError(f"symmetric heap exhausted: need {nbytes} at {off}, slice has {self.usable}")
        self._top = off + nbytes
        return off

    def host_barrier(self) -> None:
        self._shm.barrier()

    def close(self) -> None:
        from ..api import shm
        if self._shm is not None:
            torch.cuda.synchronize()
            self._shm.barrier()
            self._shm.destroy()
            self._shm = None

    @staticmethod
    def shutdown() -> None:
        from ..api import shm
        if SymmetricHeap._inited:
            shm.uninitialize(0)
            SymmetricHeap._inited = False
