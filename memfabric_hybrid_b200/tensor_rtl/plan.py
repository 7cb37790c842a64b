"""Resharding plans: which slice of a tensor that is sharded over one list of ranks has to move to which
rank so that it ends up sharded over another list.

    pt = PTensor(shard, shard.dtype, shard.ndim, device_mesh=[0, 1, 2, 3], global_size=(4096, 1024), shard_dim=0)
    pt.transfer_map([4, 5])                       # TP4 on ranks 0-3  ->  TP2 on ranks 4-5
    executor.execute(pt.get_transfer_list()); executor.wait()
    new_shard = pt.collect_tensor()               # on ranks 4 and 5

Shard i of n covers [size * i // n, size * (i + 1) // n) of the sharded dimension, so sizes that do not
divide evenly are handled too. ``shard_dim = -1`` means replicated: every new rank takes the whole tensor
from one old rank (spread round-robin over the old ranks).

Parity: app/tensorRTL/src/tensor_rtl/core/ptensor.py:12-482, core/comm_task.py of the reference.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from .abc import BaseCommTask
from .buffer_pool import BufferPool
from .utils import get_dtype_size


@dataclass
class P2PCommTask(BaseCommTask):
    """One send (``is_send``: src_rank = me, dst_rank = receiver) or receive (src_rank = me, dst_rank = sender),
    the orientation the reference uses."""
    idx: int = 0
    numel: Optional[int] = None
    is_send: bool = False
    src_rank: int = 0
    dst_rank: int = 0
    buffer: Optional[torch.Tensor] = None
    stream: object = None
    tensor_slice: Tuple[int, int] = (0, 0)   # [begin, end) on the sharded dimension, in GLOBAL coordinates


@dataclass
class MFCommTask(BaseCommTask):
    """One copy through a BigMemory pool: writers put ``buffer`` at ``gva_ptr`` of ``pool_rank``'s slice,
    readers fetch from there."""
    idx: int = 0
    size: int = 0
    is_send: bool = False
    src_rank: int = 0
    dst_rank: int = 0
    pool_rank: int = 0
    gva_ptr: int = 0
    buffer: Optional[torch.Tensor] = None
    tensor_slice: Tuple[int, int] = (0, 0)


def shard_bounds(size: int, parts: int, i: int) -> Tuple[int, int]:
    return size * i // parts, size * (i + 1) // parts


def overlaps(size: int, old_mesh: Sequence[int], new_mesh: Sequence[int]):
    """All (old_rank, new_rank, begin, end) pieces of the sharded dimension that have to move, ordered by
    old shard then new shard. Pure function of its arguments: every rank computes the same list."""
    out = []
    for i, src in enumerate(old_mesh):
        a0, a1 = shard_bounds(size, len(old_mesh), i)
        for j, dst in enumerate(new_mesh):
            b0, b1 = shard_bounds(size, len(new_mesh), j)
            lo, hi = max(a0, b0), min(a1, b1)
            if lo < hi:
                out.append((src, dst, lo, hi))
    return out


class PTensor:
    def __init__(self, tensor: Optional[torch.Tensor], dtype: torch.dtype, ndim: int, device_mesh: Sequence[int],
                 global_size: Sequence[int], shard_dim: int, rank: Optional[int] = None, backend: str = "nccl", check_sanity: bool = True,
                 reuse_buffers: bool = False):
        """``reuse_buffers``: staging and receive buffers live in ``self.buffer_pool`` and are used again by every later
        ``transfer_map`` with the same mesh sizes (a plan that repeats allocates once; each ``transfer_map`` then starts a
        new plan, and the tensor returned by ``collect_tensor`` is overwritten by the next round)."""
        self.tensor, self.dtype, self.ndim = tensor, dtype, ndim
        self.buffer_pool = BufferPool()
        self.reuse_buffers = reuse_buffers
        self.device_mesh = list(device_mesh)
        self.global_size = torch.Size(global_size)
        self.shard_dim = shard_dim
        if rank is None:
            import torch.distributed as dist
            rank = dist.get_rank()
        self.rank = rank
        self.backend = "p2p" if backend in ("nccl", "hccl", "gloo", "p2p") else backend
        if check_sanity:
            self._validate()
        self._op_list: List = []
        self._recv: List[Tuple[int, torch.Tensor]] = []   # (begin on the sharded dim, buffer)
        self.pool_offset = 0   # where this tensor's pieces start inside a writer's pool slice (set by PTensorSet)

    # ------------------------------------------------------------------ validation
    def _validate(self) -> None:
        if self.backend not in ("p2p", "mf"):
            raise ValueError(f"backend must be 'nccl'/'gloo' (point to point) or 'mf' (memory pool), got {self.backend}")
        if len(self.global_size) != self.ndim:
            raise ValueError(f"global_size {tuple(self.global_size)} does not have ndim={self.ndim} entries")
        if not -1 <= self.shard_dim < self.ndim:
            raise ValueError(f"shard_dim {self.shard_dim} is outside [-1, {self.ndim})")
        self._check_mesh(self.device_mesh, "device_mesh")
        if self.rank in self.device_mesh:
            if self.tensor is None:
                raise ValueError("a rank of device_mesh must hold its shard")
            if self.tensor.dtype != self.dtype:
                raise ValueError(f"tensor dtype {self.tensor.dtype} differs from dtype {self.dtype}")
            exp = list(self.global_size)
            if self.shard_dim >= 0:
                b0, b1 = shard_bounds(exp[self.shard_dim], len(self.device_mesh), self.device_mesh.index(self.rank))
                exp[self.shard_dim] = b1 - b0
            if list(self.tensor.shape) != exp:
                raise ValueError(f"shard shape {tuple(self.tensor.shape)} differs from the expected {tuple(exp)}")

    @staticmethod
    def _check_mesh(mesh, name: str) -> None:
        if not isinstance(mesh, (list, tuple)) or len(mesh) == 0:
            raise ValueError(f"{name} must be a non-empty list of ranks")
        if any((not isinstance(r, int)) or r < 0 for r in mesh):
            raise ValueError(f"{name} must hold non-negative integers")
        if len(set(mesh)) != len(mesh):
            raise ValueError(f"{name} holds a rank twice")

    # ------------------------------------------------------------------ planning
    def _pieces(self, new_mesh: Sequence[int]):
        if self.shard_dim < 0:
            # replicated: new rank j copies the whole tensor from old rank j mod n (ranks that already hold it keep it)
            n = len(self.device_mesh)
            return [(dst if dst in self.device_mesh else self.device_mesh[j % n], dst, 0, 1) for j, dst in enumerate(new_mesh)]
        return overlaps(self.global_size[self.shard_dim], self.device_mesh, new_mesh)

    def _my_shard_begin(self) -> int:
        if self.shard_dim < 0:
            return 0
        return shard_bounds(self.global_size[self.shard_dim], len(self.device_mesh), self.device_mesh.index(self.rank))[0]

    def _slice_of_mine(self, lo: int, hi: int) -> torch.Tensor:
        if self.shard_dim < 0:
            return self.tensor
        b = self._my_shard_begin()
        return self.tensor.narrow(self.shard_dim, lo - b, hi - lo)

    def _recv_shape(self, lo: int, hi: int):
        shp = list(self.global_size)
        if self.shard_dim >= 0:
            shp[self.shard_dim] = hi - lo
        return shp

    def transfer_map(self, update_device_mesh: Sequence[int], use_empty_recv: bool = True) -> None:
        """Adds the tasks of this rank for moving the tensor onto ``update_device_mesh``. Pieces that stay on
        the same rank are copied locally right away and produce no task."""
        self._check_mesh(update_device_mesh, "update_device_mesh")
        new_mesh = list(update_device_mesh)
        dev = self.tensor.device if self.tensor is not None else torch.device("cuda", torch.cuda.current_device()) \
            if torch.cuda.is_available() else torch.device("cpu")
        ops = []
        pool_off = {}
        lengths = (len(self.device_mesh), len(new_mesh))
        if self.reuse_buffers:
            self._op_list, self._recv = [], []
        for idx, (src, dst, lo, hi) in enumerate(self._pieces(new_mesh)):
            shape = self._recv_shape(lo, hi)
            numel = 1
            for s in shape:
                numel *= s
            nbytes = numel * get_dtype_size(self.dtype)
            off = self.pool_offset + pool_off.get(src, 0)          # position of this piece inside src's pool slice
            pool_off[src] = pool_off.get(src, 0) + (nbytes + 255) // 256 * 256
            if src == dst:
                if self.rank == src:
                    if self.reuse_buffers:
                        keep = self.buffer_pool.get_or_create(lengths, ("keep", lo, hi), lambda: torch.empty(shape, dtype=self.dtype, device=dev))
                        keep.copy_(self._slice_of_mine(lo, hi))
                    else:
                        keep = self._slice_of_mine(lo, hi).clone()
                    self._recv.append((lo, keep))
                continue
            if self.rank == src:
                mine = self._slice_of_mine(lo, hi)
                if mine.is_contiguous():
                    buf = mine                                   # sent from where it lies
                elif self.reuse_buffers:
                    buf = self.buffer_pool.get_or_create(lengths, ("send", lo, hi), lambda: torch.empty(shape, dtype=self.dtype, device=dev))
                    buf.copy_(mine)
                else:
                    buf = mine.contiguous()
                if self.backend == "mf":
                    ops.append(MFCommTask(idx, nbytes, True, src, dst, src, off, buf, (lo, hi)))
                else:
                    ops.append(P2PCommTask(idx, numel, True, src, dst, buf, None, (lo, hi)))
            if self.rank == dst:
                if self.reuse_buffers:
                    buf = self.buffer_pool.get_or_create(lengths, ("recv", src, lo, hi), lambda: torch.empty(shape, dtype=self.dtype, device=dev))
                else:
                    buf = torch.empty(shape, dtype=self.dtype, device=dev)
                self._recv.append((lo, buf))
                if self.backend == "mf":
                    ops.append(MFCommTask(idx, nbytes, False, dst, src, src, off, buf, (lo, hi)))
                else:
                    ops.append(P2PCommTask(idx, numel, False, dst, src, buf, None, (lo, hi)))
        self.pool_bytes = max(pool_off.values(), default=0)
        self._op_list.extend(ops)

    def get_transfer_list(self) -> List:
        return self._op_list

    def collect_tensor(self) -> Optional[torch.Tensor]:
        """The new shard of this rank (pieces joined along the sharded dimension), or None if it holds none."""
        if not self._recv:
            return None
        parts = [b for _, b in sorted(self._recv, key=lambda p: p[0])]
        if len(parts) == 1 or self.shard_dim < 0:
            return parts[0]
        return torch.cat(parts, dim=self.shard_dim)


class PTensorSet:
    """Many tensors resharded together: one task list, one executor call."""

    def __init__(self, ptensor_list: List[PTensor]):
        if not ptensor_list:
            raise ValueError("ptensor_list is empty")
        self.ptensors = list(ptensor_list)
        self._ops: List = []

    def transfer_map(self, update_map: Sequence[Sequence[int]], use_empty_recv: bool = True) -> None:
        """update_map: one new device mesh per tensor, or a single mesh for all."""
        meshes = list(update_map)
        if meshes and isinstance(meshes[0], int):
            meshes = [meshes] * len(self.ptensors)
        if len(meshes) != len(self.ptensors):
            raise ValueError(f"{len(meshes)} meshes for {len(self.ptensors)} tensors")
        off = 0
        for pt, mesh in zip(self.ptensors, meshes):
            pt.pool_offset = off
            pt.transfer_map(mesh, use_empty_recv)
            off += pt.pool_bytes
        self.pool_bytes = off
        self._ops = [t for pt in self.ptensors for t in pt.get_transfer_list()]

    def get_transfer_list(self) -> List:
        return self._ops

    def collect_tensor(self) -> List[Optional[torch.Tensor]]:
        return [pt.collect_tensor() for pt in self.ptensors]
