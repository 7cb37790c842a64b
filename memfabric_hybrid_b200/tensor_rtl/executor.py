"""Executors that carry out a list of resharding tasks.

  BatchP2PExecutor      one ``dist.batch_isend_irecv`` over all tasks (NCCL or gloo process group)
  All2AllVExecutor      packs the pieces per peer and moves them with ONE ``all_to_all_single``; with
                        ``execute_async`` the next batch is packed while the current one is in flight
  MemoryFabricExecutor  writers put their pieces into a BigMemory pool (L2G), readers fetch them (G2L): the
                        two sides need not run at the same time, nor be in one process group

Parity: app/tensorRTL/src/tensor_rtl/core/executor.py:21-271, api/abc.py of the reference (which spells the
second class ``All2AllVExcutor``; that name is kept as an alias).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from .abc import BaseCommTask, Executor, Planner  # noqa: F401
from .plan import MFCommTask, P2PCommTask


class BatchP2PExecutor(Executor):
    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        super().__init__()
        self.group = group
        self._reqs = []

    def execute(self, tasks: List[P2PCommTask]) -> None:
        ops = []
        for t in tasks:
            fn = dist.isend if t.is_send else dist.irecv
            ops.append(dist.P2POp(fn, t.buffer, t.dst_rank, self.group))
        if ops:
            self._reqs.extend(dist.batch_isend_irecv(ops))

    def wait(self) -> None:
        for r in self._reqs:
            r.wait()
        self._reqs.clear()


class All2AllVExecutor(Executor):
    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        super().__init__()
        self.group = group
        self._pending = None

    def _build(self, tasks: List[P2PCommTask]):
        world = dist.get_world_size(self.group)
        sends = [[] for _ in range(world)]
        recvs = [[] for _ in range(world)]
        for t in sorted(tasks, key=lambda t: t.idx):
            (sends if t.is_send else recvs)[t.dst_rank].append(t)
        dev = tasks[0].buffer.device if tasks else torch.device("cpu")
        in_split = [sum(t.buffer.numel() * t.buffer.element_size() for t in s) for s in sends]
        out_split = [sum(t.buffer.numel() * t.buffer.element_size() for t in r) for r in recvs]
        flat_in = torch.empty(sum(in_split), dtype=torch.uint8, device=dev)
        pos = 0
        for s in sends:
            for t in s:
                raw = t.buffer.contiguous().view(-1).view(torch.uint8)
                flat_in[pos:pos + raw.numel()] = raw
                pos += raw.numel()
        flat_out = torch.empty(sum(out_split), dtype=torch.uint8, device=dev)
        return flat_in, flat_out, in_split, out_split, recvs

    @staticmethod
    def _scatter_out(flat_out: torch.Tensor, recvs) -> None:
        pos = 0
        for r in recvs:
            for t in r:
                n = t.buffer.numel() * t.buffer.element_size()
                t.buffer.view(-1).view(torch.uint8).copy_(flat_out[pos:pos + n])
                pos += n

    def execute(self, tasks: List[P2PCommTask]) -> None:
        flat_in, flat_out, ins, outs, recvs = self._build(tasks)
        dist.all_to_all_single(flat_out, flat_in, outs, ins, group=self.group)
        self._scatter_out(flat_out, recvs)

    def build_all2all_info(self, task_list: List[P2PCommTask]):
        return self._build(task_list)

    def execute_async(self, task_list: List[P2PCommTask], pre_build_task_list: Optional[List[P2PCommTask]] = None):
        """Starts ``task_list`` (asynchronously) and, while it runs, packs ``pre_build_task_list``; returns the
        packed form, to be passed to the next call in place of its task list."""
        built = task_list if isinstance(task_list, tuple) else self._build(task_list)
        flat_in, flat_out, ins, outs, recvs = built
        work = dist.all_to_all_single(flat_out, flat_in, outs, ins, group=self.group, async_op=True)
        self._pending = (work, flat_out, recvs, flat_in)
        return self._build(pre_build_task_list) if pre_build_task_list else None

    def wait(self) -> None:
        if self._pending is not None:
            work, flat_out, recvs, _ = self._pending
            work.wait()
            self._scatter_out(flat_out, recvs)
            self._pending = None


All2AllVExcutor = All2AllVExecutor


@dataclass
class MfBmConfig:
    """Settings of the pool a MemoryFabricExecutor creates. ``mem_type``/``data_op_type`` take the enums of
    ``memfabric_hybrid.bm``; a host-DRAM pool (HOST / HOST_SHM) works without a GPU."""
    url: str = "tcp://127.0.0.1:8570"
    mem_type: object = None
    data_op_type: object = None
    local_dram_size: int = 0
    local_hbm_size: int = 0
    auto_ranking: bool = False
    hybm_int_gvm_flag: int = 0
    rank_world_size: int = 8
    start_store: Optional[bool] = None   # default: rank 0 hosts the config store
    bm_handle: object = None


class MemoryFabricExecutor(Executor):
    class ExecutorType(enum.Enum):
        WRITER = "writer"
        READER = "reader"
        MIXER = "mix"

    _initialized = False
    _handle = None

    def __init__(self, bm_config: MfBmConfig, rank_id: Optional[int] = None, executor_type: "MemoryFabricExecutor.ExecutorType" = None,
                 device_id: Optional[int] = None):
        super().__init__()
        from .. import api as mf
        from ..api import bm
        self.bm = bm
        self.executor_type = executor_type or MemoryFabricExecutor.ExecutorType.MIXER
        if bm_config.mem_type is None:
            bm_config.mem_type = bm.BmMemType.DEVICE if bm_config.local_hbm_size else bm.BmMemType.HOST
        if bm_config.data_op_type is None:
            bm_config.data_op_type = bm.BmDataOpType.SDMA if bm_config.local_hbm_size else bm.BmDataOpType.HOST_SHM
        if not MemoryFabricExecutor._initialized:
            if rank_id is None:
                rank_id = dist.get_rank()
            if device_id is None:
                device_id = torch.cuda.current_device() if torch.cuda.is_available() else 0
            rc = mf.initialize()
            if rc != 0:
                raise RuntimeError(f"memfabric initialize failed on rank {rank_id}: {rc}")
            cfg = bm.BmConfig()
            cfg.auto_ranking = bm_config.auto_ranking
            if not bm_config.auto_ranking:
                cfg.rank_id = rank_id
            cfg.flags = bm_config.hybm_int_gvm_flag
            cfg.start_store = (rank_id == 0) if bm_config.start_store is None else bm_config.start_store
            rc = bm.initialize(store_url=bm_config.url, world_size=bm_config.rank_world_size, device_id=device_id, config=cfg)
            if rc != 0:
                raise RuntimeError(f"bm.initialize failed on rank {rank_id} ({rc}): {mf.get_last_err_msg()}")
            h = bm.create(id=0, local_dram_size=bm_config.local_dram_size, local_hbm_size=bm_config.local_hbm_size,
                          data_op_type=bm_config.data_op_type)
            h.join()
            MemoryFabricExecutor._handle = h
            MemoryFabricExecutor._initialized = True
        bm_config.bm_handle = MemoryFabricExecutor._handle
        self.bm_config = bm_config
        self.bm_handle = MemoryFabricExecutor._handle

    def is_writer(self) -> bool:
        return self.executor_type is not self.ExecutorType.READER

    def is_reader(self) -> bool:
        return self.executor_type is not self.ExecutorType.WRITER

    def convert_to_batch_copy(self, task_list: List[MFCommTask], sending: bool):
        src, dst, sizes = [], [], []
        for t in task_list:
            if t.is_send != sending:
                continue
            gva = self.bm_handle.peer_rank_ptr(t.pool_rank, mem_type=self.bm_config.mem_type) + t.gva_ptr
            if sending:
                src.append(t.buffer.data_ptr())
                dst.append(gva)
            else:
                src.append(gva)
                dst.append(t.buffer.data_ptr())
            sizes.append(t.size)
        return src, dst, sizes

    def write(self, tasks: List[MFCommTask]) -> None:
        """Puts this rank's pieces into its own slice of the pool."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        src, dst, sizes = self.convert_to_batch_copy(tasks, True)
        if src:
            rc = self.bm_handle.copy_data_batch(src, dst, sizes, len(src), self.bm.BmCopyType.L2G, 0)
            if rc != 0:
                raise RuntimeError(f"pool write failed ({rc})")

    def read(self, tasks: List[MFCommTask]) -> None:
        """Fetches the pieces meant for this rank from the writers' slices. The writers must have finished
        (``execute`` puts a process-group barrier between the two halves; separate writer and reader jobs
        synchronise by their own means)."""
        src, dst, sizes = self.convert_to_batch_copy(tasks, False)
        if src:
            rc = self.bm_handle.copy_data_batch(src, dst, sizes, len(src), self.bm.BmCopyType.G2L, 0)
            if rc != 0:
                raise RuntimeError(f"pool read failed ({rc})")

    def execute(self, tasks: List[MFCommTask]) -> None:
        if self.is_writer():
            self.write(tasks)
        if self.executor_type is self.ExecutorType.MIXER and dist.is_initialized():
            dist.barrier()
        if self.is_reader():
            self.read(tasks)

    def wait(self) -> None:
        self.bm_handle.wait()

    @classmethod
    def shutdown(cls) -> None:
        if cls._initialized:
            from ..api import bm
            cls._handle.leave()
            cls._handle.destroy()
            bm.uninitialize()
            cls._handle, cls._initialized = None, False
