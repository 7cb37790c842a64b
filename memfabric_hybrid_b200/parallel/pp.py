"""Pipeline-parallel activation exchange. Stage-to-stage traffic stays on NCCL point-to-point calls, on a
stream of its own so that it overlaps the stage's compute (the reference has no pipeline schedule either;
it only provides send/recv, zbal_pytorch_process_group.h:164-166). The zbal send/recv kernels are available through the
"zbal" backend for small latency-critical messages; for large activations NCCL's copy-engine path frees
the SMs for the next micro-batch.

    p2p = StageLink(mesh)                     # mesh.prev_stage / mesh.next_stage
    x = p2p.recv_forward(shape, dtype)        # None on the first stage
    y = stage(x); p2p.send_forward(y)
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist


class StageLink:
    def __init__(self, mesh, group: Optional[dist.ProcessGroup] = None):
        self.prev, self.next = mesh.prev_stage, mesh.next_stage
        self.group = group
        self.stream = torch.cuda.Stream()
        self._pending = []

    def _post(self, ops):
        if not ops:
            return
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            self._pending.extend(dist.batch_isend_irecv(ops))

    def send_forward(self, t: torch.Tensor) -> None:
        if self.next is not None:
            t.record_stream(self.stream)
            self._post([dist.P2POp(dist.isend, t.contiguous(), self.next, self.group)])

    def send_backward(self, t: torch.Tensor) -> None:
        if self.prev is not None:
            t.record_stream(self.stream)
            self._post([dist.P2POp(dist.isend, t.contiguous(), self.prev, self.group)])

    def recv_forward(self, shape: Sequence[int], dtype: torch.dtype) -> Optional[torch.Tensor]:
        if self.prev is None:
            return None
        buf = torch.empty(tuple(shape), dtype=dtype, device="cuda")
        self._post([dist.P2POp(dist.irecv, buf, self.prev, self.group)])
        self.wait()
        return buf

    def recv_backward(self, shape: Sequence[int], dtype: torch.dtype) -> Optional[torch.Tensor]:
        if self.next is None:
            return None
        buf = torch.empty(tuple(shape), dtype=dtype, device="cuda")
        self._post([dist.P2POp(dist.irecv, buf, self.next, self.group)])
        self.wait()
        return buf

    def wait(self) -> None:
        for r in self._pending:
            r.wait()
        self._pending.clear()
        torch.cuda.current_stream().wait_stream(self.stream)
