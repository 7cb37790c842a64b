"""Data-parallel gradient reduction on the zbal collectives: gradients are packed into buckets that live in
the symmetric heap, so the all-reduce runs in direct mode (peers read and write the bucket in place) with
the 1/world average fused into the kernel, on a side stream that overlaps the rest of the backward pass.

    reducer = GradReducer(model.parameters(), group=mesh.dp_group, bucket_mb=64)
    loss.backward(); reducer.reduce(); reducer.wait()      # p.grad now holds the average

The reference enables data parallelism only indirectly, by providing the collectives DeepSpeed ZeRO calls
(app/zbal/doc/user_guide/get_started.md:50-176); this is the same idea without the external framework.
Buckets are sized for NVSwitch: large enough that the launch and handshake latency (tens of microseconds)
is amortised, not so large that the first reduction waits for the whole backward pass.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch
import torch.distributed as dist


class GradReducer:
    def __init__(self, params: Iterable[torch.nn.Parameter], group: Optional[dist.ProcessGroup] = None, bucket_mb: int = 64,
                 symmetric: bool = True):
        self.params = [p for p in params if p.requires_grad]
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._buckets: List[tuple] = []     # (flat tensor, [(param, offset, numel)])
        self._works = []
        cap = bucket_mb << 20
        by_dtype = {}
        for p in reversed(self.params):     # gradients become ready roughly in reverse order
            by_dtype.setdefault(p.dtype, []).append(p)
        from .. import zbal
        use_heap = symmetric and zbal.is_initialized()
        for dtype, ps in by_dtype.items():
            cur, size = [], 0
            for p in ps + [None]:
                if p is None or (cur and (size + p.numel()) * p.element_size() > cap):
                    if cur:
                        n = sum(q.numel() for q in cur)
                        if use_heap:
                            with zbal.switch_to_allocator():
                                flat = torch.zeros(n, dtype=dtype, device=cur[0].device)
                        else:
                            flat = torch.zeros(n, dtype=dtype, device=cur[0].device)
                        slots, off = [], 0
                        for q in cur:
                            slots.append((q, off, q.numel()))
                            off += q.numel()
                        self._buckets.append((flat, slots))
                    cur, size = [], 0
                if p is not None:
                    cur.append(p)
                    size += p.numel()

    def reduce(self) -> None:
        """Packs the gradients and starts one averaged all-reduce per bucket (asynchronously)."""
        for flat, slots in self._buckets:
            for p, off, n in slots:
                if p.grad is not None:
                    flat[off:off + n].copy_(p.grad.reshape(-1))
                else:
                    flat[off:off + n].zero_()
            if self.world > 1:
                self._works.append(dist.all_reduce(flat, op=dist.ReduceOp.AVG, group=self.group, async_op=True))

    def wait(self) -> None:
        for w in self._works:
            w.wait()
        self._works.clear()
        for flat, slots in self._buckets:
            for p, off, n in slots:
                if p.grad is not None:
                    p.grad.copy_(flat[off:off + n].view_as(p.grad))
