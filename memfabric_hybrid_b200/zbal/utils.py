"""Small helpers of the MoE ``Buffer`` API: ``Config`` (kernel tuning knobs) and ``EventOverlap``.
Parity: app/zbal/src/python/zbal/zbal_utils.py:8-40 and the ``Config`` class of the reference's adaptor."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass
class Config:
    """Tuning of a dispatch/combine call. Only ``num_sms`` has an effect here (CTAs of the push kernels);
    the chunking fields are accepted for signature compatibility: the kernels store straight into the
    peers' receive buffers, so there are no send/receive chunk queues to size."""
    num_sms: int = 148
    num_max_nvl_chunked_send_tokens: int = 6
    num_max_nvl_chunked_recv_tokens: int = 256
    num_max_rdma_chunked_send_tokens: int = 6
    num_max_rdma_chunked_recv_tokens: int = 256

    def get_nvl_buffer_size_hint(self, hidden_bytes: int, num_ranks: int) -> int:
        return self.num_max_nvl_chunked_recv_tokens * hidden_bytes * num_ranks


class EventOverlap:
    """A CUDA event plus tensors kept alive until it is waited on; usable as a context manager:
    the body runs, then the current stream waits for the event."""

    def __init__(self, event: Optional[torch.cuda.Event] = None, extra_tensors: Optional[Tuple[torch.Tensor, ...]] = None):
        self.event = event
        self.extra_tensors = extra_tensors

    def current_stream_wait(self) -> None:
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.current_stream_wait()
        return False
