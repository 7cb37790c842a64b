"""Communication buffers kept between resharding rounds, so that a plan that repeats (weights handed from training to
inference after every step) allocates its staging and receive buffers once. Keyed first by the pair (old mesh length,
new mesh length), then by the slice of the tensor the buffer carries.
Parity: app/tensorRTL/src/tensor_rtl/core/buffer_pool.py of the reference (register / get / get_keys)."""
from __future__ import annotations

from typing import Callable, Dict, Hashable, Optional

import torch


class BufferPool:
    def __init__(self):
        self.send_buffer_dict: Dict[Hashable, Dict[Hashable, torch.Tensor]] = {}

    def register(self, length_tuple, tensor_slice, buffer: torch.Tensor) -> None:
        """Keeps ``buffer`` unless the slot is taken already (the first registration wins)."""
        self.send_buffer_dict.setdefault(length_tuple, {}).setdefault(tensor_slice, buffer)

    def get(self, length_tuple, tensor_slice) -> Optional[torch.Tensor]:
        return self.send_buffer_dict.get(length_tuple, {}).get(tensor_slice)

    def get_keys(self):
        return self.send_buffer_dict.keys()

    def get_or_create(self, length_tuple, tensor_slice, make: Callable[[], torch.Tensor]) -> torch.Tensor:
        buf = self.get(length_tuple, tensor_slice)
        if buf is None:
            buf = make()
            self.register(length_tuple, tensor_slice, buf)
        return buf

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for d in self.send_buffer_dict.values() for b in d.values())

    def clear(self) -> None:
        self.send_buffer_dict.clear()
