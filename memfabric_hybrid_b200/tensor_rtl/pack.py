"""Packs tensors of mixed shapes and dtypes into one flat tensor for a single transfer and back.
Parity: app/tensorRTL/src/tensor_rtl/utils/dtype_converter.py:10-119 of the reference."""
from __future__ import annotations

from typing import Any, Dict, List, Tuple

import torch


def pack_tensors(tensor_list: List[torch.Tensor], target_dtype: torch.dtype = torch.int8) -> Tuple[torch.Tensor, Dict[str, Any]]:
    if not tensor_list:
        raise ValueError("tensor_list is empty")
    dev = tensor_list[0].device
    tsz = torch.empty((), dtype=target_dtype).element_size()
    meta = {"original_shapes": [], "original_dtypes": [], "element_counts": [], "original_element_counts": [], "target_dtype": target_dtype}
    total = 0
    for t in tensor_list:
        if t.device != dev:
            raise ValueError("all tensors must be on one device")
        nbytes = t.numel() * t.element_size()
        cnt = (nbytes + tsz - 1) // tsz
        meta["original_shapes"].append(tuple(t.shape))
        meta["original_dtypes"].append(t.dtype)
        meta["original_element_counts"].append(t.numel())
        meta["element_counts"].append(cnt)
        total += cnt
    packed = torch.zeros(total * tsz, dtype=torch.uint8, device=dev)
    pos = 0
    for t, cnt in zip(tensor_list, meta["element_counts"]):
        raw = t.contiguous().view(-1).view(torch.uint8)
        packed[pos:pos + raw.numel()] = raw
        pos += cnt * tsz
    return packed.view(target_dtype), meta


def unpack_tensors(packed_tensor: torch.Tensor, metadata: Dict[str, Any]) -> List[torch.Tensor]:
    raw = packed_tensor.contiguous().view(-1).view(torch.uint8)
    tsz = torch.empty((), dtype=metadata["target_dtype"]).element_size()
    out, pos = [], 0
    for shape, dt, cnt, n in zip(metadata["original_shapes"], metadata["original_dtypes"], metadata["element_counts"],
                                 metadata["original_element_counts"]):
        nbytes = n * torch.empty((), dtype=dt).element_size()
        out.append(raw[pos:pos + nbytes].clone().view(dt).view(shape))
        pos += cnt * tsz
    return out
