"""Small helpers of the resharding layer. Parity: app/tensorRTL/src/tensor_rtl/utils/utils.py of the reference."""
import torch


def get_dtype_size(dtype: torch.dtype) -> int:
    """Bytes per element (bool and the 8-bit floats: 1; complex types: both halves)."""
    return torch.empty((), dtype=dtype).element_size()
