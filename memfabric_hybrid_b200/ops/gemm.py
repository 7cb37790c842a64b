"""tcgen05 / TMEM GEMMs (csrc/kernels/mf_gemm.cu, mf_gemm_fp8.cu, mf_gemm_fp8_mx.cu).

    gemm_bf16(a, b)                  C[M,N] = A[M,K] . B[N,K]^T   (bf16 in, fp32 accumulate in TMEM, bf16 out)

The status word is a device int that a kernel sets when one of its bounded pipeline waits gives up;
``check_status`` turns that into an exception."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N

_lib = None
_status = {}


def _cu():
    global _lib
    if _lib is None:
        l = N.cuda()
        l.mf_gemm_bf16.restype = C.c_int
        l.mf_gemm_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int64,
                                   C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        for fn in (l.mf_gemm_bf16_pair, l.mf_gemm_bf16_one):
            fn.restype = C.c_int
            fn.argtypes = l.mf_gemm_bf16.argtypes
        _lib = l
    return _lib


def status_word(device=None) -> torch.Tensor:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    t = _status.get(dev)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[dev] = t
    return t


def check_status(device=None) -> None:
    st = status_word(device)
    v = int(st.item())
    if v != 0:
        st.zero_()
        raise RuntimeError(f"a GEMM pipeline wait gave up (code {v:#x})")


def sm_count(device=None) -> int:
    return torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device()).multi_processor_count


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor, tile: int = 128) -> torch.Tensor:
    """[F,K] gate and up weights -> [2F,K] with, per 256 rows, 128 gate rows followed by their 128 up rows: the
    layout the fused SwiGLU epilogue expects (F must divide by 128)."""
    F, K = w_gate.shape
    assert w_up.shape == (F, K) and F % tile == 0
    return torch.stack([w_gate.view(F // tile, tile, K), w_up.view(F // tile, tile, K)], dim=1).reshape(2 * F, K).contiguous()


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, sms: int | None = None,
              swiglu: bool = False, pair: bool | None = None) -> torch.Tensor:
    """C = A[M,K] . B[N,K]^T. pair=True runs the CTA-pair kernel (one 256 x 256 tile per two SMs), False the one-CTA
    kernel (128 x 256 tiles); None lets the library pick by how well the tiles fill the SMs (MF_GEMM_PAIR=0 / 1 forces it)."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_cuda and b.is_cuda
    assert a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1], "A[M,K] and B[N,K] must share K"
    assert a.stride(1) == 1 and b.stride(1) == 1, "K must be the contiguous dimension"
    M, K = a.shape
    Nn = b.shape[0]
    if out is None:
        out = torch.empty((M, Nn // 2 if swiglu else Nn), dtype=torch.bfloat16, device=a.device)
    fn = _cu().mf_gemm_bf16 if pair is None else (_cu().mf_gemm_bf16_pair if pair else _cu().mf_gemm_bf16_one)
    rc = fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, Nn, K, a.stride(0), b.stride(0), out.stride(0),
            status_word(a.device).data_ptr(), sms or sm_count(a.device), 1 if swiglu else 0,
            torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"mf_gemm_bf16 failed to launch ({rc})")
    return out
