"""Tensor-parallel fusions on the symmetric heap (kernels in csrc/kernels/mf_gemm.cu and mf_gemm_fp8_mx.cu).

    tp = TensorParallel(heap, max_tokens=8192, hidden=8192)
    h  = tp.ag_gemm(x_shard, w_gate_up_interleaved, swiglu=True)     # all-gather fused into the gate/up GEMM
    y  = tp.gemm_rs(h, w_down)                                        # down-proj GEMM fused with reduce-scatter

fp8 (e4m3, 1 x 128 activation scales, 128 x 128 weight scales, all powers of two, applied by the tensor core):

    tp = TensorParallel(heap, max_tokens=8192, hidden=8192, fp8=True)
    hq, hs = tp.ag_gemm_fp8(x_shard, wq_gate_up, ws_gate_up)          # quantise-on-gather + GEMM + SwiGLU + re-quantisation
    y      = tp.gemm_rs_fp8(hq, hs, wq_down, ws_down)                 # fp8 GEMM fused with the reduce-scatter

Every rank must issue the same sequence of calls. Buffers are double-buffered by call parity: a rank can
start call k+2 only after every peer started call k+1, i.e. finished reading the buffers of call k.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N
from . import gemm
from .gemm import status_word, sm_count
from .heap import TeamC, _HeapBase

_lib = None


def _cu():
    global _lib
    if _lib is None:
        l = N.cuda()
        P = C.POINTER
        l.mf_ag_gemm_bf16.restype = C.c_int
        l.mf_ag_gemm_bf16.argtypes = [P(TeamC), C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int,
                                      C.c_int, C.c_uint64, C.c_uint64, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_int, C.c_int,
                                      C.c_void_p]
        l.mf_gemm_rs_bf16.restype = C.c_int
        l.mf_gemm_rs_bf16.argtypes = [P(TeamC), C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int, C.c_int,
                                      C.c_int, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_float, C.c_void_p, C.c_int, C.c_void_p]
        vp, ci, i64, u64, u32 = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_uint32
        l.mf_ag_gemm_fp8.restype = ci
        l.mf_ag_gemm_fp8.argtypes = [P(TeamC), vp, i64, ci, vp, vp, vp, i64, vp, ci, ci, u64, u64, u64, vp, u32, u32, vp, ci, ci, vp]
        l.mf_gemm_rs_fp8.restype = ci
        l.mf_gemm_rs_fp8.argtypes = [P(TeamC), vp, vp, vp, vp, vp, i64, ci, ci, ci, u64, u64, u32, u32, C.c_float, vp, ci, vp]
        _lib = l
    return _lib


class TensorParallel:
    def __init__(self, heap: _HeapBase, max_tokens: int, hidden: int, max_out: int | None = None, fp8: bool = False):
        assert not heap.emu, "the fused TP kernels need real ranks (world 1 on one GPU is fine)"
        self.heap = heap
        self.world, self.rank = heap.world, heap.rank
        self.max_tokens, self.hidden = max_tokens, hidden
        max_out = max_out or hidden
        # gather buffers [tokens, hidden] bf16 and landing zones [world][tokens / world][max_out] bf16, two of each
        self._ag = [heap.alloc(max_tokens * hidden * 2, 1024) for _ in range(2)]
        # fp8: the gather buffer holds e4m3 bytes (the first half of the bf16 buffer is enough) and their 1 x 128 scales
        self._ags = [heap.alloc(max_tokens * (hidden // 128) * 4, 1024) for _ in range(2)] if fp8 else None
        self._ready = [heap.alloc(64 * 4, 256) for _ in range(2)]
        self._land = [heap.alloc(max_tokens * max_out * 2, 1024) for _ in range(2)]
        tiles = (max_tokens // self.world // 128 + 1) * ((max_out + 255) // 256)
        self._cnt = [heap.alloc(tiles * 4, 256) for _ in range(2)]
        self.max_out = max_out
        dev = torch.device("cuda", torch.cuda.current_device())
        self._push = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(2)]
        self._ag_calls = [0, 0]
        self._rs_calls = [0, 0]
        self._epoch = 0
        # world 1: the bf16 calls run the plain GEMM; False keeps them on the fused kernels (self-gather / self-scatter)
        self.plain_at_world1 = True
        for off, n in ((self._ready[0], 64 * 4), (self._ready[1], 64 * 4), (self._cnt[0], tiles * 4), (self._cnt[1], tiles * 4)):
            heap.view(off, (n,), torch.uint8).zero_()
        torch.cuda.synchronize()
        if hasattr(heap, "host_barrier"):
            heap.host_barrier()

    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, swiglu: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
        """x_shard [T/W, H] (this rank's sequence shard), w [N, H] -> [T, N] (or [T, N/2] with swiglu)."""
        assert x_shard.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x_shard.stride(1) == 1 and w.stride(1) == 1
        rows, K = x_shard.shape
        assert rows % 128 == 0 and rows * self.world <= self.max_tokens and K == self.hidden
        Nn = w.shape[0]
        T = rows * self.world
        if out is None:
            out = torch.empty((T, Nn // 2 if swiglu else Nn), dtype=torch.bfloat16, device=x_shard.device)
        if self.world == 1 and self.plain_at_world1:   # nothing to gather: the plain GEMM (CTA pairs where the shape fills them)
            return gemm.gemm_bf16(x_shard, w, out=out, swiglu=swiglu)
        self._epoch += 1
        b = self._epoch & 1
        self._ag_calls[b] += 1
        team = self.heap.team()
        rc = _cu().mf_ag_gemm_bf16(C.byref(team), x_shard.data_ptr(), x_shard.stride(0), rows, w.data_ptr(), w.stride(0), out.data_ptr(),
                                   out.stride(0), Nn, K, self._ag[b], self._ready[b], self._push[b].data_ptr(), self._epoch,
                                   self._ag_calls[b], status_word(x_shard.device).data_ptr(), sm_count(x_shard.device),
                                   1 if swiglu else 0, torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"mf_ag_gemm_bf16 failed to launch ({rc})")
        return out

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, scale: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
        """a [T, K] (full sequence, this rank's K-slice), w [N, K] -> this rank's [T/W, N] of sum_over_ranks(a . w^T) * scale."""
        assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.stride(1) == 1 and w.stride(1) == 1
        T, K = a.shape
        Nn = w.shape[0]
        assert T % (self.world * 128) == 0 and T <= self.max_tokens and Nn <= self.max_out and Nn % 8 == 0
        rows = T // self.world
        if out is None:
            out = torch.empty((rows, Nn), dtype=torch.bfloat16, device=a.device)
        if self.world == 1 and scale == 1.0 and self.plain_at_world1:   # nothing to reduce
            return gemm.gemm_bf16(a, w, out=out)
        self._epoch += 1
        b = self._epoch & 1
        self._rs_calls[b] += 1
        team = self.heap.team()
        rc = _cu().mf_gemm_rs_bf16(C.byref(team), a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), rows,
                                   Nn, K, self._land[b], self._cnt[b], self._epoch, self._rs_calls[b], float(scale),
                                   status_word(a.device).data_ptr(), sm_count(a.device), torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"mf_gemm_rs_bf16 failed to launch ({rc})")
        return out

    # ------------------------------------------------------------------ fp8 (block-scaled tensor-core MMA)
    def ag_gemm_fp8(self, x_shard: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, epi: str = "swiglu_fp8"):
        """x_shard [T/W, H] bf16 (this rank's sequence shard; quantised to e4m3 + 1 x 128 power-of-two scales on its way
        into the gather buffers), wq [N, H] e4m3 (``ops.moe.quantize_weight_fp8``; for the SwiGLU epilogues gate / up rows
        interleaved per 128: ``ops.moe.interleave_gate_up_fp8(w[None], 128)[0]``), ws [N/128, H/128] in original row order.
        epi "swiglu_fp8": -> (h e4m3 [T, N/2], scales [T, N/256]); "swiglu": -> h bf16 [T, N/2]; "plain": -> bf16 [T, N]."""
        assert self._ags is not None, "create TensorParallel(..., fp8=True)"
        assert x_shard.dtype == torch.bfloat16 and x_shard.stride(1) == 1 and wq.is_contiguous() and ws.dtype == torch.float32 and ws.is_contiguous()
        rows, K = x_shard.shape
        Nn = wq.shape[0]
        assert rows % 128 == 0 and rows * self.world <= self.max_tokens and K == self.hidden and K % 512 == 0 and Nn % 256 == 0
        T = rows * self.world
        dev = x_shard.device
        code = {"plain": 0, "swiglu": 1, "swiglu_fp8": 3}[epi]
        out_s = None
        if code == 3:
            out = torch.empty((T, Nn // 2), dtype=torch.uint8, device=dev)
            out_s = torch.empty((T, Nn // 256), dtype=torch.float32, device=dev)
        else:
            out = torch.empty((T, Nn // 2 if code == 1 else Nn), dtype=torch.bfloat16, device=dev)
        self._epoch += 1
        b = self._epoch & 1
        self._ag_calls[b] += 1
        team = self.heap.team()
        rc = _cu().mf_ag_gemm_fp8(C.byref(team), x_shard.data_ptr(), x_shard.stride(0), rows, wq.data_ptr(), ws.data_ptr(), out.data_ptr(),
                                  out.stride(0), out_s.data_ptr() if out_s is not None else None, Nn, K, self._ag[b], self._ags[b], self._ready[b],
                                  self._push[b].data_ptr(), self._epoch, self._ag_calls[b], status_word(dev).data_ptr(), sm_count(dev), code,
                                  torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"mf_ag_gemm_fp8 failed to launch ({rc})")
        return (out.view(torch.float8_e4m3fn), out_s) if code == 3 else out

    def gemm_rs_fp8(self, aq: torch.Tensor, a_scale: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, scale: float = 1.0,
                    out: torch.Tensor | None = None) -> torch.Tensor:
        """aq [T, K] e4m3 with a_scale [T, K/128] (full sequence, this rank's K-slice), wq [N, K] e4m3 with ws [N/128, K/128]
        -> this rank's [T/W, N] bf16 of sum_over_ranks(a . w^T) * scale."""
        T, K = aq.shape
        Nn = wq.shape[0]
        assert aq.is_contiguous() and a_scale.is_contiguous() and wq.is_contiguous() and ws.is_contiguous()
        assert T % (self.world * 128) == 0 and T <= self.max_tokens and Nn <= self.max_out and Nn % 256 == 0 and K % 128 == 0
        rows = T // self.world
        if out is None:
            out = torch.empty((rows, Nn), dtype=torch.bfloat16, device=aq.device)
        self._epoch += 1
        b = self._epoch & 1
        self._rs_calls[b] += 1
        team = self.heap.team()
        rc = _cu().mf_gemm_rs_fp8(C.byref(team), aq.data_ptr(), a_scale.data_ptr(), wq.data_ptr(), ws.data_ptr(), out.data_ptr(), out.stride(0), rows,
                                  Nn, K, self._land[b], self._cnt[b], self._epoch, self._rs_calls[b], float(scale),
                                  status_word(aq.device).data_ptr(), sm_count(aq.device), torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"mf_gemm_rs_fp8 failed to launch ({rc})")
        return out
