"""Expert-parallel MoE on the symmetric heap: layout -> notify -> fused fp8 dispatch -> grouped expert
GEMMs (tcgen05, fp8 block-scaled) with SwiGLU and combine fused into their epilogues -> slot reduce.

    moe = MoEComm(heap, max_tokens=4096, hidden=7168, experts=256, topk=8)
    st  = moe.dispatch(x, topk_idx, topk_w)                  # device-resident counts, no host sync
    moe.expert_ffn(st, w1, w1_scale, w2, w2_scale)           # gate/up+SwiGLU, requant, down+weighted push
    y   = moe.combine(st)                                    # [T, hidden] bf16

Calls must alternate dispatch ... combine on every rank: the wait inside combine is what guarantees that
peers finished reading the receive buffers before the next dispatch overwrites them.
Kernels: csrc/kernels/mf_moe.cu, csrc/kernels/mf_gemm_fp8.cu.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import torch

from .. import _native as N
from .gemm import sm_count, status_word
from .heap import TeamC, _HeapBase


_CANARY_BYTES = 4096
_CANARY_WORD = 0x5AFEC0DE - (1 << 32) if 0x5AFEC0DE >= (1 << 31) else 0x5AFEC0DE


class MoeShapeC(C.Structure):
    _fields_ = [("T", C.c_int), ("K", C.c_int), ("E", C.c_int), ("H", C.c_int), ("max_recv", C.c_int)]


class MoeHeapC(C.Structure):
    _fields_ = [("counts", C.c_uint64), ("recv_x", C.c_uint64), ("recv_scale", C.c_uint64), ("recv_info", C.c_uint64),
                ("comb", C.c_uint64), ("flags", C.c_uint64)]


class DispatchArgsC(C.Structure):
    _fields_ = [("team", TeamC), ("hp", MoeHeapC), ("sh", MoeShapeC), ("x", C.c_void_p), ("topk_idx", C.c_void_p),
                ("topk_w", C.c_void_p), ("send_idx", C.c_void_p), ("put_off", C.c_void_p), ("done_count", C.c_void_p),
                ("epoch", C.c_uint32), ("seq", C.c_uint32), ("status", C.c_void_p), ("raw_bf16", C.c_int),
                ("smooth", C.c_void_p)]


_lib = None


def _cu():
    global _lib
    if _lib is None:
        l = N.cuda()
        P, vp, ci = C.POINTER, C.c_void_p, C.c_int
        l.mf_moe_layout.restype = ci
        l.mf_moe_layout.argtypes = [vp, ci, ci, ci, ci, vp, vp, vp, vp, vp]
        l.mf_moe_notify.restype = ci
        l.mf_moe_notify.argtypes = [P(TeamC), P(MoeHeapC), ci, vp, vp, vp, vp, vp, C.c_uint32, vp]
        l.mf_moe_dispatch.restype = ci
        l.mf_moe_dispatch.argtypes = [P(DispatchArgsC), ci, vp]
        l.mf_moe_wait_all.restype = ci
        l.mf_moe_wait_all.argtypes = [P(TeamC), P(MoeHeapC), ci, C.c_uint32, vp, vp]
        l.mf_moe_signal_all.restype = ci
        l.mf_moe_signal_all.argtypes = [P(TeamC), P(MoeHeapC), ci, C.c_uint32, vp]
        l.mf_moe_combine_reduce.restype = ci
        l.mf_moe_combine_reduce.argtypes = [P(TeamC), P(MoeHeapC), P(MoeShapeC), vp, vp, ci, vp]
        l.mf_moe_combine_push.restype = ci
        l.mf_moe_combine_push.argtypes = [P(TeamC), P(MoeHeapC), vp, C.c_int64, vp, ci, ci, ci, ci, vp]
        l.mf_moe_ll_dispatch.restype = ci
        l.mf_moe_ll_dispatch.argtypes = [P(DispatchArgsC), vp, vp, vp, vp, vp, ci, vp]
        l.mf_moe_ll_combine.restype = ci
        l.mf_moe_ll_combine.argtypes = [P(TeamC), P(MoeHeapC), P(MoeShapeC), vp, C.c_int64, vp, ci, vp, vp, vp, C.c_uint32, vp, vp, ci, vp]
        l.mf_quant_rows_fp8.restype = ci
        l.mf_quant_rows_fp8.argtypes = [vp, C.c_int64, vp, ci, vp, vp, ci, vp]
        l.mf_grouped_gemm_fp8.restype = ci
        l.mf_grouped_gemm_fp8.argtypes = [vp, vp, ci, vp, vp, vp, ci, ci, ci, vp, C.c_int64, ci, P(TeamC), vp, C.c_uint64, ci, vp, ci, vp]
        l.mf_grouped_gemm_fp8_mx.restype = ci
        l.mf_grouped_gemm_fp8_mx.argtypes = [vp, vp, ci, vp, vp, vp, ci, ci, ci, vp, C.c_int64, vp, ci, P(TeamC), vp, C.c_uint64, ci, vp, ci, vp]
        l.mf_grouped_gemm_fp8_mx_supported.restype = ci
        l.mf_grouped_gemm_fp8_mx_supported.argtypes = [ci, ci, ci, ci]
        _lib = l
    return _lib


def _s() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ok(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: launch failed ({rc})")


def quantize_weight_fp8(w: torch.Tensor):
    """[..., N, K] bf16/fp32 -> (fp8 e4m3 [..., N, K], fp32 scales [..., N/128, K/128]); 128 x 128 blocks.
    Every scale is a power of two (the smallest with amax / scale <= 448): the block-scaled tensor-core MMA takes
    such a scale as one UE8M0 byte, and the activation quantisers of this library produce the same kind."""
    *lead, Nn, K = w.shape
    assert Nn % 128 == 0 and K % 128 == 0
    blk = w.float().reshape(*lead, Nn // 128, 128, K // 128, 128)
    amax = blk.abs().amax(dim=(-3, -1), keepdim=True).clamp_min(1e-30)
    scale = torch.exp2(torch.ceil(torch.log2(amax / 448.0))).clamp_min(2.0 ** -126)
    q = (blk / scale).clamp(-448, 448).to(torch.float8_e4m3fn).reshape(*lead, Nn, K)
    return q.contiguous(), scale.reshape(*lead, Nn // 128, K // 128).contiguous()


def gate_up_tile(experts: int, intermediate: int, hidden: int) -> int:
    """Rows per gate / up run that ``expert_ffn`` expects in the first GEMM's weights: 128 when the 128 x 256
    block-scaled kernel takes the layer's shapes, else 64 (the 128 x 128 kernel that applies the scales in registers)."""
    try:
        cu = _cu()
    except (RuntimeError, OSError):
        return 128
    ok = cu.mf_grouped_gemm_fp8_mx_supported(experts, 2 * intermediate, hidden, 3) and \
        cu.mf_grouped_gemm_fp8_mx_supported(experts, hidden, intermediate, 2)
    return 128 if ok else 64


def interleave_gate_up_fp8(w1q: torch.Tensor, tile: int | None = None) -> torch.Tensor:
    """[G, 2I, K] (gate rows then up rows) -> per 2 x tile rows: tile gate rows followed by their tile up rows.
    ``tile`` defaults to what ``expert_ffn`` expects for these shapes (``gate_up_tile``)."""
    G, two_i, K = w1q.shape
    i = two_i // 2
    if tile is None:
        tile = gate_up_tile(G, i, K)
    assert i % tile == 0
    gate = w1q[:, :i].reshape(G, i // tile, tile, K)
    up = w1q[:, i:].reshape(G, i // tile, tile, K)
    return torch.stack([gate, up], dim=2).reshape(G, two_i, K).contiguous()


_row_bounds_cache: dict = {}


def _row_bounds(T: int, dev) -> torch.Tensor:
    """[0, T] on the device (the one-group row offsets of ``dense_ffn_fp8``), made once per T: building it is a synchronous copy."""
    key = (T, str(dev))
    t = _row_bounds_cache.get(key)
    if t is None:
        if len(_row_bounds_cache) > 64:
            _row_bounds_cache.clear()
        t = torch.tensor([0, T], dtype=torch.int32, device=dev)
        _row_bounds_cache[key] = t
    return t


def dense_ffn_fp8(x: torch.Tensor, w1q: torch.Tensor, w1s: torch.Tensor, w2q: torch.Tensor, w2s: torch.Tensor,
                  smooth: torch.Tensor | None = None, sms: int | None = None) -> torch.Tensor:
    """One dense SwiGLU expert on every row of x (the shared expert of a DeepSeek-style layer):
    y = (silu(x W1g^T) * (x W1u^T)) W2^T with block-scaled fp8 tensor-core GEMMs. x [T, H] bf16;
    w1q [2I, H] e4m3 with gate / up rows interleaved per 128 (``interleave_gate_up_fp8(w[None], 128)[0]``), w1s [2I/128, H/128]
    in original row order; w2q [H, I], w2s [H/128, I/128]. Three launches: row quantisation, gate/up GEMM whose epilogue
    applies SwiGLU and re-quantises, down GEMM. ``smooth`` ([H] fp32) multiplies the rows before quantisation."""
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    T, H = x.shape
    two_i = w1q.shape[0]
    I = two_i // 2
    assert w1q.shape == (two_i, H) and w2q.shape == (H, I) and two_i % 256 == 0 and H % 256 == 0 and I % 128 == 0
    cu = _cu()
    dev = x.device
    stw = status_word(dev).data_ptr()
    sms = sms or sm_count(dev)
    if smooth is not None:
        x = (x.float() * smooth.view(1, H)).to(torch.bfloat16)
    rows = _row_bounds(T, dev)
    xq = torch.empty((T, H), dtype=torch.uint8, device=dev)
    xs = torch.empty((T, H // 128), dtype=torch.float32, device=dev)
    _ok(cu.mf_quant_rows_fp8(x.data_ptr(), H, rows[1:].data_ptr(), H, xq.data_ptr(), xs.data_ptr(), sms * 4, _s()), "quant_rows_fp8")
    hq = torch.empty((T, I), dtype=torch.uint8, device=dev)
    hs = torch.empty((T, I // 128), dtype=torch.float32, device=dev)
    _ok(cu.mf_grouped_gemm_fp8_mx(xq.data_ptr(), xs.data_ptr(), T, w1q.data_ptr(), w1s.data_ptr(), rows.data_ptr(), 1, two_i, H,
                                  hq.data_ptr(), I, hs.data_ptr(), 3, None, None, 0, 1, stw, sms, _s()), "grouped_gemm_fp8_mx (shared gate/up)")
    y = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    _ok(cu.mf_grouped_gemm_fp8_mx(hq.data_ptr(), hs.data_ptr(), T, w2q.data_ptr(), w2s.data_ptr(), rows.data_ptr(), 1, H, I,
                                  y.data_ptr(), H, None, 0, None, None, 0, 1, stw, sms, _s()), "grouped_gemm_fp8_mx (shared down)")
    return y


@dataclass
class DispatchState:
    T: int
    topk_idx: torch.Tensor       # [T, K] int32
    send_idx: torch.Tensor
    tokens_per_expert: torch.Tensor
    tokens_per_rank: torch.Tensor
    is_token_in_rank: torch.Tensor
    recv_per_expert: torch.Tensor  # [El] int32, device
    row_off: torch.Tensor          # [El + 1] int32, device; row_off[-1] = rows received
    put_off: torch.Tensor
    src_off: torch.Tensor
    epoch: int


class MoEComm:
    def __init__(self, heap: _HeapBase, max_tokens: int, hidden: int, experts: int, topk: int, max_recv: int | None = None,
                 intermediate: int | None = None, raw_bf16: bool = False):
        assert not heap.emu and hidden % 128 == 0 and experts % heap.world == 0
        self.heap, self.world, self.rank = heap, heap.world, heap.rank
        self.T, self.H, self.E, self.K = max_tokens, hidden, experts, topk
        self.El = experts // self.world
        self.max_recv = max_recv or max_tokens * self.world * min(topk, self.El)
        self.dev = torch.device("cuda", torch.cuda.current_device())
        hp = MoeHeapC()
        hp.counts = heap.alloc(self.world * experts * 4, 256)
        hp.flags = heap.alloc(4 * 16 * 4, 256)
        self.raw_bf16 = raw_bf16  # rows travel as bf16 instead of block-scaled fp8
        # Debug aid (MF_MOE_CANARY=1): guard words between the receive areas that peers write into. A peer that stores past
        # the end of a row, a scale array or a combine slot lands in a guard first; check_canaries() finds it.
        self._canary = os.environ.get("MF_MOE_CANARY", "0") not in ("", "0")
        self._guards = []

        def guard():
            if self._canary:
                self._guards.append(heap.alloc(_CANARY_BYTES, 256))

        guard()
        hp.recv_x = heap.alloc(self.max_recv * hidden * (2 if raw_bf16 else 1), 1024)
        guard()
        hp.recv_scale = heap.alloc(self.max_recv * (hidden // 128) * 4, 256)
        guard()
        hp.recv_info = heap.alloc(self.max_recv * 16, 256)
        guard()
        hp.comb = heap.alloc(max_tokens * topk * hidden * 2, 1024)
        guard()
        for off in self._guards:
            heap.view(off, (_CANARY_BYTES // 4,), torch.int32).fill_(_CANARY_WORD)
        self.hp = hp
        heap.view(hp.flags, (4 * 16,), torch.int32).zero_()
        heap.view(hp.counts, (self.world * experts,), torch.int32).zero_()
        self._epoch = 0
        self._done = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self._dispatches = 0
        self._ll_done = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self._ll_grid = None
        self._grid = sm_count(self.dev)
        self._inter = intermediate
        self._h = self._hq = self._hs = None
        torch.cuda.synchronize()
        if hasattr(heap, "host_barrier"):
            heap.host_barrier()

    def check_canaries(self) -> None:
        """Raises when a guard word between the receive areas of THIS rank was overwritten (MF_MOE_CANARY=1)."""
        for i, off in enumerate(self._guards):
            g = self.heap.view(off, (_CANARY_BYTES // 4,), torch.int32)
            bad = (g != _CANARY_WORD).nonzero()
            if bad.numel():
                raise RuntimeError(f"MoE receive area: guard {i} (slot offset {off:#x}) was overwritten at word {int(bad[0])}: "
                                   "a peer stored outside its row, scale or combine slot")

    # views of the receive area (valid rows: state.row_off[-1])
    def recv_x(self) -> torch.Tensor:
        if self.raw_bf16:
            return self.heap.view(self.hp.recv_x, (self.max_recv, self.H), torch.bfloat16)
        return self.heap.view(self.hp.recv_x, (self.max_recv, self.H), torch.uint8).view(torch.float8_e4m3fn)

    def recv_scale(self) -> torch.Tensor:
        return self.heap.view(self.hp.recv_scale, (self.max_recv, self.H // 128), torch.float32)

    def recv_info(self) -> torch.Tensor:
        return self.heap.view(self.hp.recv_info, (self.max_recv, 4), torch.int32)

    def _shape(self, T: int) -> MoeShapeC:
        return MoeShapeC(T, self.K, self.E, self.H, self.max_recv)

    # ------------------------------------------------------------------ stages
    def get_dispatch_layout(self, topk_idx: torch.Tensor):
        T = topk_idx.shape[0]
        idx = topk_idx.to(torch.int32).contiguous()
        tpe = torch.empty(self.E, dtype=torch.int32, device=self.dev)
        tpr = torch.empty(self.world, dtype=torch.int32, device=self.dev)
        sidx = torch.zeros(T * self.K, dtype=torch.int32, device=self.dev)
        inr = torch.empty((T, self.world), dtype=torch.uint8, device=self.dev)
        _ok(_cu().mf_moe_layout(idx.data_ptr(), T, self.K, self.E, self.world, tpe.data_ptr(), tpr.data_ptr(), sidx.data_ptr(),
                                inr.data_ptr(), _s()), "moe_layout")
        return idx, tpe, tpr, sidx, inr

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, smooth: torch.Tensor | None = None) -> DispatchState:
        """smooth: optional [H] fp32 factors every row is multiplied by before it is quantised (smooth quant; the matching
        weights carry the inverse factors). fp8 rows only."""
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[1] == self.H and x.shape[0] <= self.T
        if smooth is not None:
            assert not self.raw_bf16 and smooth.dtype == torch.float32 and smooth.is_contiguous() and smooth.numel() == self.H
        T = x.shape[0]
        idx, tpe, tpr, sidx, inr = self.get_dispatch_layout(topk_idx)
        self._epoch += 1
        team = self.heap.team()
        rpe = torch.empty(self.El, dtype=torch.int32, device=self.dev)
        row_off = torch.empty(self.El + 1, dtype=torch.int32, device=self.dev)
        put_off = torch.empty(self.E, dtype=torch.int32, device=self.dev)
        src_off = torch.empty(self.El * self.world, dtype=torch.int32, device=self.dev)
        _ok(_cu().mf_moe_notify(C.byref(team), C.byref(self.hp), self.E, tpe.data_ptr(), rpe.data_ptr(), row_off.data_ptr(),
                                put_off.data_ptr(), src_off.data_ptr(), self._epoch, _s()), "moe_notify")
        w = topk_w.to(torch.float32).contiguous()
        self._dispatches += 1
        a = DispatchArgsC(team, self.hp, self._shape(T), x.data_ptr(), idx.data_ptr(), w.data_ptr(), sidx.data_ptr(), put_off.data_ptr(),
                          self._done.data_ptr(), self._epoch, self._dispatches, status_word(self.dev).data_ptr(), 1 if self.raw_bf16 else 0,
                          smooth.data_ptr() if smooth is not None else None)
        self._keep = (w, idx, smooth)
        # one CTA per SM on every call: the completion counter of the kernel counts CTAs
        _ok(_cu().mf_moe_dispatch(C.byref(a), self._grid, _s()), "moe_dispatch")
        _ok(_cu().mf_moe_wait_all(C.byref(team), C.byref(self.hp), 0, self._epoch, status_word(self.dev).data_ptr(), _s()), "moe_wait")
        return DispatchState(T, idx, sidx, tpe, tpr, inr, rpe, row_off, put_off, src_off, self._epoch)

    def dispatch_cached(self, x: torch.Tensor, st: DispatchState, topk_w: torch.Tensor) -> DispatchState:
        """Pushes another tensor along the routing of an earlier ``dispatch`` (same top-k table, same positions in the
        receivers' buffers): no layout pass and no count exchange. Every rank must make the same call. -> a state for
        ``expert_ffn`` / ``combine`` that shares the first call's tables."""
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape == (st.T, self.H)
        import dataclasses
        self._epoch += 1
        self._dispatches += 1
        team = self.heap.team()
        w = topk_w.to(torch.float32).contiguous()   # the weights travel with the rows again
        a = DispatchArgsC(team, self.hp, self._shape(st.T), x.data_ptr(), st.topk_idx.data_ptr(), w.data_ptr(), st.send_idx.data_ptr(),
                          st.put_off.data_ptr(), self._done.data_ptr(), self._epoch, self._dispatches, status_word(self.dev).data_ptr(),
                          1 if self.raw_bf16 else 0, None)
        self._keep = (w, st.topk_idx, None)
        _ok(_cu().mf_moe_dispatch(C.byref(a), self._grid, _s()), "moe_dispatch")
        _ok(_cu().mf_moe_wait_all(C.byref(team), C.byref(self.hp), 0, self._epoch, status_word(self.dev).data_ptr(), _s()), "moe_wait")
        return dataclasses.replace(st, epoch=self._epoch)

    def expert_ffn(self, st: DispatchState, w1q: torch.Tensor, w1s: torch.Tensor, w2q: torch.Tensor, w2s: torch.Tensor) -> None:
        """w1q [El, 2I, H] fp8 tile-interleaved (interleave_gate_up_fp8), w1s [El, 2I/128, H/128] in ORIGINAL row order;
        w2q [El, H, I] fp8, w2s [El, H/128, I/128]. The result rows are pushed, weighted, to the tokens' home ranks."""
        El, two_i, H = w1q.shape
        I = two_i // 2
        assert El == self.El and H == self.H and w2q.shape == (El, H, I)
        if self._hq is None or self._hq.shape[1] != I:
            self._h = None
            self._hq = torch.empty((self.max_recv, I), dtype=torch.uint8, device=self.dev)
            self._hs = torch.empty((self.max_recv, I // 128), dtype=torch.float32, device=self.dev)
        team = self.heap.team()
        stw = status_word(self.dev).data_ptr()
        cu = _cu()
        if cu.mf_grouped_gemm_fp8_mx_supported(El, two_i, H, 3) and cu.mf_grouped_gemm_fp8_mx_supported(El, H, I, 2):
            # two launches: gate/up + SwiGLU + re-quantisation to fp8 in the first GEMM's epilogue, down projection +
            # weighted push to the tokens' home ranks in the second's; w1q interleaved with tile 128
            _ok(cu.mf_grouped_gemm_fp8_mx(self.heap.ptr(self.rank, self.hp.recv_x), self.heap.ptr(self.rank, self.hp.recv_scale), self.max_recv,
                                          w1q.data_ptr(), w1s.data_ptr(), st.row_off.data_ptr(), El, two_i, H, self._hq.data_ptr(), I,
                                          self._hs.data_ptr(), 3, None, None, 0, self.K, stw, self._grid, _s()), "grouped_gemm_fp8_mx (gate/up)")
            _ok(cu.mf_grouped_gemm_fp8_mx(self._hq.data_ptr(), self._hs.data_ptr(), self.max_recv, w2q.data_ptr(), w2s.data_ptr(),
                                          st.row_off.data_ptr(), El, H, I, None, 0, None, 2, C.byref(team),
                                          self.heap.ptr(self.rank, self.hp.recv_info), self.hp.comb, self.K, stw, self._grid, _s()),
                "grouped_gemm_fp8_mx (down+combine)")
            _ok(cu.mf_moe_signal_all(C.byref(team), C.byref(self.hp), 1, st.epoch, _s()), "moe_signal")
            return
        # shapes the 128 x 256 kernel does not take (N not a multiple of 256): the 128 x 128 kernel that applies the
        # scales in registers, with w1q interleaved with tile 64 and a separate re-quantisation pass
        if self._h is None:
            self._h = torch.empty((self.max_recv, I), dtype=torch.bfloat16, device=self.dev)
        _ok(cu.mf_grouped_gemm_fp8(self.heap.ptr(self.rank, self.hp.recv_x), self.heap.ptr(self.rank, self.hp.recv_scale), self.max_recv,
                                   w1q.data_ptr(), w1s.data_ptr(), st.row_off.data_ptr(), El, two_i, H, self._h.data_ptr(), I, 1, None, None,
                                   0, self.K, stw, self._grid, _s()), "grouped_gemm_fp8 (gate/up)")
        _ok(cu.mf_quant_rows_fp8(self._h.data_ptr(), I, st.row_off[El:].data_ptr(), I, self._hq.data_ptr(), self._hs.data_ptr(),
                                 self._grid * 4, _s()), "quant_rows_fp8")
        _ok(cu.mf_grouped_gemm_fp8(self._hq.data_ptr(), self._hs.data_ptr(), self.max_recv, w2q.data_ptr(), w2s.data_ptr(),
                                   st.row_off.data_ptr(), El, H, I, None, 0, 2, C.byref(team), self.heap.ptr(self.rank, self.hp.recv_info),
                                   self.hp.comb, self.K, stw, self._grid, _s()), "grouped_gemm_fp8 (down+combine)")
        _ok(cu.mf_moe_signal_all(C.byref(team), C.byref(self.hp), 1, st.epoch, _s()), "moe_signal")

    def combine(self, st: DispatchState, out: torch.Tensor | None = None) -> torch.Tensor:
        team = self.heap.team()
        if out is None:
            out = torch.empty((st.T, self.H), dtype=torch.bfloat16, device=self.dev)
        _ok(_cu().mf_moe_wait_all(C.byref(team), C.byref(self.hp), 1, st.epoch, status_word(self.dev).data_ptr(), _s()), "moe_wait")
        sh = self._shape(st.T)
        _ok(_cu().mf_moe_combine_reduce(C.byref(team), C.byref(self.hp), C.byref(sh), st.topk_idx.data_ptr(), out.data_ptr(),
                                        min(st.T, self._grid * 4), _s()), "moe_combine_reduce")
        if self._canary:
            torch.cuda.synchronize()
            self.check_canaries()
        return out

    # ------------------------------------------------------------------ standalone combine (caller ran its own expert FFN)
    def combine_push(self, y: torch.Tensor, st: DispatchState, weighted: bool = True) -> None:
        """y: [>= rows received, hidden] bf16, row r answering row r of the receive buffers. Pushes every row to
        the combine slot of its token on the token's home rank and raises the combine flag."""
        assert y.dtype == torch.bfloat16 and y.shape[1] == self.H and y.stride(1) == 1
        team = self.heap.team()
        _ok(_cu().mf_moe_combine_push(C.byref(team), C.byref(self.hp), y.data_ptr(), y.stride(0), st.row_off[self.El:].data_ptr(), self.H,
                                      self.K, 1 if weighted else 0, self._grid * 2, _s()), "moe_combine_push")
        _ok(_cu().mf_moe_signal_all(C.byref(team), C.byref(self.hp), 1, st.epoch, _s()), "moe_signal")

    # ------------------------------------------------------------------ low-latency pair (one cooperative launch each)
    def _ll_setup(self):
        if self._ll_grid is None:
            self._ll_grid = max(1, min(self.T, self._grid))  # fixed for the life of the object
            d = self.dev
            i32 = torch.int32
            self._ll_epoch = torch.zeros(1, dtype=i32, device=d)   # call counter of the pair, advanced by the kernel
            self._ll_bufs = dict(sidx=torch.zeros(self.T * self.K, dtype=i32, device=d), tpe=torch.zeros(self.E, dtype=i32, device=d),
                                 rpe=torch.zeros(self.El, dtype=i32, device=d), row_off=torch.zeros(self.El + 1, dtype=i32, device=d),
                                 put_off=torch.zeros(self.E, dtype=i32, device=d), src_off=torch.zeros(self.El * self.world, dtype=i32, device=d))
            hp = MoeHeapC.from_buffer_copy(self.hp)
            hp.flags += 2 * 16 * 4  # flag rows 2 and 3 belong to the low-latency pair
            self._ll_hp = hp

    def ll_dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, smooth: torch.Tensor | None = None) -> DispatchState:
        """One cooperative launch. The outputs live in buffers owned by this object (overwritten by the next call)
        and nothing depends on host-side counters, so the call may be captured in a CUDA graph and replayed."""
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[1] == self.H and x.shape[0] <= self.T
        T = x.shape[0]
        self._ll_setup()
        idx = topk_idx if topk_idx.dtype == torch.int32 and topk_idx.is_contiguous() else topk_idx.to(torch.int32).contiguous()
        w = topk_w if topk_w.dtype == torch.float32 and topk_w.is_contiguous() else topk_w.to(torch.float32).contiguous()
        b = self._ll_bufs
        a = DispatchArgsC(self.heap.team(), self._ll_hp, self._shape(T), x.data_ptr(), idx.data_ptr(), w.data_ptr(), b["sidx"].data_ptr(),
                          b["put_off"].data_ptr(), self._ll_done.data_ptr(), 0, 0, status_word(self.dev).data_ptr(),
                          1 if self.raw_bf16 else 0, smooth.data_ptr() if smooth is not None else None)
        self._keep = (w, idx, smooth)
        _ok(_cu().mf_moe_ll_dispatch(C.byref(a), b["tpe"].data_ptr(), b["rpe"].data_ptr(), b["row_off"].data_ptr(), b["src_off"].data_ptr(),
                                     self._ll_epoch.data_ptr(), self._ll_grid, _s()), "moe_ll_dispatch")
        return DispatchState(T, idx, b["sidx"], b["tpe"], None, None, b["rpe"], b["row_off"], b["put_off"], b["src_off"], -1)

    def ll_combine(self, y: torch.Tensor, st: DispatchState, weighted: bool = True, out: torch.Tensor | None = None,
                   home_weights: torch.Tensor | None = None) -> torch.Tensor:
        """weighted: multiply each row by the weight that travelled with it; home_weights: [T, K] fp32 applied on the home rank instead."""
        assert y.dtype == torch.bfloat16 and y.shape[1] == self.H and y.stride(1) == 1
        if out is None:
            out = torch.empty((st.T, self.H), dtype=torch.bfloat16, device=self.dev)
        team, sh = self.heap.team(), self._shape(st.T)
        hw = home_weights.to(torch.float32).contiguous() if home_weights is not None else None
        _ok(_cu().mf_moe_ll_combine(C.byref(team), C.byref(self._ll_hp), C.byref(sh), y.data_ptr(), y.stride(0), st.row_off[self.El:].data_ptr(),
                                    1 if weighted else 0, st.topk_idx.data_ptr(), hw.data_ptr() if hw is not None else None, out.data_ptr(), 0, self._ll_epoch.data_ptr(),
                                    status_word(self.dev).data_ptr(),
                                    self._ll_grid or self._grid, _s()), "moe_ll_combine")
        return out
