"""DeepEP-style expert-parallel communication buffer on the zbal symmetric heap.

    buf = zbal.Buffer(group, hidden=7168, num_experts=256, num_topk=8, num_max_tokens=4096)
    n_rank, _, n_expert, in_rank, _ = buf.get_dispatch_layout(topk_idx, num_experts)
    (recv_x, recv_scales), recv_expert, recv_w, counts, handle, ev = buf.dispatch(
        x, num_tokens_per_rank=n_rank, is_token_in_rank=in_rank, num_tokens_per_expert=n_expert,
        topk_idx=topk_idx, topk_weights=topk_w)
    y = my_expert_ffn(recv_x, recv_scales, counts)            # rows grouped by local expert
    out, _, ev = buf.combine(y, handle)                        # weighted sum back on the home ranks

Method names and argument order follow the reference (app/zbal/src/python/zbal/zbal_buffer.py:84-710).
What differs, and why:
  * Rows arrive as block-scaled fp8 e4m3 (1 x 128 scales) by default, the quantisation being fused into
    the push kernel; ``Buffer(..., use_fp8=False)`` moves bf16 rows unchanged. The reference's optional
    quantisation is int8 per token (DEEP_NORMAL_MODE_USE_INT8_QUANT).
  * The receive buffers live in the symmetric heap and the tensors returned by ``dispatch`` are views of
    them: they stay valid until the next ``dispatch`` of this buffer.
  * ``dispatch`` needs no host synchronisation when ``num_worst_tokens > 0``: the counts stay on the
    device and the views cover the worst case. Otherwise the per-expert counts are read back once
    (the reference reads the total back at the same point, adaptor/deepep/zbal_deepep.cpp:261-395).
  * The buffer shapes are fixed at construction (``hidden``, ``num_experts``, ``num_topk``,
    ``num_max_tokens``); DeepEP's byte-size hints are accepted and ignored.
  * ``fused_deep_moe`` takes fp8 weights with 128 x 128 block scales (see ``ops.moe.quantize_weight_fp8``)
    instead of int8 weights with per-channel scales.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, Optional, Tuple, Union

import torch
import torch.distributed as dist

from ..ops.heap import TeamC, _HeapBase, tensor_at
from ..ops import moe as moe_ops
from ..ops.moe import DispatchState, MoEComm
from . import _capi as K
from . import module as M
from .utils import Config, EventOverlap

_buffer_count = 0


class _CommHeap(_HeapBase):
    """The slice of the symmetric heap seen through one zbal communicator: offsets are relative to the
    communicator's slot, allocations come from the zbal allocator (identical offsets on every member as
    long as the members allocate in the same order, which constructing a Buffer collectively ensures)."""

    def __init__(self, comm):
        super().__init__()
        p = K.CommPropertyC()
        K.check(K.lib().zbal_comm_get_property(comm, C.byref(p)), "zbal_comm_get_property")
        out = M.bootstrap_output()
        self.world, self.rank, self.emu = int(p.groupSize), int(p.groupRank), False
        self.stride = int(p.rankStep) * int(out.symmetricSize)
        self._slot = int(p.signalGva)
        self.base = self._slot - self.rank * self.stride
        self._ptrs = []
        self._comm = comm

    def alloc(self, nbytes: int, align: int = 256) -> int:
        ptr = K.lib().zbal_pluggable_malloc(nbytes + align, 0, None)
        if not ptr:
            raise MemoryError(f"symmetric heap exhausted: {K.last_error()}")
        self._ptrs.append(ptr)
        aligned = (ptr + align - 1) // align * align
        return aligned - self._slot

    def free_all(self) -> None:
        for p in self._ptrs:
            K.lib().zbal_pluggable_free(p, 0, 0, None)
        self._ptrs.clear()

    def host_barrier(self) -> None:
        torch.cuda.synchronize()
        K.check(K.lib().zbal_barrier(self._comm, None), "zbal_barrier")
        torch.cuda.synchronize()


def pack_ue8m0(scales: torch.Tensor) -> torch.Tensor:
    """Power-of-two fp32 scales [rows, groups] -> their exponent bytes (UE8M0), four per int32: [rows, ceil(groups / 4)] int32,
    byte j of word w = exponent of group 4 w + j."""
    rows, groups = scales.shape
    e = ((scales.contiguous().view(torch.int32) >> 23) & 0xFF).to(torch.uint8)
    pad = (-groups) % 4
    if pad:
        e = torch.nn.functional.pad(e, (0, pad))
    return e.contiguous().view(torch.int32)


class Buffer:
    num_sms: int = 148

    def __init__(self, group: Optional[dist.ProcessGroup] = None, num_nvl_bytes: int = 0, num_rdma_bytes: int = 0,
                 low_latency_mode: bool = False, num_qps_per_rank: int = 12, allow_nvlink_for_low_latency_mode: bool = True,
                 allow_mnnvl: bool = False, *, hidden: int = 7168, num_experts: int = 256, num_topk: int = 8, num_max_tokens: int = 4096,
                 num_max_recv_tokens: Optional[int] = None, use_fp8: bool = True) -> None:
        global _buffer_count
        if not M.is_initialized():
            raise RuntimeError("zbal.Buffer needs zbal_init() (or a process group of backend 'zbal' that ran a collective)")
        out = M.bootstrap_output()
        if group is not None and dist.is_initialized():
            ranks = dist.get_process_group_ranks(group)
        else:
            ranks = list(range(out.worldSize))
        step = ranks[1] - ranks[0] if len(ranks) > 1 else 1
        if any(ranks[i + 1] - ranks[i] != step for i in range(len(ranks) - 1)):
            raise NotImplementedError("zbal.Buffer needs evenly spaced ranks")
        # a communicator of its own keeps the buffer's flags apart from everybody else's (the reference clones the group)
        o = K.CommOptionsC()
        o.name = f"zbal_buffer_{ranks[0]}:{ranks[-1]}:{step}_{_buffer_count}".encode()
        _buffer_count += 1
        o.firstRank, o.rankStep, o.groupSize = ranks[0], step, len(ranks)
        h = C.c_void_p()
        K.check(K.lib().zbal_comm_create(C.byref(o), C.byref(h)), "zbal_comm_create (buffer)")
        self._comm = h.value
        self._heap = _CommHeap(self._comm)
        self.rank, self.group_size, self.group = self._heap.rank, self._heap.world, group
        self.low_latency_mode = low_latency_mode
        self.hidden, self.num_experts, self.num_topk, self.num_max_tokens = hidden, num_experts, num_topk, num_max_tokens
        self.use_fp8 = use_fp8
        self._moe = MoEComm(self._heap, num_max_tokens, hidden, num_experts, num_topk, max_recv=num_max_recv_tokens, raw_bf16=not use_fp8)
        self._side = None   # second stream: the shared expert of fused_deep_moe runs there while the routed rows travel
        self._state: Optional[DispatchState] = None

    # ------------------------------------------------------------------ configuration helpers (DeepEP names)
    @staticmethod
    def get_dispatch_config(num_ranks: int) -> Config:
        return Config(Buffer.num_sms)

    @staticmethod
    def get_combine_config(num_ranks: int) -> Config:
        return Config(Buffer.num_sms)

    @staticmethod
    def set_num_sms(new_num_sms: int) -> None:
        assert new_num_sms > 0
        Buffer.num_sms = new_num_sms

    @staticmethod
    def capture() -> EventOverlap:
        ev = torch.cuda.Event()
        ev.record()
        return EventOverlap(ev)

    @staticmethod
    def get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int, num_experts: int) -> int:
        """Bytes of symmetric heap a low-latency buffer of this shape takes (receive rows, scales, origins, combine slots)."""
        recv = num_max_dispatch_tokens_per_rank * num_ranks * min(8, max(1, num_experts // num_ranks))
        return recv * (hidden + hidden // 128 * 4 + 16) + num_max_dispatch_tokens_per_rank * 8 * hidden * 2 + num_ranks * num_experts * 4

    def destroy(self) -> None:
        if self._moe is not None:
            torch.cuda.synchronize()
            self._moe = None
            self._heap.free_all()
            K.lib().zbal_comm_destroy(self._comm, 0)

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _before(previous_event):
        if previous_event is not None and getattr(previous_event, "event", None) is not None:
            torch.cuda.current_stream().wait_event(previous_event.event)

    @staticmethod
    def _after(async_finish: bool, keep=None) -> EventOverlap:
        if not async_finish:
            return EventOverlap(None)
        ev = torch.cuda.Event()
        ev.record()
        return EventOverlap(ev, keep)

    # ------------------------------------------------------------------ normal mode
    def get_dispatch_layout(self, topk_idx: torch.Tensor, num_experts: int, previous_event: Optional[EventOverlap] = None,
                            async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """-> (num_tokens_per_rank [ranks] int32, None, num_tokens_per_expert [experts] int32, is_token_in_rank [T, ranks] bool, event)"""
        assert num_experts == self.num_experts
        self._before(previous_event)
        idx, tpe, tpr, sidx, inr = self._moe.get_dispatch_layout(topk_idx)
        self._layout = (topk_idx, idx, tpe, tpr, sidx, inr)
        return tpr, None, tpe, inr.bool(), self._after(async_finish)

    def dispatch(self, x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]], handle: Optional[Tuple] = None,
                 num_tokens_per_rank: Optional[torch.Tensor] = None, num_tokens_per_rdma_rank: Optional[torch.Tensor] = None,
                 is_token_in_rank: Optional[torch.Tensor] = None, num_tokens_per_expert: Optional[torch.Tensor] = None,
                 topk_idx: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None, expert_alignment: int = 1,
                 num_worst_tokens: int = 0, config: Optional[Config] = None, previous_event: Optional[EventOverlap] = None,
                 async_finish: bool = False, allocate_on_comm_stream: bool = False,
                 dispatch_wait_recv_cost_stats: Optional[torch.Tensor] = None):
        """-> (recv_x or (recv_x_fp8, recv_scales), recv_expert_idx [rows] int64, recv_weights [rows] fp32,
               num_recv_tokens_per_expert_list, handle, event). Rows are grouped by local expert."""
        if isinstance(x, tuple):
            # pre-quantised rows (e4m3 + one scale per 128 elements): turned back into bf16, which is exact for e4m3 values
            # times a power-of-two scale, and quantised again by the push kernel (the same values come out when the scales
            # follow this library's rule: the smallest power of two that brings the group's largest value under 448)
            xq, xs = x
            T0, H0 = xq.shape
            x = (xq.view(torch.float8_e4m3fn).float().view(T0, H0 // 128, 128) * xs.float().view(T0, H0 // 128, 1)).view(T0, H0).to(torch.bfloat16)
        self._before(previous_event)
        moe = self._moe
        if handle is not None:
            # cached layout: the routing of an earlier dispatch is reused for another tensor (DeepEP's handle argument);
            # no layout, no count exchange, the rows land where the first call's rows landed
            st = moe.dispatch_cached(x, handle[4], handle[2])
            topk_weights = handle[2]
        else:
            if topk_idx is None or topk_weights is None:
                raise ValueError("topk_idx and topk_weights must be given")
            st = moe.dispatch(x, topk_idx, topk_weights)
        self._state = st
        El = moe.El
        if num_worst_tokens > 0:
            rows, counts = min(num_worst_tokens, moe.max_recv), []
        else:
            counts = st.recv_per_expert.tolist()  # the one host read of this call
            rows = sum(counts)
        info = moe.recv_info()[:rows]
        recv_w = info[:, 3].contiguous().view(torch.float32)
        # local expert of every row, from the group boundaries (device side, no sync)
        bounds = st.row_off[1:El + 1].to(torch.int64)
        recv_e = torch.bucketize(torch.arange(rows, device=x.device), bounds, right=True).clamp_(max=El - 1)
        rx = moe.recv_x()[:rows]
        recv_x = (rx, moe.recv_scale()[:rows]) if self.use_fp8 else rx
        handle = (st.is_token_in_rank, st.topk_idx, topk_weights, st.put_off, st)
        return recv_x, recv_e, recv_w, counts, handle, self._after(async_finish)

    def combine(self, x: torch.Tensor, handle: Tuple, topk_weights: Optional[torch.Tensor] = None,
                bias: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor], None] = None, config: Optional[Config] = None,
                previous_event: Optional[EventOverlap] = None, async_finish: bool = False, allocate_on_comm_stream: bool = False,
                combine_send_cost_stats: Optional[torch.Tensor] = None):
        """x: [rows, hidden] bf16 in the row order ``dispatch`` delivered. The rows are multiplied by the routing
        weights that travelled with them and summed per token on the token's home rank (the reference's combine
        does the same weighted sum, ops/dispatch_combine_normal/zbal_kernel_combine_normal.h:180-606).
        -> (combined_x [T, hidden] bf16, None, event)"""
        self._before(previous_event)
        st: DispatchState = handle[4]
        self._moe.combine_push(x, st, weighted=True)
        out = self._moe.combine(st)
        if bias is not None:   # one tensor or a pair, [T, hidden], added to the combined rows (DeepEP's bias argument)
            for b in (bias if isinstance(bias, (tuple, list)) else (bias,)):
                if b is not None:
                    out.add_(b.to(out.dtype))
        return out, None, self._after(async_finish)

    # ------------------------------------------------------------------ low-latency mode
    def clean_low_latency_buffer(self, num_max_dispatch_tokens_per_rank: int, hidden: int, num_experts: int) -> None:
        """Nothing to clean: flags carry call numbers that only grow, no buffer has to be zeroed between calls."""

    def low_latency_dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, num_max_dispatch_tokens_per_rank: int, num_experts: int,
                             cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None, use_fp8: bool = True,
                             round_scale: bool = False, use_ue8m0: bool = False, async_finish: bool = False,
                             return_recv_hook: bool = False, topk_weights: Optional[torch.Tensor] = None):
        """One cooperative kernel: layout, count exchange, quantise + push, wait for every peer's rows.
        -> ((recv_x, recv_scales) or recv_x, recv_count [local experts] int32, handle, event, hook).
        Rows are packed by local expert (``handle[1]`` holds the group offsets); the routing weights may be
        given here (they travel with the rows) or later to ``low_latency_combine``."""
        assert num_experts == self.num_experts and x.shape[0] <= min(num_max_dispatch_tokens_per_rank, self.num_max_tokens)
        assert use_fp8 == self.use_fp8, "the row format is fixed when the Buffer is built"
        # round_scale: the scales of this library are always powers of two, nothing to switch. use_ue8m0: they are handed
        # out as their exponent bytes, four per int32 along the last dimension (DeepEP's packed form)
        moe = self._moe
        w = topk_weights if topk_weights is not None else torch.ones(topk_idx.shape, dtype=torch.float32, device=x.device)
        st = moe.ll_dispatch(x, topk_idx, w)
        self._state = st
        if cumulative_local_expert_recv_stats is not None:
            cumulative_local_expert_recv_stats.add_(st.recv_per_expert)
        recv_x = (moe.recv_x(), moe.recv_scale()) if self.use_fp8 else moe.recv_x()
        if use_ue8m0 and self.use_fp8:
            recv_x = (recv_x[0], pack_ue8m0(recv_x[1]))
        handle = (st, st.row_off, num_max_dispatch_tokens_per_rank, self.hidden, num_experts, topk_weights is not None)
        hook: Callable = (lambda: None)
        return recv_x, st.recv_per_expert, handle, self._after(async_finish), hook

    def low_latency_combine(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, handle: tuple,
                            zero_copy: bool = False, async_finish: bool = False, return_recv_hook: bool = False,
                            out: Optional[torch.Tensor] = None):
        """x: [rows, hidden] bf16 in the packed row order of ``low_latency_dispatch``. One cooperative kernel:
        push home, signal + wait, weighted sum. -> (combined_x, event, hook)"""
        st: DispatchState = handle[0]
        moe = self._moe
        if not handle[5]:
            # the weights did not travel with the rows: they are applied on the home side
            y = moe.ll_combine(x.reshape(-1, self.hidden), st, weighted=False, out=out, home_weights=topk_weights)
            return y, self._after(async_finish), (lambda: None)
        y = moe.ll_combine(x.reshape(-1, self.hidden), st, weighted=True, out=out)
        return y, self._after(async_finish), (lambda: None)

    # ------------------------------------------------------------------ fused path
    def fused_deep_moe(self, x: torch.Tensor, topk_idx: torch.Tensor, gmm1_permuted_weight: torch.Tensor,
                       gmm1_permuted_weight_scale: torch.Tensor, gmm2_weight: torch.Tensor, gmm2_weight_scale: torch.Tensor,
                       topk_weights: torch.Tensor, num_experts: int, shared_expert_num: int = 0, shared_expert_rank_num: int = 0,
                       quant_mode: int = 0, num_max_dispatch_tokens_per_rank: int = 0, is_tensor_list: bool = False,
                       expert_smooth_scales: Optional[torch.Tensor] = None, share_gmm1_weight: Optional[torch.Tensor] = None,
                       share_gmm1_scale: Optional[torch.Tensor] = None, share_gmm2_weight: Optional[torch.Tensor] = None,
                       share_gmm2_scale: Optional[torch.Tensor] = None, share_smooth_scales: Optional[torch.Tensor] = None,
                       x_active_mask: Optional[torch.Tensor] = None, share_gmm1_h_len: int = 0, fuse_mode: int = 0,
                       **unused) -> Tuple[torch.Tensor, torch.Tensor]:
        """dispatch (fp8 quant fused) -> grouped GEMM1 + SwiGLU -> requant -> grouped GEMM2 with the weighted
        push home fused into its epilogue -> slot reduce. gmm1 weights: [local experts, 2I, H] fp8, gate/up
        tile-interleaved (``ops.moe.interleave_gate_up_fp8``) with [.., 2I/128, H/128] scales; gmm2: [.., H, I].
        ``x_active_mask`` ([T] bool): rows that are False take no part (padding of a decode batch): they are sent to no
        expert and their output rows are zero.
        ``expert_smooth_scales`` ([H] fp32, the reference's SMOOTH_QUANT flag): every row is multiplied by it inside the
        dispatch kernel, before quantisation; gmm1's weights carry the inverse factors.
        ``share_gmm1_weight`` .. ``share_gmm2_scale`` (the SHARED_EXPERT flag): one dense expert applied to every active row
        of x on this rank, in the expert weights' format (share_gmm1_weight [2 Is, H] tile-interleaved per 128 with
        [2 Is/128, H/128] scales, share_gmm2_weight [H, Is] with [H/128, Is/128]); it runs on a second stream while the
        routed rows travel, and its result is added to the combined rows. ``share_smooth_scales`` is its smooth-quant vector.
        ``is_tensor_list``: the routed weights arrive as lists of per-expert tensors. shared_expert_num,
        shared_expert_rank_num, share_gmm1_h_len (read from the weight's shape) and fuse_mode are accepted and ignored, as
        the reference's wrapper does (app/zbal/src/python/zbal/zbal_buffer.py:611-700).
        -> (output [T, H] bf16, tokens received per local expert)"""
        assert self.use_fp8, "the fused path runs on fp8 rows"
        if is_tensor_list:
            gmm1_permuted_weight, gmm1_permuted_weight_scale, gmm2_weight, gmm2_weight_scale = (
                torch.stack(list(t)) if isinstance(t, (list, tuple)) else t
                for t in (gmm1_permuted_weight, gmm1_permuted_weight_scale, gmm2_weight, gmm2_weight_scale))
        if x_active_mask is not None:
            topk_idx = topk_idx.masked_fill(~x_active_mask.to(torch.bool).view(-1, 1), -1)   # the kernels skip negative ids
        moe = self._moe
        smooth = None
        if expert_smooth_scales is not None:
            smooth = expert_smooth_scales.to(torch.float32).contiguous().view(-1)
        shared = None
        if share_gmm1_weight is not None and share_gmm1_weight.numel() > 0:
            assert share_gmm1_scale is not None and share_gmm2_weight is not None and share_gmm2_scale is not None, \
                "the shared expert needs both weights and both scale tensors"
            main = torch.cuda.current_stream()
            if self._side is None:
                self._side = torch.cuda.Stream()
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                ssm = None if share_smooth_scales is None else share_smooth_scales.to(torch.float32).contiguous().view(-1)
                shared = moe_ops.dense_ffn_fp8(x, share_gmm1_weight, share_gmm1_scale, share_gmm2_weight, share_gmm2_scale, smooth=ssm)
                if x_active_mask is not None:
                    shared.masked_fill_(~x_active_mask.to(torch.bool).view(-1, 1), 0)
        st = moe.dispatch(x, topk_idx, topk_weights, smooth=smooth)
        moe.expert_ffn(st, gmm1_permuted_weight, gmm1_permuted_weight_scale, gmm2_weight, gmm2_weight_scale)
        out = moe.combine(st)
        if shared is not None:
            torch.cuda.current_stream().wait_stream(self._side)
            shared.record_stream(torch.cuda.current_stream())   # allocated under the side stream, last used on this one
            out.add_(shared)
        return out, st.recv_per_expert
