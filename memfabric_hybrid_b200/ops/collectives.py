"""Collectives on a symmetric heap (sm_100a kernels in csrc/kernels/mf_coll.cu).

    comm = Communicator(heap, stage_bytes=32 << 20)
    comm.all_reduce(x, scale=1 / world, out_dtype=torch.bfloat16)     # fused x(1/world) + cast
    comm.reduce_scatter(x), comm.all_gather(x), comm.broadcast(x, root), comm.all_to_all_v(...),
    comm.send(x, peer) / comm.recv(x, peer), comm.barrier()

Every rank must issue the same sequence of calls (the flag epochs advance in lockstep). With an
``EmulatedHeap`` the tensors carry a leading ``world`` dimension and one launch runs all ranks.
Algorithm choice follows the message size: one-shot all-reduce up to 256 KiB, two-shot above; the
number of CTAs grows with the size (the analogue of the reference's per-size block-count table,
zbal_kernel_utils.h:117-152).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N
from .heap import TeamC, _HeapBase

DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2, torch.int32: 3}
OPS = {"sum": 0, "max": 1, "min": 2, "prod": 3}
ONE_SHOT_MAX = 256 << 10
DIRECT_MIN = 256 << 10  # above this, buffers that live in the heap are used in place (no staging copies)


class CollArgsC(C.Structure):
    _fields_ = [("team", TeamC), ("inp", C.c_uint64), ("out", C.c_uint64), ("in_rank_stride", C.c_uint64),
                ("out_rank_stride", C.c_uint64), ("n", C.c_uint64), ("stage_a", C.c_uint64), ("stage_b", C.c_uint64),
                ("scale", C.c_float), ("op", C.c_int), ("epoch", C.c_uint32), ("zero_copy", C.c_uint32),
                ("root", C.c_uint32), ("algo", C.c_uint32), ("part_stride", C.c_uint64)]


class A2AArgsC(C.Structure):
    _fields_ = [("team", TeamC), ("inp", C.c_uint64), ("out", C.c_uint64), ("in_rank_stride", C.c_uint64),
                ("out_rank_stride", C.c_uint64), ("meta", C.c_uint64), ("meta_rank_stride", C.c_uint64),
                ("in_bytes", C.c_uint64), ("stage_a", C.c_uint64), ("epoch", C.c_uint32)]


class P2PArgsC(C.Structure):
    _fields_ = [("team", TeamC), ("buf", C.c_uint64), ("bytes", C.c_uint64), ("stage_off", C.c_uint64),
                ("peer", C.c_uint32), ("epoch", C.c_uint32), ("channel", C.c_uint32)]


_lib = None


def _cu():
    global _lib
    if _lib is None:
        l = N.cuda()
        l.mf_coll_launch.restype = C.c_int
        l.mf_coll_launch.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(CollArgsC), C.c_int, C.c_int, C.c_void_p]
        l.mf_coll_alltoallv.restype = C.c_int
        l.mf_coll_alltoallv.argtypes = [C.POINTER(A2AArgsC), C.c_int, C.c_int, C.c_void_p]
        l.mf_coll_send.restype = C.c_int
        l.mf_coll_send.argtypes = [C.POINTER(P2PArgsC), C.c_int, C.c_void_p]
        l.mf_coll_recv.restype = C.c_int
        l.mf_coll_recv.argtypes = [C.POINTER(P2PArgsC), C.c_int, C.c_void_p]
        l.mf_coll_barrier.restype = C.c_int
        l.mf_coll_barrier.argtypes = [C.POINTER(TeamC), C.c_uint32, C.c_uint32, C.c_void_p]
        l.mf_coll_wait_flag.restype = C.c_int
        l.mf_coll_wait_flag.argtypes = [C.POINTER(TeamC), C.c_uint64, C.c_uint32, C.c_void_p]
        l.mf_coll_args_size.restype = C.c_uint
        assert l.mf_coll_args_size() == C.sizeof(CollArgsC), "CollArgs layout differs between Python and CUDA"
        _lib = l
    return _lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: launch failed with code {rc}")


class Communicator:
    def __init__(self, heap: _HeapBase, stage_bytes: int = 32 << 20, max_ctas: int | None = None):
        self.heap = heap
        self.world = heap.world
        self.rank = heap.rank
        self.stage_bytes = (stage_bytes + 4095) // 4096 * 4096
        # two sets of (A, B): calls alternate so that no trailing synchronisation is needed
        self._sets = [(heap.alloc(self.stage_bytes), heap.alloc(self.stage_bytes)) for _ in range(2)]
        self._p2p_stage = None  # landing areas for send/recv, allocated on first use
        self._p2p_bytes = 4 << 20
        self._epoch = 0
        self._p2p_epochs = {}
        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        self.max_ctas = min(max_ctas or sms, 256)
        if heap.emu:
            # a cooperative launch of world x ctas blocks must be co-resident
            self.max_ctas = max(1, min(self.max_ctas, sms // heap.world))  # one 512-thread CTA per SM is always resident
        self._meta = None
        self._a2a_meta = {}  # split tables of all_to_all_v already on the device, by their content
        # Variant choice when the heap has an NVLink multicast alias: None = by size and world (see _multicast), True /
        # False = always / never (the benchmark measures both).
        self.multicast = None

    # ------------------------------------------------------------------ helpers
    def _next(self):
        self._epoch += 1
        return self._epoch, self._sets[self._epoch & 1]

    def _ctas(self, nbytes: int) -> int:
        if nbytes <= 16 << 10:
            c = 1
        elif nbytes <= 64 << 10:
            c = 4
        elif nbytes <= 256 << 10:
            c = 16
        elif nbytes <= 1 << 20:
            c = 32
        elif nbytes <= 8 << 20:
            c = 64
        else:
            c = self.max_ctas
        return max(1, min(c, self.max_ctas))

    @property
    def no_multicast(self) -> bool:
        return self.multicast is False

    @no_multicast.setter
    def no_multicast(self, v: bool) -> None:
        self.multicast = False if v else None

    def _multicast(self, kind: str, nbytes: int) -> bool:
        """Whether a direct-mode collective goes through the multicast alias (in-switch reduction / one store reaching
        every rank) or through peer loads and stores. Measured on B200 + NVSwitch: with 2 GPUs the switch has nothing to
        save (one peer) and the peer kernels are faster at every size; from 4 GPUs on the in-switch all-reduce wins once
        the message is large enough to be bandwidth-bound; reduce-scatter and all-gather move the same bytes either way."""
        if self.heap.mc_base == 0:
            return False
        if self.multicast is not None:
            return bool(self.multicast)
        if kind == "all_reduce":
            # 8 GPUs: ahead from 1 MiB on (1 MiB 25 vs 27 us, 256 MiB 645 vs 799 us); 4 GPUs: from 64 MiB on (32 MiB 119 vs 113 us,
            # 256 MiB 641 vs 711 us)
            return (self.world >= 8 and nbytes >= (1 << 20)) or (self.world >= 4 and nbytes >= (64 << 20))
        if kind == "reduce_scatter":
            # 8 GPUs: the in-switch load-reduce is ahead between 1 MiB and 256 MiB (16 MiB 45 vs 49 us, 256 MiB 410 vs 430 us) and
            # behind at 1 GiB (1501 vs 1477 us); at 4 GPUs the peer loads win from 16 MiB on
            return self.world >= 8 and (1 << 20) <= nbytes <= (256 << 20)
        return False

    def _local(self, t: torch.Tensor):
        """(address of rank 0's buffer, per-rank stride in bytes, per-rank element count)."""
        assert t.is_cuda and t.is_contiguous(), "collective tensors must be contiguous CUDA tensors"
        if self.heap.emu:
            assert t.shape[0] == self.world, "emulated collectives take tensors with a leading world dimension"
            return t.data_ptr(), t.stride(0) * t.element_size(), t[0].numel()
        return t.data_ptr(), 0, t.numel()

    def _args(self, x, out, n, epoch, stage, scale=1.0, op="sum", root=0, algo=0) -> CollArgsC:
        xin, xs, _ = self._local(x)
        xo, os_, _ = self._local(out)
        return CollArgsC(self.heap.team(), xin, xo, xs, os_, n, stage[0], stage[1], float(scale), OPS[op], epoch, 0, root, algo, 0)

    def _in_heap(self, t: torch.Tensor) -> bool:
        """True when the tensor lies inside this rank's slice of a real symmetric heap (peers can reach it)."""
        if self.heap.emu:
            return False
        lo = self.heap.base + self.rank * self.heap.stride
        p = t.data_ptr()
        return lo <= p and p + t.numel() * t.element_size() <= lo + getattr(self.heap, "usable", self.heap.stride)

    def _empty_like(self, x: torch.Tensor, per_rank_numel: int, dtype: torch.dtype) -> torch.Tensor:
        if self.heap.emu:
            return torch.empty((self.world, per_rank_numel), dtype=dtype, device=x.device)
        return torch.empty((per_rank_numel,), dtype=dtype, device=x.device)

    # ------------------------------------------------------------------ collectives
    def barrier(self, channel: int = 0) -> None:
        self._epoch += 1
        team = self.heap.team()
        _check(_cu().mf_coll_barrier(C.byref(team), channel, self._epoch, _stream()), "barrier")

    def all_reduce(self, x: torch.Tensor, out: torch.Tensor | None = None, op: str = "sum", scale: float = 1.0,
                   out_dtype: torch.dtype | None = None, algo: str | None = None) -> torch.Tensor:
        od = out_dtype or x.dtype
        _, _, n = self._local(x)
        if out is None:
            out = self._empty_like(x, n, od)
        es = x.element_size()
        if algo in (None, "direct") and n * es > DIRECT_MIN and self._in_heap(x) and self._in_heap(out):
            epoch, stage = self._next()
            args = self._args(x, out, n, epoch, stage, scale, op, 0, 1)
            # with a multicast alias of the heap the switch does the adding (sum of one floating type, no cast)
            mc = op == "sum" and od == x.dtype and x.dtype != torch.int32 and self._multicast("all_reduce", n * es)
            args.zero_copy = 3 if mc else 2
            _check(_cu().mf_coll_launch(0, DT[x.dtype], DT[od], C.byref(args), self._ctas(n * es), 512, _stream()), "all_reduce (direct)")
            return out
        assert algo != "direct", "direct mode needs input and output inside the symmetric heap"
        piece = self.stage_bytes // max(es, out.element_size())
        piece -= piece % (8 * self.world)
        a = {"oneshot": 0, "twoshot": 1, None: None}[algo]
        done = 0
        while done < n:
            cnt = min(piece, n - done)
            use = a if a is not None else (0 if cnt * es <= ONE_SHOT_MAX else 1)
            epoch, stage = self._next()
            args = self._args(x, out, cnt, epoch, stage, scale, op, 0, use)
            args.inp += done * es
            args.out += done * out.element_size()
            _check(_cu().mf_coll_launch(0, DT[x.dtype], DT[od], C.byref(args), self._ctas(cnt * es), 512, _stream()), "all_reduce")
            done += cnt
        return out

    def reduce_scatter(self, x: torch.Tensor, out: torch.Tensor | None = None, op: str = "sum", scale: float = 1.0,
                       out_dtype: torch.dtype | None = None) -> torch.Tensor:
        od = out_dtype or x.dtype
        _, _, n = self._local(x)
        assert n % self.world == 0, "reduce_scatter input must divide by the world size"
        m = n // self.world
        if out is None:
            out = self._empty_like(x, m, od)
        es = x.element_size()
        if n * es > DIRECT_MIN and self._in_heap(x):
            epoch, stage = self._next()
            args = self._args(x, out, n, epoch, stage, scale, op)
            mc = op == "sum" and x.dtype != torch.int32 and self._multicast("reduce_scatter", n * es) and \
                (od == x.dtype or (x.dtype == torch.float32 and od == torch.bfloat16))
            args.zero_copy = 3 if mc else 2
            _check(_cu().mf_coll_launch(1, DT[x.dtype], DT[od], C.byref(args), self._ctas(n * es), 512, _stream()), "reduce_scatter (direct)")
            return out
        # a piece is a column block [c0, c1) of the [world, m] view: staged as world rows of (c1 - c0)
        piece = self.stage_bytes // es // self.world
        piece -= piece % 8
        if m <= piece:
            epoch, stage = self._next()
            args = self._args(x, out, n, epoch, stage, scale, op)
            _check(_cu().mf_coll_launch(1, DT[x.dtype], DT[od], C.byref(args), self._ctas(n * es), 512, _stream()), "reduce_scatter")
            return out
        xv = x.view(self.world, self.world, m) if self.heap.emu else x.view(self.world, m)
        c0 = 0
        while c0 < m:
            c1 = min(m, c0 + piece)
            part = xv[..., c0:c1].contiguous()
            po = self.reduce_scatter(part.view(self.world, -1) if self.heap.emu else part.view(-1), None, op, scale, od)
            (out.view(self.world, m) if self.heap.emu else out)[..., c0:c1] = po
            c0 = c1
        return out

    def all_gather(self, x: torch.Tensor, out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
                   scale: float = 1.0) -> torch.Tensor:
        od = out_dtype or x.dtype
        _, _, m = self._local(x)
        if out is None:
            out = self._empty_like(x, m * self.world, od)
        oes = out.element_size()
        if m * self.world * oes > DIRECT_MIN and self._in_heap(out):
            epoch, stage = self._next()
            args = self._args(x, out, m, epoch, stage, scale)
            args.zero_copy = 3 if self._multicast("all_gather", m * self.world * oes) else 2
            _check(_cu().mf_coll_launch(2, DT[x.dtype], DT[od], C.byref(args), self._ctas(m * self.world * oes), 512, _stream()),
                   "all_gather (direct)")
            return out
        piece = self.stage_bytes // oes // self.world
        piece -= piece % 8
        if m <= piece:
            epoch, stage = self._next()
            args = self._args(x, out, m, epoch, stage, scale)
            _check(_cu().mf_coll_launch(2, DT[x.dtype], DT[od], C.byref(args), self._ctas(m * self.world * oes), 512, _stream()),
                   "all_gather")
            return out
        ov = out.view(self.world, self.world, m) if self.heap.emu else out.view(self.world, m)
        xv = x.view(self.world, m) if self.heap.emu else x
        c0 = 0
        while c0 < m:
            c1 = min(m, c0 + piece)
            po = self.all_gather(xv[..., c0:c1].contiguous(), None, od, scale)
            ov[..., c0:c1] = po.view(self.world, self.world, c1 - c0) if self.heap.emu else po.view(self.world, c1 - c0)
            c0 = c1
        return out

    def broadcast(self, x: torch.Tensor, root: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
        """Every rank passes a tensor of the same shape; the root's content lands in ``out`` (default: in place)."""
        out = x if out is None else out
        _, _, n = self._local(x)
        es = x.element_size()
        unit = 4 if es == 4 else 2
        assert (n * es) % unit == 0
        total = n * es // unit
        piece = self.stage_bytes // unit
        piece -= piece % 8
        done = 0
        while done < total:
            cnt = min(piece, total - done)
            epoch, stage = self._next()
            args = self._args(x, out, cnt, epoch, stage, 1.0, "sum", root)
            args.inp += done * unit
            args.out += done * unit
            _check(_cu().mf_coll_launch(3, 2 if unit == 4 else 0, 2 if unit == 4 else 0, C.byref(args), self._ctas(cnt * unit), 512,
                                        _stream()), "broadcast")
            done += cnt
        return out

    def all_to_all_v(self, x: torch.Tensor, out: torch.Tensor, send_counts, send_offsets, recv_counts, recv_offsets) -> torch.Tensor:
        """Counts and offsets in ELEMENTS of x.dtype, one entry per peer; in emulation they are [world][world] lists."""
        es = x.element_size()
        xin, xs, n = self._local(x)
        xo, os_, n_out = self._local(out)
        # pieces land in the RECEIVER's staging area before they are copied to `out`
        assert n_out * es + 4096 <= self.stage_bytes, "all_to_all_v receive buffer exceeds the staging area"
        rows = self.world if self.heap.emu else 1
        # the split table on the device; a layer that repeats its splits (the common case) pays the upload once
        key = (es, repr(send_counts), repr(send_offsets), repr(recv_counts), repr(recv_offsets)) if not self.heap.emu else None
        cached = self._a2a_meta.get(key) if key is not None else None
        if cached is None:
            meta = torch.empty((rows, self.world, 4), dtype=torch.int64)
            for r in range(rows):
                sc, so, rcnt, ro = (v[r] for v in (send_counts, send_offsets, recv_counts, recv_offsets)) if self.heap.emu else \
                    (send_counts, send_offsets, recv_counts, recv_offsets)
                for p in range(self.world):
                    meta[r, p, 0] = int(so[p]) * es
                    meta[r, p, 1] = int(sc[p]) * es
                    meta[r, p, 2] = int(ro[p]) * es
                    meta[r, p, 3] = int(rcnt[p]) * es
            cached = meta.to(x.device, non_blocking=False)
            if key is not None:
                if len(self._a2a_meta) >= 32:
                    self._a2a_meta.clear()
                self._a2a_meta[key] = cached
        self._meta = cached
        epoch, stage = self._next()
        args = A2AArgsC(self.heap.team(), xin, xo, xs, os_, self._meta.data_ptr(), self.world * 32 if self.heap.emu else 0,
                        n * es, stage[0], epoch)
        ctas = self._ctas(n * es)   # a cooperative launch: max_ctas keeps the grid co-resident
        _check(_cu().mf_coll_alltoallv(C.byref(args), ctas, 512, _stream()), "all_to_all_v")
        return out

    # ------------------------------------------------------------------ point to point (real heaps only)
    def _p2p(self, peer: int, sending: bool):
        assert not self.heap.emu, "send/recv need separate ranks"
        if self._p2p_stage is None:
            # one landing area per possible sender, same layout on every rank
            self._p2p_stage = self.heap.alloc(self._p2p_bytes * self.world)
        src, dst = (self.rank, peer) if sending else (peer, self.rank)
        key = (src, dst)
        self._p2p_epochs[key] = self._p2p_epochs.get(key, 0) + 1
        # channel: flags live in the barrier-flag rows 16..63, one row per sender rank (world <= 16 here)
        channel = 16 + src % 48
        return self._p2p_epochs[key], channel, self._p2p_stage + src * self._p2p_bytes

    def send(self, x: torch.Tensor, peer: int) -> None:
        nbytes = x.numel() * x.element_size()
        done = 0
        while done < nbytes:
            cnt = min(self._p2p_bytes, nbytes - done)
            epoch, channel, stage = self._p2p(peer, True)
            args = P2PArgsC(self.heap.team(), x.data_ptr() + done, cnt, stage, peer, epoch, channel)
            _check(_cu().mf_coll_send(C.byref(args), min(self._ctas(cnt), 32), _stream()), "send")
            done += cnt

    def recv(self, x: torch.Tensor, peer: int) -> None:
        nbytes = x.numel() * x.element_size()
        done = 0
        while done < nbytes:
            cnt = min(self._p2p_bytes, nbytes - done)
            epoch, channel, stage = self._p2p(peer, False)
            args = P2PArgsC(self.heap.team(), x.data_ptr() + done, cnt, stage, peer, epoch, channel)
            _check(_cu().mf_coll_recv(C.byref(args), min(self._ctas(cnt), 32), _stream()), "recv")
            done += cnt

    # ------------------------------------------------------------------ derived
    def gather(self, x: torch.Tensor, root: int = 0) -> torch.Tensor:
        g = self.all_gather(x)
        return g

    def scatter(self, x: torch.Tensor, root: int = 0) -> torch.Tensor:
        """x: [world * m] on every rank (only the root's content matters); returns this rank's m elements."""
        full = self.broadcast(x.clone(), root)
        if self.heap.emu:
            m = full.shape[1] // self.world
            return torch.stack([full[r, r * m:(r + 1) * m] for r in range(self.world)])
        m = full.numel() // self.world
        return full[self.rank * m:(self.rank + 1) * m].clone()

    def wait_flag_probe(self, flag_off: int, epoch: int) -> None:
        """Launches a wait on a flag of the own slot (used to demonstrate the bounded-wait status path)."""
        team = self.heap.team()
        _check(_cu().mf_coll_wait_flag(C.byref(team), flag_off, epoch, _stream()), "wait_flag")
