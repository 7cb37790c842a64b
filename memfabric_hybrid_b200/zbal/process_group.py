"""``torch.distributed`` backend "zbal": collectives of CUDA tensors run as zbal kernels over NVLink peer
memory; what zbal does not implement falls back to NCCL.

    import zbal                                   # registers the backend
    dist.init_process_group("zbal", rank=r, world_size=w)
    dist.all_reduce(t)                            # -> zbal_all_reduce on the group's side stream

Implemented: allreduce, _allgather_base, allgather, gather, broadcast, scatter, reduce_scatter,
_reduce_scatter_base, barrier, alltoall_base, send, recv (the method set of the reference's backend,
app/zbal/src/csrc/adaptor/pytorch_npu/zbal_pytorch_process_group.h:130-166). Everything else, tensors of
types the kernels cannot reduce, and groups whose ranks are not evenly spaced go to an internal NCCL
process group (the reference falls back to its vendor library in the same way, selected by an
environment list; here the list is ZBAL_NCCL_OP, or the reference's name ZBAL_HCCL_OP: comma separated op names, for forcing the fallback).

Stream discipline (zbal_pytorch_process_group.cpp:312-367 of the reference): one side stream per group;
it first waits on an event recorded on the caller's stream, the operation is enqueued, an end event is
recorded into the returned Work; ``Work.wait()`` makes the CALLER's stream wait on that event, the host
does not block. With ZBAL_OP_DEFAULT_STREAM=1 operations run on the caller's stream directly.

Two implementations with the same behaviour: the native ``c10d::Backend`` (csrc/c10d/zbal_process_group.cpp, built as
``lib/_zbal_c10d.so``; the default) and the ``ProcessGroup`` subclass below (``ZBAL_PG_IMPL=python``, or when the
extension is not built). The native one builds its NCCL / gloo fallbacks through a factory given by ``_create_native``.

Group naming: ``zbal_<first>:<last>:<stride>_group_<n>``; point-to-point communicators are 2-member
groups named ``"<low>:<high>"`` created on first use, the lower world rank being member 0.
"""
from __future__ import annotations

import ctypes as C
import os
from datetime import timedelta

import torch
import torch.distributed as dist
from torch._C._distributed_c10d import ReduceOp

from . import _capi as K
from . import module as M

_OPS = {ReduceOp.SUM: K.OP_SUM, ReduceOp.MAX: K.OP_MAX, ReduceOp.MIN: K.OP_MIN, ReduceOp.PRODUCT: K.OP_PROD}
_group_counters: dict = {}
_live = []
_native_ext = None


def _forget_all() -> None:
    if _native_ext:
        _native_ext.forget_all()
    for pg in list(_live):
        pg._comm = None
        pg._p2p.clear()
    _live.clear()


class WorkZBAL(dist._Work):
    """Completion handle: an event on the stream the operation ran on."""

    def __init__(self, event, result, keep=None):
        super().__init__()
        self._event = event
        self._result = result
        self._keep = keep
        self._future = None

    def wait(self, timeout=timedelta(seconds=0)):
        if self._event is not None:
            torch.cuda.current_stream().wait_event(self._event)
        return True

    def is_completed(self):
        return self._event is None or self._event.query()

    def is_success(self):
        return True

    def synchronize(self):
        self.wait()

    def result(self):
        return self._result

    def get_future(self):
        if self._future is None:
            devs = sorted({t.device for t in (self._result if isinstance(self._result, (list, tuple)) else [self._result])
                           if isinstance(t, torch.Tensor) and t.is_cuda}, key=str)
            self._future = torch.futures.Future(devices=devs) if devs else torch.futures.Future()
            self.wait()                            # the current stream waits for the operation, then the future records it
            self._future.set_result(self._result)  # marked complete at once, like the reference (cpp:352-355)
        return self._future


class ProcessGroupZBAL(dist.ProcessGroup):
    def __init__(self, store, rank: int, size: int, global_ranks=None, timeout=None):
        super().__init__(rank, size)
        self._store = store
        self._rank, self._size = rank, size
        self._ranks = list(global_ranks) if global_ranks else list(range(size))
        self._timeout = timeout or timedelta(minutes=30)
        self._comm = None
        self._p2p = {}
        self._nccl = None
        self._gloo = None
        self._stream = None
        self._strided = self._check_strided()
        self._forced = {s.strip() for s in os.environ.get("ZBAL_NCCL_OP", os.environ.get("ZBAL_HCCL_OP", "")).split(",") if s.strip()}
        self._own_stream = os.environ.get("ZBAL_OP_DEFAULT_STREAM", os.environ.get("ZBAL_OP_DEFUALT_STREAM", "0")) != "1"
        _live.append(self)
        if M.is_initialized():
            self._communicator()

    # ------------------------------------------------------------------ plumbing
    def getBackendName(self):
        return "zbal"

    def name(self):
        return "zbal"

    def __repr__(self):
        return f"ProcessGroupZBAL(rank={self._rank}, size={self._size}, ranks={self._ranks})"

    def _check_strided(self) -> bool:
        r = self._ranks
        if len(r) <= 1:
            return True
        step = r[1] - r[0]
        return step > 0 and all(r[i + 1] - r[i] == step for i in range(len(r) - 1))

    def _ensure_init(self) -> None:
        if M.is_initialized():
            return
        # lazy bootstrap from the environment, as the reference does on the first collective
        world = int(os.environ.get("WORLD_SIZE", self._size))
        rank = int(os.environ.get("RANK", self._rank))
        dev = torch.cuda.current_device()
        size = int(os.environ.get("ZBAL_DEVICE_MEM_SIZE", str(4 << 30)))
        M.zbal_init(world, dev, rank, size, start_config_server=True)

    def _communicator(self):
        if self._comm is not None:
            return self._comm
        if not self._strided:
            return None
        self._ensure_init()
        l = K.lib()
        out = M.bootstrap_output()
        first, last = self._ranks[0], self._ranks[-1]
        step = self._ranks[1] - first if self._size > 1 else 1
        if self._size == out.worldSize and first == 0 and step == 1 and not any(pg is not self and pg._comm == l.zbal_comm_get_global() for pg in _live):
            self._comm = l.zbal_comm_get_global()
            return self._comm
        key = (first, last, step)
        n = _group_counters.get(key, 0)
        _group_counters[key] = n + 1
        o = K.CommOptionsC()
        o.name = f"zbal_{first}:{last}:{step}_group_{n}".encode()
        o.firstRank, o.rankStep, o.groupSize = first, step, self._size
        h = C.c_void_p()
        K.check(l.zbal_comm_create(C.byref(o), C.byref(h)), f"zbal_comm_create({o.name.decode()})")
        self._comm = h.value
        return self._comm

    def _p2p_comm(self, peer_group_rank: int):
        """(communicator of the pair, my rank in it, the peer's rank in it)."""
        me_w, peer_w = self._ranks[self._rank], self._ranks[peer_group_rank]
        lo, hi = min(me_w, peer_w), max(me_w, peer_w)
        if (lo, hi) not in self._p2p:
            self._ensure_init()
            l = K.lib()
            name = f"{lo}:{hi}".encode()
            h = l.zbal_comm_get_by_name(name)
            if not h:
                o = K.CommOptionsC()
                o.name = name
                o.firstRank, o.rankStep, o.groupSize = lo, hi - lo, 2
                hh = C.c_void_p()
                K.check(l.zbal_comm_create(C.byref(o), C.byref(hh)), f"zbal_comm_create({name.decode()})")
                h = hh.value
            self._p2p[(lo, hi)] = h
        return self._p2p[(lo, hi)], (0 if me_w == lo else 1), (1 if me_w == lo else 0)

    def _fallback(self, t=None):
        """NCCL for CUDA tensors; gloo for host tensors (object collectives of torch.distributed use them)."""
        if isinstance(t, (list, tuple)):
            t = t[0] if t else None
            if isinstance(t, (list, tuple)):
                t = t[0] if t else None
        if t is not None and not t.is_cuda:
            if self._gloo is None:
                self._gloo = dist.ProcessGroupGloo(dist.PrefixStore("zbal_gloo_fallback/", self._store), self._rank, self._size,
                                                   timeout=self._timeout)
            return self._gloo
        if self._nccl is None:
            opts = dist.ProcessGroupNCCL.Options()
            self._nccl = dist.ProcessGroupNCCL(dist.PrefixStore("zbal_nccl_fallback/", self._store), self._rank, self._size, opts)
        return self._nccl

    def _use_zbal(self, op: str, *tensors) -> bool:
        if op in self._forced or not self._strided:
            return False
        return all(t.is_cuda and t.is_contiguous() for t in tensors)

    def _run(self, tensors, fn, result):
        """Applies the stream discipline around ``fn(stream_handle)``."""
        cur = torch.cuda.current_stream()
        if not self._own_stream:
            fn(cur.cuda_stream)
            ev = torch.cuda.Event()
            ev.record(cur)
            return WorkZBAL(ev, result)
        if self._stream is None:
            self._stream = torch.cuda.Stream()
        ready = torch.cuda.Event()
        ready.record(cur)
        self._stream.wait_event(ready)
        for t in tensors:
            t.record_stream(self._stream)
        fn(self._stream.cuda_stream)
        done = torch.cuda.Event()
        done.record(self._stream)
        return WorkZBAL(done, result, keep=tensors)

    # ------------------------------------------------------------------ collectives
    def allreduce(self, tensors, opts=None):
        t = tensors[0]
        op = _OPS.get(opts.reduceOp if opts is not None else ReduceOp.SUM)
        avg = opts is not None and opts.reduceOp == ReduceOp.AVG
        if avg:
            op = K.OP_SUM
        if len(tensors) != 1 or op is None or t.dtype not in K.REDUCIBLE or not self._use_zbal("allreduce", t):
            return self._fallback(tensors).allreduce(tensors, opts) if opts is not None else self._fallback(tensors).allreduce(tensors)
        comm, l = self._communicator(), K.lib()
        scale = 1.0 / self._size if avg else 1.0

        def go(s):
            K.check(l.zbal_all_reduce_scaled(t.data_ptr(), t.data_ptr(), t.numel(), K.DT[t.dtype], K.DT[t.dtype], op, scale, comm, s),
                    "zbal_all_reduce")
        return self._run([t], go, tensors)

    def allreduce_coalesced(self, tensors, opts=None):
        return self._fallback(tensors).allreduce_coalesced(tensors, opts)

    def _allgather_base(self, output, input, opts=None):
        if not self._use_zbal("_allgather_base", output, input) or (input.numel() * input.element_size()) % 2:
            return self._fallback(input)._allgather_base(output, input, opts) if opts is not None else self._fallback(input)._allgather_base(output, input)
        comm, l = self._communicator(), K.lib()

        def go(s):
            K.check(l.zbal_all_gather(input.data_ptr(), output.data_ptr(), input.numel(), K.DT[input.dtype], comm, s), "zbal_all_gather")
        return self._run([input, output], go, output)

    def allgather(self, output_tensors, input_tensors, opts=None):
        inp, outs = input_tensors[0], output_tensors[0]
        if len(input_tensors) != 1 or inp.dtype not in K.DT or not self._use_zbal("allgather", inp) or (inp.numel() * inp.element_size()) % 2 or \
                any(o.numel() != inp.numel() for o in outs):
            return self._fallback(input_tensors).allgather(output_tensors, input_tensors, opts) if opts is not None else \
                self._fallback(input_tensors).allgather(output_tensors, input_tensors)
        comm, l = self._communicator(), K.lib()
        flat = torch.empty((self._size, inp.numel()), dtype=inp.dtype, device=inp.device)

        def go(s):
            K.check(l.zbal_all_gather(inp.data_ptr(), flat.data_ptr(), inp.numel(), K.DT[inp.dtype], comm, s), "zbal_all_gather")
            with torch.cuda.stream(torch.cuda.ExternalStream(s)):
                for r, o in enumerate(outs):
                    o.copy_(flat[r].view_as(o))
        return self._run([inp, flat] + list(outs), go, output_tensors)

    def allgather_into_tensor_coalesced(self, outputs, inputs, opts=None):
        return self._fallback(inputs).allgather_into_tensor_coalesced(outputs, inputs, opts)

    def gather(self, output_tensors, input_tensors, opts=None):
        inp = input_tensors[0]
        root = opts.rootRank if opts is not None else 0
        if inp.dtype not in K.DT or not self._use_zbal("gather", inp) or (inp.numel() * inp.element_size()) % 2:
            return self._fallback(input_tensors).gather(output_tensors, input_tensors, opts)
        comm, l = self._communicator(), K.lib()
        flat = torch.empty((self._size, inp.numel()), dtype=inp.dtype, device=inp.device)
        outs = output_tensors[0] if (self._rank == root and output_tensors) else []

        def go(s):
            K.check(l.zbal_gather(inp.data_ptr(), flat.data_ptr(), inp.numel(), K.DT[inp.dtype], root, comm, s), "zbal_gather")
            with torch.cuda.stream(torch.cuda.ExternalStream(s)):
                for r, o in enumerate(outs):
                    o.copy_(flat[r].view_as(o))
        return self._run([inp, flat] + list(outs), go, output_tensors)

    def broadcast(self, tensors, opts=None):
        t = tensors[0]
        root = opts.rootRank if opts is not None else 0
        if len(tensors) != 1 or t.dtype not in K.DT or not self._use_zbal("broadcast", t) or (t.numel() * t.element_size()) % 2:
            return self._fallback(tensors).broadcast(tensors, opts) if opts is not None else self._fallback(tensors).broadcast(tensors)
        comm, l = self._communicator(), K.lib()

        def go(s):
            K.check(l.zbal_broadcast(t.data_ptr(), t.numel(), K.DT[t.dtype], root, comm, s), "zbal_broadcast")
        return self._run([t], go, tensors)

    def scatter(self, output_tensors, input_tensors, opts=None):
        out = output_tensors[0]
        root = opts.rootRank if opts is not None else 0
        if out.dtype not in K.DT or not self._use_zbal("scatter", out) or (out.numel() * out.element_size()) % 2:
            return self._fallback(output_tensors).scatter(output_tensors, input_tensors, opts)
        comm, l = self._communicator(), K.lib()
        src = None
        if self._rank == root:
            src = torch.stack([p.reshape(-1) for p in input_tensors[0]]).contiguous()

        def go(s):
            K.check(l.zbal_scatter(src.data_ptr() if src is not None else None, out.data_ptr(), out.numel(), K.DT[out.dtype], root, comm, s),
                    "zbal_scatter")
        return self._run([out] + ([src] if src is not None else []), go, output_tensors)

    def _reduce_scatter_base(self, output, input, opts=None):
        op = _OPS.get(opts.reduceOp if opts is not None else ReduceOp.SUM)
        if op is None or input.dtype not in K.REDUCIBLE or not self._use_zbal("_reduce_scatter_base", output, input) or \
                input.numel() != output.numel() * self._size:
            return self._fallback(input)._reduce_scatter_base(output, input, opts) if opts is not None else \
                self._fallback(input)._reduce_scatter_base(output, input)
        comm, l = self._communicator(), K.lib()

        def go(s):
            K.check(l.zbal_reduce_scatter(input.data_ptr(), output.data_ptr(), output.numel(), K.DT[input.dtype], op, comm, s),
                    "zbal_reduce_scatter")
        return self._run([input, output], go, output)

    def reduce_scatter(self, output_tensors, input_tensors, opts=None):
        out, parts = output_tensors[0], input_tensors[0]
        op = _OPS.get(opts.reduceOp if opts is not None else ReduceOp.SUM)
        if op is None or out.dtype not in K.REDUCIBLE or not self._use_zbal("reduce_scatter", out) or any(p.numel() != out.numel() for p in parts):
            return self._fallback(output_tensors).reduce_scatter(output_tensors, input_tensors, opts)
        comm, l = self._communicator(), K.lib()
        flat = torch.stack([p.reshape(-1) for p in parts]).contiguous()

        def go(s):
            K.check(l.zbal_reduce_scatter(flat.data_ptr(), out.data_ptr(), out.numel(), K.DT[out.dtype], op, comm, s), "zbal_reduce_scatter")
        return self._run([flat, out], go, output_tensors)

    def reduce_scatter_tensor_coalesced(self, outputs, inputs, opts=None):
        return self._fallback(inputs).reduce_scatter_tensor_coalesced(outputs, inputs, opts)

    def reduce(self, tensors, opts=None):
        return self._fallback(tensors).reduce(tensors, opts)

    def alltoall(self, output_tensors, input_tensors, opts=None):
        return self._fallback(input_tensors).alltoall(output_tensors, input_tensors, opts)

    def barrier(self, opts=None):
        if "barrier" in self._forced or not self._strided:
            return self._fallback().barrier(opts) if opts is not None else self._fallback().barrier()
        comm, l = self._communicator(), K.lib()

        def go(s):
            K.check(l.zbal_barrier(comm, s), "zbal_barrier")
        work = self._run([], go, None)
        work._event.synchronize()  # a barrier returns when every rank has arrived
        return work

    def alltoall_base(self, output, input, output_split_sizes, input_split_sizes, opts=None):
        es = input.element_size()
        if not self._use_zbal("alltoall_base", output, input) or input.dtype not in K.DT:
            return self._fallback(input).alltoall_base(output, input, output_split_sizes, input_split_sizes, opts)
        row_in = input[0].numel() if input.dim() > 1 else 1
        row_out = output[0].numel() if output.dim() > 1 else 1
        ins = list(input_split_sizes) if input_split_sizes else [input.shape[0] // self._size] * self._size
        outs = list(output_split_sizes) if output_split_sizes else [output.shape[0] // self._size] * self._size
        nbytes = max(input.numel(), output.numel()) * es   # the pieces land in the receiver's staging area
        stage = self._stage_bytes()
        if nbytes + 4096 > stage or nbytes % 2:
            return self._fallback(input).alltoall_base(output, input, output_split_sizes, input_split_sizes, opts)
        meta = torch.empty((self._size, 4), dtype=torch.int64).pin_memory()
        so = ro = 0
        for p in range(self._size):
            meta[p, 0], meta[p, 1] = so * row_in * es, ins[p] * row_in * es
            meta[p, 2], meta[p, 3] = ro * row_out * es, outs[p] * row_out * es
            so += ins[p]
            ro += outs[p]
        comm, l = self._communicator(), K.lib()
        dev_meta = torch.empty((self._size, 4), dtype=torch.int64, device=input.device)

        def go(s):
            with torch.cuda.stream(torch.cuda.ExternalStream(s)):
                dev_meta.copy_(meta, non_blocking=True)
            K.check(l.zbal_all_to_all_v(input.data_ptr(), output.data_ptr(), dev_meta.data_ptr(), nbytes, comm, s), "zbal_all_to_all_v")
        return self._run([input, output, dev_meta], go, output)

    def _stage_bytes(self) -> int:
        p = K.CommPropertyC()
        K.check(K.lib().zbal_comm_get_property(self._communicator(), C.byref(p)), "zbal_comm_get_property")
        return int(p.stageBytes)

    # ------------------------------------------------------------------ point to point
    def send(self, tensors, dst_rank, tag=0):
        t = tensors[0]
        if not self._use_zbal("send", t) or t.dtype not in K.DT:
            return self._fallback(tensors).send(tensors, dst_rank, tag)
        comm, _, peer = self._p2p_comm(dst_rank)
        l = K.lib()

        def go(s):
            K.check(l.zbal_send(t.data_ptr(), t.numel(), K.DT[t.dtype], peer, comm, s), "zbal_send")
        return self._run([t], go, tensors)

    def recv(self, tensors, src_rank, tag=0):
        t = tensors[0]
        if not self._use_zbal("recv", t) or t.dtype not in K.DT:
            return self._fallback(tensors).recv(tensors, src_rank, tag)
        comm, _, peer = self._p2p_comm(src_rank)
        l = K.lib()

        def go(s):
            K.check(l.zbal_recv(t.data_ptr(), t.numel(), K.DT[t.dtype], peer, comm, s), "zbal_recv")
        return self._run([t], go, tensors)

    def recv_anysource(self, tensors, tag=0):
        return self._fallback(tensors).recv_anysource(tensors, tag)

    # ------------------------------------------------------------------ diagnostics
    def device_status(self):
        """(code, where, epoch, count) of this rank's device-side wait status; code 0 = no wait ever ran out."""
        st = (C.c_uint32 * 4)()
        K.check(K.lib().zbal_comm_get_device_status(self._communicator(), C.byref(st)), "zbal_comm_get_device_status")
        return tuple(int(v) for v in st)


def _build_native(path) -> None:
    """Builds the extension in-tree when it is missing (a fresh checkout); ranks that start together take turns."""
    import fcntl
    try:
        path.parent.mkdir(exist_ok=True)
        with open(path.parent / ".c10d.lock", "w") as lock:
            fcntl.flock(lock, fcntl.LOCK_EX)
            if not path.exists():
                from .. import _build
                _build.build_c10d()
    except Exception as e:  # noqa: BLE001 - no compiler or headers: the Python implementation serves
        import warnings
        warnings.warn(f"zbal: could not build the native c10d extension ({e}); using the Python process group")


def native_extension():
    """The C++ ``c10d::Backend`` module (csrc/c10d/zbal_process_group.cpp), or None when it was not built."""
    global _native_ext
    if _native_ext is None:
        import importlib.util
        from .. import _native as N
        path = N._LIB_DIR / "_zbal_c10d.so"
        if not path.exists() and os.environ.get("ZBAL_PG_IMPL", "native").lower() != "python":
            _build_native(path)
        if not path.exists():
            _native_ext = False
        else:
            K.lib()  # libmf_smem.so first, so that both sides share one copy of the library's state
            spec = importlib.util.spec_from_file_location("_zbal_c10d", str(path))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            _native_ext = mod
    return _native_ext or None


def implementation() -> str:
    """"native" (C++ c10d::Backend, the default when built) or "python" (``ZBAL_PG_IMPL=python``, or no extension)."""
    want = os.environ.get("ZBAL_PG_IMPL", "native").lower()
    if want == "python":
        return "python"
    if native_extension() is None:
        if want == "native" and "ZBAL_PG_IMPL" in os.environ:
            raise RuntimeError("ZBAL_PG_IMPL=native but lib/_zbal_c10d.so is not built (python -m memfabric_hybrid_b200._build --c10d)")
        return "python"
    return "native"


def _create_native(o):
    ext = native_extension()
    store, rank, size, timeout = o.store, o.group_rank, o.group_size, o.timeout
    pg = ext.ProcessGroupZBAL(store, rank, size, [int(r) for r in (o.global_ranks_in_group or [])], timeout)

    def fallback(cuda: bool):
        if cuda:
            return dist.ProcessGroupNCCL(dist.PrefixStore("zbal_nccl_fallback/", store), rank, size, dist.ProcessGroupNCCL.Options())
        return dist.ProcessGroupGloo(dist.PrefixStore("zbal_gloo_fallback/", store), rank, size, timeout=timeout)
    pg.set_fallback_factory(fallback)
    return pg


def _create(dist_backend_opts, pg_options):
    if implementation() == "native":
        return _create_native(dist_backend_opts)
    return ProcessGroupZBAL(dist_backend_opts.store, dist_backend_opts.group_rank, dist_backend_opts.group_size,
                            dist_backend_opts.global_ranks_in_group, dist_backend_opts.timeout)


def register() -> None:
    if "ZBAL" not in getattr(dist.Backend, "_plugins", {}):
        dist.Backend.register_backend("zbal", _create, extended_api=True, devices=["cuda", "cpu"])
