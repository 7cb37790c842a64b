"""``memfabric_hybrid.TransferEngine``: the point-to-point transfer adapter used by serving stacks.

Two deployment shapes, both supported by the reference's adapter:

* per-receiver stores (default): every process whose role equals ``store_server_role`` hosts a
  config store at the ``ip:port`` prefix of its own session id; a sender opens one connection per
  destination (cached by prefix) and replays its registered buffers on it;
* one shared store: pass ``store_server_role=None`` and every process uses ``store_url``.

Parity: src/smem/csrc/python_wrapper/mk_transfer_adapter/csrc/pytransfer.cpp:52-781.
"""
from __future__ import annotations

import ctypes as C
import enum
import os
import socket
import threading
from typing import Sequence

from .. import _native as N


@N.register_decls
def _decls(l):
    P = C.POINTER
    N._sig(l, "smem_trans_config_init", N.i32, P(N.TransConfigC))
    N._sig(l, "smem_trans_init", N.i32, P(N.TransConfigC))
    N._sig(l, "smem_trans_uninit", None, N.u32)
    N._sig(l, "smem_trans_create", N.vp, N.cp, N.cp, P(N.TransConfigC))
    N._sig(l, "smem_trans_destroy", None, N.vp, N.u32)
    N._sig(l, "smem_trans_register_mem", N.i32, N.vp, N.vp, C.c_size_t, N.u32)
    N._sig(l, "smem_trans_batch_register_mem", N.i32, N.vp, P(N.vp), P(C.c_size_t), N.u32, N.u32)
    N._sig(l, "smem_trans_deregister_mem", N.i32, N.vp, N.vp)
    N._sig(l, "smem_trans_write", N.i32, N.vp, N.vp, N.cp, N.vp, C.c_size_t, N.u32)
    N._sig(l, "smem_trans_read", N.i32, N.vp, N.vp, N.cp, N.vp, C.c_size_t, N.u32)
    N._sig(l, "smem_trans_batch_write", N.i32, N.vp, P(N.vp), N.cp, P(N.vp), P(C.c_size_t), N.u32, N.u32)
    N._sig(l, "smem_trans_batch_read", N.i32, N.vp, P(N.vp), N.cp, P(N.vp), P(C.c_size_t), N.u32, N.u32)
    N._sig(l, "smem_trans_write_submit", N.i32, N.vp, N.vp, N.cp, N.vp, C.c_size_t, N.vp, N.u32)
    N._sig(l, "smem_trans_read_submit", N.i32, N.vp, N.vp, N.cp, N.vp, C.c_size_t, N.vp, N.u32)
    N._sig(l, "smem_trans_batch_write_submit", N.i32, N.vp, P(N.vp), N.cp, P(N.vp), P(C.c_size_t), N.u32, N.vp, N.u32)
    N._sig(l, "smem_trans_batch_read_submit", N.i32, N.vp, P(N.vp), N.cp, P(N.vp), P(C.c_size_t), N.u32, N.vp, N.u32)
    N._sig(l, "smem_trans_batch_quant_write", N.i32, N.vp, P(N.TransQuantParamC))
    N._sig(l, "smem_trans_set_peer_down_callback", N.i32, N.vp, N.PEER_DOWN_FN, N.vp)


class TransDataOpType(enum.IntEnum):
    SDMA = 1 << 0
    DEVICE_RDMA = 1 << 3


class TransferOpcode(enum.IntEnum):
    Read = 0
    Write = 1


def _prefix(session_id: str) -> str:
    return session_id.split("_", 1)[0]


def _arr(values: Sequence[int], ctype):
    return (ctype * len(values))(*[int(v) for v in values])


class TransferEngine:
    def __init__(self) -> None:
        self._cfg = N.TransConfigC()
        self._session = ""
        self._proto = "tcp://"
        self._shared_url = None
        self._own = None             # handle on our own store (store-server role / shared store)
        self._conns = {}             # peer prefix -> handle
        self._regs = {}              # addr -> capacity (replayed on new connections)
        self._allocs = {}            # trans_malloc allocations
        self._lock = threading.Lock()
        self._down_cb = None
        self._port_sock = None
        self._inited = False

    # ---------------------------------------------------------------- lifecycle
    def initialize(self, store_url: str, session_id: str, role: str, device_id: int,
                   data_op_type: TransDataOpType = TransDataOpType.SDMA, store_server_role: str | None = "Decode") -> int:
        if role not in ("Prefill", "Decode"):
            return -1
        l = N.lib()
        l.smem_init(0)
        lv = os.environ.get("MF_LOG_LEVEL", "")
        if len(lv) == 1 and lv.isdigit():
            l.smem_set_log_level(int(lv))
        l.smem_trans_config_init(C.byref(self._cfg))
        self._cfg.role = 1 if role == "Prefill" else 2
        self._cfg.deviceId = device_id
        self._cfg.dataOpType = int(data_op_type)
        self._session = session_id
        if "://" in store_url:
            self._proto = store_url.split("://", 1)[0] + "://"
        rc = l.smem_trans_init(C.byref(self._cfg))
        if rc != 0:
            return rc
        self._inited = True
        if store_server_role is None:
            self._shared_url = store_url
            self._own = l.smem_trans_create(store_url.encode(), session_id.encode(), C.byref(self._cfg))
            return 0 if self._own else -1
        if store_server_role == role:
            url = self._proto + _prefix(session_id)
            rc = l.smem_create_config_store(url.encode(), 1)
            if rc != 0:
                return rc
            self._own = l.smem_trans_create(url.encode(), session_id.encode(), C.byref(self._cfg))
            self._own_url = url
            return 0 if self._own else -1
        return 0

    def get_rpc_port(self) -> str:
        """A free TCP port, kept bound until destroy, joined with the pid: the tail of a session id."""
        if self._port_sock is None:
            s = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            s.bind(("0.0.0.0", 0))
            self._port_sock = s
        return f"{self._port_sock.getsockname()[1]}_{os.getpid()}"

    def _conn(self, dest_session: str):
        if self._shared_url is not None:
            return self._own
        pref = _prefix(dest_session)
        with self._lock:
            h = self._conns.get(pref)
            if h:
                return h
            if self._own and pref == _prefix(self._session):
                return self._own
            url = self._proto + pref
            h = N.lib().smem_trans_create(url.encode(), self._session.encode(), C.byref(self._cfg))
            if not h:
                return None
            if self._down_cb is not None:
                N.lib().smem_trans_set_peer_down_callback(h, self._down_cb, None)
            for addr, cap in self._regs.items():  # replay registrations on the new connection
                N.lib().smem_trans_register_mem(h, addr, cap, 0)
            self._conns[pref] = h
            return h

    def _handles(self):
        hs = list(self._conns.values())
        if self._own:
            hs.append(self._own)
        return hs

    def set_peer_down_callback(self, fn) -> int:
        def tramp(uid, _ud):
            name = (uid or b"").decode()
            with self._lock:
                self._conns.pop(_prefix(name), None)
            fn(name)
        self._down_cb = N.PEER_DOWN_FN(tramp)
        rc = 0
        for h in self._handles():
            rc = rc or N.lib().smem_trans_set_peer_down_callback(h, self._down_cb, None)
        return rc

    # ---------------------------------------------------------------- memory
    def register_memory(self, buffer_addr: int, capacity: int) -> int:
        with self._lock:
            self._regs[int(buffer_addr)] = int(capacity)
        rc = 0
        for h in self._handles():
            rc = rc or N.lib().smem_trans_register_mem(h, buffer_addr, capacity, 0)
        return rc

    def batch_register_memory(self, buffer_addrs: Sequence[int], capacities: Sequence[int]) -> int:
        with self._lock:
            for a, c in zip(buffer_addrs, capacities):
                self._regs[int(a)] = int(c)
        rc = 0
        for h in self._handles():
            rc = rc or N.lib().smem_trans_batch_register_mem(h, _arr(buffer_addrs, C.c_void_p),
                                                            _arr(capacities, C.c_size_t), len(buffer_addrs), 0)
        return rc

    def unregister_memory(self, buffer_addr: int) -> int:
        with self._lock:
            self._regs.pop(int(buffer_addr), None)
        rc = 0
        for h in self._handles():
            rc = rc or N.lib().smem_trans_deregister_mem(h, buffer_addr)
        return rc

    def trans_malloc(self, capacity: int) -> int:
        """Device memory when a GPU is attached (a torch uint8 tensor keeps it alive), else host memory."""
        try:
            import torch
            if torch.cuda.is_available():
                t = torch.empty(capacity, dtype=torch.uint8, device=f"cuda:{self._cfg.deviceId}")
                self._allocs[t.data_ptr()] = t
                return t.data_ptr()
        except Exception:
            pass
        buf = C.create_string_buffer(capacity)
        addr = C.addressof(buf)
        self._allocs[addr] = buf
        return addr

    def trans_free(self, buffer_addr: int) -> int:
        return 0 if self._allocs.pop(int(buffer_addr), None) is not None else -1

    # ---------------------------------------------------------------- data
    def transfer_sync_write(self, dest_session: str, buffer: int, peer_buffer: int, length: int, flags: int = 0) -> int:
        h = self._conn(dest_session)
        return -1 if not h else N.lib().smem_trans_write(h, buffer, dest_session.encode(), peer_buffer, length, flags)

    def transfer_sync_read(self, dest_session: str, buffer: int, peer_buffer: int, length: int, flags: int = 0) -> int:
        h = self._conn(dest_session)
        return -1 if not h else N.lib().smem_trans_read(h, buffer, dest_session.encode(), peer_buffer, length, flags)

    def batch_transfer_sync_write(self, dest_session: str, buffers, peer_buffers, lengths, flags: int = 0) -> int:
        h = self._conn(dest_session)
        if not h:
            return -1
        return N.lib().smem_trans_batch_write(h, _arr(buffers, C.c_void_p), dest_session.encode(), _arr(peer_buffers, C.c_void_p),
                                              _arr(lengths, C.c_size_t), len(buffers), flags)

    def batch_transfer_sync_read(self, dest_session: str, buffers, peer_buffers, lengths, flags: int = 0) -> int:
        h = self._conn(dest_session)
        if not h:
            return -1
        return N.lib().smem_trans_batch_read(h, _arr(buffers, C.c_void_p), dest_session.encode(), _arr(peer_buffers, C.c_void_p),
                                             _arr(lengths, C.c_size_t), len(buffers), flags)

    def transfer_async_write_submit(self, dest_session: str, buffer: int, peer_buffer: int, length: int, stream: int, flags: int = 0) -> int:
        h = self._conn(dest_session)
        return -1 if not h else N.lib().smem_trans_write_submit(h, buffer, dest_session.encode(), peer_buffer, length, stream or None, flags)

    def transfer_async_read_submit(self, dest_session: str, buffer: int, peer_buffer: int, length: int, stream: int, flags: int = 0) -> int:
        h = self._conn(dest_session)
        return -1 if not h else N.lib().smem_trans_read_submit(h, buffer, dest_session.encode(), peer_buffer, length, stream or None, flags)

    def batch_transfer_async_write_submit(self, dest_session: str, buffers, peer_buffers, lengths, stream: int, flags: int = 0) -> int:
        h = self._conn(dest_session)
        if not h:
            return -1
        return N.lib().smem_trans_batch_write_submit(h, _arr(buffers, C.c_void_p), dest_session.encode(), _arr(peer_buffers, C.c_void_p),
                                                     _arr(lengths, C.c_size_t), len(buffers), stream or None, flags)

    def batch_transfer_async_read_submit(self, dest_session: str, buffers, peer_buffers, lengths, stream: int, flags: int = 0) -> int:
        h = self._conn(dest_session)
        if not h:
            return -1
        return N.lib().smem_trans_batch_read_submit(h, _arr(buffers, C.c_void_p), dest_session.encode(), _arr(peer_buffers, C.c_void_p),
                                                    _arr(lengths, C.c_size_t), len(buffers), stream or None, flags)

    def batch_transfer_write_with_quant(self, dest_session: str, buffers, peer_buffers, lengths, scale_buffers, offset_buffers,
                                        unit_num: int, input_type: int = 0, stream: int = 0, flags: int = 0) -> int:
        h = self._conn(dest_session)
        if not h:
            return -1
        p = N.TransQuantParamC()
        uid = dest_session.encode()
        p.remoteUniqueId = uid
        p.localAddrs = _arr(buffers, C.c_void_p)
        p.remoteAddrs = _arr(peer_buffers, C.c_void_p)
        p.dataSizes = _arr(lengths, C.c_size_t)
        p.scale = _arr(scale_buffers, C.c_void_p)
        p.offset = _arr(offset_buffers or [0] * len(buffers), C.c_void_p)
        p.batchSize = len(buffers)
        p.unitNum = unit_num
        p.stream = stream or None
        p.inputType = input_type
        p.flags = flags
        return N.lib().smem_trans_batch_quant_write(h, C.byref(p))

    # ---------------------------------------------------------------- teardown
    def destroy(self) -> None:
        for h in self._handles():
            N.lib().smem_trans_destroy(h, 0)
        self._conns.clear()
        self._own = None
        if getattr(self, "_own_url", None):
            N.lib().smem_destroy_config_store(self._own_url.encode())
            self._own_url = None
        if self._port_sock is not None:
            self._port_sock.close()
            self._port_sock = None

    def unInitialize(self) -> None:
        self.destroy()
        if self._inited:
            N.lib().smem_trans_uninit(0)
            N.lib().smem_uninit()
            self._inited = False
