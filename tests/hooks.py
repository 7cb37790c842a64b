"""ctypes declarations of the mf_t_* entry points (csrc/smem/mf_testhooks.cpp) used by the control-plane tests."""
import ctypes as C

from memfabric_hybrid_b200 import _native as N

WATCH_CB = C.CFUNCTYPE(None, C.c_int, C.c_char_p, C.POINTER(C.c_char), C.c_int)
RANK_CB = C.CFUNCTYPE(None, C.c_uint32)
CHANGE_CB = C.CFUNCTYPE(C.c_int, C.c_int, C.c_uint32)

ERR_TIMEOUT, ERR_NOT_EXIST, ERR_IN_USE, ERR_NOT_CONNECTED = -2004, -2007, -2009, -2014

_done = False


def lib():
    global _done
    l = N.lib()
    if _done:
        return l
    vp, cp, i32, u32, u64, i64, u16 = C.c_void_p, C.c_char_p, C.c_int, C.c_uint32, C.c_uint64, C.c_int64, C.c_uint16
    P = C.POINTER
    s = N._sig
    s(l, "mf_t_server_start", vp, cp, u16, u32, u64, P(i32))
    s(l, "mf_t_server_stop", None, vp)
    s(l, "mf_t_server_keys", u64, vp)
    s(l, "mf_t_server_state", i32, vp)
    s(l, "mf_t_server_port", u16, vp)
    s(l, "mf_t_server_set_backend", None, vp, cp, i32)
    s(l, "mf_t_client_new", vp, cp, u16, u32, u32, u32, P(i32))
    s(l, "mf_t_store_prefixed", vp, vp, cp)
    s(l, "mf_t_store_free", None, vp)
    s(l, "mf_t_client_crash", None, vp)
    s(l, "mf_t_client_set_reconnect", None, vp, u32, u32)
    s(l, "mf_t_store_connected", i32, vp)
    s(l, "mf_t_store_rank", u32, vp)
    s(l, "mf_t_store_set", i32, vp, cp, cp, i32)
    s(l, "mf_t_store_get", i32, vp, cp, cp, i32, i64)
    s(l, "mf_t_store_add", i32, vp, cp, i64, P(i64))
    s(l, "mf_t_store_remove", i32, vp, cp, i32)
    s(l, "mf_t_store_append", i32, vp, cp, cp, i32, P(u64))
    s(l, "mf_t_store_cas", i32, vp, cp, cp, i32, cp, i32, cp, i32, P(i32))
    s(l, "mf_t_store_write", i32, vp, cp, u32, cp, i32)
    s(l, "mf_t_store_prefix_get", i32, vp, cp, cp, i32)
    s(l, "mf_t_store_watch", i32, vp, cp, WATCH_CB, P(u32))
    s(l, "mf_t_store_unwatch", i32, vp, u32)
    s(l, "mf_t_store_watch_rank", i32, vp, RANK_CB, P(u32))
    s(l, "mf_t_store_query_alive", i32, vp, u32, P(i32))
    s(l, "mf_t_store_auto_rank", i32, vp, P(u32))
    s(l, "mf_t_ha_new", vp, cp, u16, u32, u32, cp, i32)
    s(l, "mf_t_ha_set_timings", None, vp, u32, u32, u32, u32)
    s(l, "mf_t_ha_start", i32, vp, u32)
    s(l, "mf_t_ha_is_leader", i32, vp)
    s(l, "mf_t_ha_leader_addr", i32, vp, cp, i32)
    s(l, "mf_t_ha_kill_leader", None, vp)
    s(l, "mf_t_ha_new_etcd", vp, cp, u16, u32, u32, cp, u16, cp, i32)
    s(l, "mf_t_etcd_new", vp, cp, u16, cp, cp, cp, u32)
    s(l, "mf_t_etcd_free", None, vp)
    s(l, "mf_t_etcd_connect", i32, vp)
    s(l, "mf_t_etcd_put", i32, vp, cp, cp, i32, u32)
    s(l, "mf_t_etcd_get", i32, vp, cp, cp, i32)
    s(l, "mf_t_etcd_prefix_get", i32, vp, cp, cp, i32)
    s(l, "mf_t_etcd_delete", i32, vp, cp)
    s(l, "mf_t_etcd_clear", i32, vp, cp)
    s(l, "mf_t_etcd_exist", i32, vp, cp)
    s(l, "mf_t_etcd_lock", i32, vp, cp)
    s(l, "mf_t_etcd_try_lock", i32, vp, cp)
    s(l, "mf_t_etcd_unlock", i32, vp, cp)
    s(l, "mf_t_etcd_last_error", i32, vp, cp, i32)
    s(l, "mf_t_ex_new", vp, u16, u32, u32, u64, u64)
    s(l, "mf_t_ex_free", None, vp)
    s(l, "mf_t_ex_record_size", u32)
    s(l, "mf_t_ex_export", i32, vp, cp)
    s(l, "mf_t_ex_import", i32, vp, cp, u32, i32)
    s(l, "mf_t_ex_mapped_bytes", u64, vp, u32)
    s(l, "mf_t_backend_set_reachable", None, cp, i32)
    s(l, "mf_t_backend_reset", None, cp)
    s(l, "mf_t_group_new", vp, vp, u32, u32, u64, i32, CHANGE_CB)
    s(l, "mf_t_group_free", None, vp)
    s(l, "mf_t_group_barrier", i32, vp)
    s(l, "mf_t_group_allgather", i32, vp, cp, u32, cp, u32)
    s(l, "mf_t_group_sub_barrier", i32, vp, cp, u32, u32)
    s(l, "mf_t_group_sub_allgather", i32, vp, cp, u32, u32, cp, u32, cp, u32)
    s(l, "mf_t_group_start_listen", i32, vp)
    s(l, "mf_t_group_join", i32, vp)
    s(l, "mf_t_group_update", i32, vp)
    s(l, "mf_t_group_leave", i32, vp)
    s(l, "mf_t_group_joined", i32, vp)
    s(l, "mf_t_group_size", u32, vp)
    s(l, "mf_t_group_info", None, vp, P(u32), P(u32), P(u32), P(u64))
    s(l, "mf_t_group_alloc_number", i32, vp, u32, P(i32))
    s(l, "mf_t_group_release_number", i32, vp, i32)
    s(l, "mf_t_trace_start", i32, cp, u32)
    s(l, "mf_t_trace_stop", None)
    s(l, "mf_t_trace_hit", None, u32, i32, u32)
    s(l, "mf_t_trace_dump", i32, cp, i32, i32)
    s(l, "mf_t_trace_file", i32, cp, i32)
    s(l, "mf_t_trace_row", None, u32, P(u64 * 6))
    s(l, "mf_t_trace_name", cp, u32)
    s(l, "mf_t_trace_count", u32)
    s(l, "mf_t_fip_init", None, cp)
    s(l, "mf_t_fip_exit", None)
    s(l, "mf_t_fip_activate", i32, cp, i32, i32, i64)
    s(l, "mf_t_fip_deactivate", i32, cp)
    s(l, "mf_t_fip_is_active", i32, cp)
    s(l, "mf_t_fip_reload", None)
    s(l, "mf_t_fip_run", i32, cp, P(i32))
    _done = True
    return l


class Store:
    """Thin object view of a store handle."""

    def __init__(self, h):
        assert h, "store handle is NULL"
        self.h = h
        self._cbs = []

    @classmethod
    def connect(cls, port, world=4, rank=0, timeout_ms=5000, ip=b"127.0.0.1"):
        rc = C.c_int()
        h = lib().mf_t_client_new(ip, port, world, rank, timeout_ms, C.byref(rc))
        if not h:
            raise ConnectionError(f"client start-up failed: {rc.value}")
        return cls(h)

    def prefixed(self, prefix: str) -> "Store":
        return Store(lib().mf_t_store_prefixed(self.h, prefix.encode()))

    def close(self):
        if self.h:
            lib().mf_t_store_free(self.h)
            self.h = None

    def set(self, k, v: bytes):
        return lib().mf_t_store_set(self.h, k.encode(), v, len(v))

    def get(self, k, timeout_ms=0, cap=1 << 16):
        buf = C.create_string_buffer(cap)
        n = lib().mf_t_store_get(self.h, k.encode(), buf, cap, timeout_ms)
        return n if n < 0 else buf.raw[:n]

    def add(self, k, inc):
        r = C.c_int64()
        rc = lib().mf_t_store_add(self.h, k.encode(), inc, C.byref(r))
        assert rc == 0, rc
        return r.value

    def remove(self, k, quiet=False):
        return lib().mf_t_store_remove(self.h, k.encode(), 1 if quiet else 0)

    def append(self, k, v: bytes):
        n = C.c_uint64()
        rc = lib().mf_t_store_append(self.h, k.encode(), v, len(v), C.byref(n))
        assert rc == 0, rc
        return n.value

    def cas(self, k, expect: bytes, desired: bytes):
        buf = C.create_string_buffer(4096)
        n = C.c_int()
        rc = lib().mf_t_store_cas(self.h, k.encode(), expect, len(expect), desired, len(desired), buf, 4096, C.byref(n))
        return rc, buf.raw[:n.value]

    def write(self, k, off, v: bytes):
        return lib().mf_t_store_write(self.h, k.encode(), off, v, len(v))

    def keys(self, prefix):
        buf = C.create_string_buffer(1 << 16)
        n = lib().mf_t_store_prefix_get(self.h, prefix.encode(), buf, 1 << 16)
        assert n >= 0, n
        return [k for k in buf.value.decode().split("\n") if k]

    def watch(self, k, fn):
        cb = WATCH_CB(lambda rc, key, val, n: fn(rc, key.decode(), C.string_at(val, n) if n > 0 else b""))
        self._cbs.append(cb)
        wid = C.c_uint32()
        rc = lib().mf_t_store_watch(self.h, k.encode(), cb, C.byref(wid))
        assert rc == 0, rc
        return wid.value

    def unwatch(self, wid):
        return lib().mf_t_store_unwatch(self.h, wid)

    def watch_rank(self, fn):
        cb = RANK_CB(lambda r: fn(r))
        self._cbs.append(cb)
        wid = C.c_uint32()
        rc = lib().mf_t_store_watch_rank(self.h, cb, C.byref(wid))
        assert rc == 0, rc
        return wid.value

    def alive(self, rank):
        a = C.c_int()
        rc = lib().mf_t_store_query_alive(self.h, rank, C.byref(a))
        assert rc == 0, rc
        return bool(a.value)

    def auto_rank(self):
        r = C.c_uint32()
        rc = lib().mf_t_store_auto_rank(self.h, C.byref(r))
        return rc, r.value

    def connected(self):
        return bool(lib().mf_t_store_connected(self.h))


def start_server(port, world=4, flags=0):
    rc = C.c_int()
    h = lib().mf_t_server_start(b"127.0.0.1", port, world, flags, C.byref(rc))
    assert h, f"server start-up failed: {rc.value}"
    return h
