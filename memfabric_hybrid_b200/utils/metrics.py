"""Metrics in the Prometheus text format: the host trace-point table (calls, failures, latency per data-path and
control-plane operation), the copy-path counters of registered pools and the symmetric-heap allocator.

    from memfabric_hybrid_b200.utils import metrics
    metrics.register_pool("kv", bm_handle)         # optional: per-pool copy counters
    metrics.serve(9464)                            # GET http://127.0.0.1:9464/metrics
    print(metrics.render())                        # or scrape by hand

The reference ships this layer as a design only (examples/memory_pool/05_observability/*: the exporter and
dashboards are "not yet committed"); its built-in numbers are the ptracer table (doc/ptracer.md:19-39), which is
what the ``mf_trace_*`` families below export.
"""
from __future__ import annotations

import ctypes as C
import http.server
import threading
from typing import Dict, List, Tuple

from .. import _native as N

_pools: Dict[str, object] = {}
_server = None


def register_pool(name: str, handle) -> None:
    """``handle``: a ``bm.BigMemory``; its copy counters are exported with label pool="<name>"."""
    _pools[name] = handle


def unregister_pool(name: str) -> None:
    _pools.pop(name, None)


def _trace_rows() -> List[Tuple[str, Tuple[int, ...]]]:
    l = N.lib()
    l.mf_t_trace_count.restype = C.c_uint32
    l.mf_t_trace_name.restype, l.mf_t_trace_name.argtypes = C.c_char_p, [C.c_uint32]
    l.mf_t_trace_row.restype, l.mf_t_trace_row.argtypes = None, [C.c_uint32, C.POINTER(C.c_uint64 * 6)]
    rows = []
    for i in range(l.mf_t_trace_count()):
        out = (C.c_uint64 * 6)()
        l.mf_t_trace_row(i, C.byref(out))
        if out[0]:
            rows.append(((l.mf_t_trace_name(i) or b"?").decode(), tuple(int(v) for v in out)))
    return rows


def _trace_histograms() -> List[Tuple[Dict[str, str], float]]:
    """Samples of the histogram family mf_trace_duration_seconds (cumulative ``le`` buckets, ``_sum``, ``_count``) for every
    point that has completed an operation. The buckets double from 1 us; they cover the whole run (the periodic table,
    which resets its own columns, leaves them alone)."""
    l = N.lib()
    l.mf_t_trace_count.restype = C.c_uint32
    l.mf_t_trace_name.restype, l.mf_t_trace_name.argtypes = C.c_char_p, [C.c_uint32]
    l.mf_t_trace_hist.restype, l.mf_t_trace_hist.argtypes = C.c_uint32, [C.c_uint32, C.POINTER(C.c_uint64)]
    nb = l.mf_t_trace_hist(0, None)
    out = []
    for pid in range(l.mf_t_trace_count()):
        buf = (C.c_uint64 * (nb + 2))()
        l.mf_t_trace_hist(pid, buf)
        if not any(buf[i] for i in range(nb + 1)):
            continue
        p = (l.mf_t_trace_name(pid) or b"?").decode()
        acc = 0
        for i in range(nb):
            acc += buf[i]
            out.append(({"point": p, "le": f"{1e-6 * (1 << i):.9g}", "__suffix__": "_bucket"}, float(acc)))
        acc += buf[nb]
        out.append(({"point": p, "le": "+Inf", "__suffix__": "_bucket"}, float(acc)))
        out.append(({"point": p, "__suffix__": "_sum"}, buf[nb + 1] * 1e-9))
        out.append(({"point": p, "__suffix__": "_count"}, float(acc)))
    return out


def collect() -> List[Tuple[str, str, str, List[Tuple[Dict[str, str], float]]]]:
    """[(family, type, help, [(labels, value)])]."""
    fams = []
    rows = _trace_rows()
    if rows:
        def fam(name, typ, hlp, idx, scale=1.0):
            fams.append((name, typ, hlp, [({"point": p}, r[idx] * scale) for p, r in rows]))
        fam("mf_trace_calls_total", "counter", "operations started at a trace point", 0)
        fam("mf_trace_ok_total", "counter", "operations that returned success", 1)
        fam("mf_trace_failed_total", "counter", "operations that returned an error", 2)
        fams.append(("mf_trace_in_flight", "gauge", "operations started and not yet finished",
                     [({"point": p}, float(max(0, r[0] - r[1] - r[2]))) for p, r in rows]))
        fam("mf_trace_seconds_total", "counter", "time spent inside the trace point", 5, 1e-9)
        fams.append(("mf_trace_min_seconds", "gauge", "fastest completed operation",
                     [({"point": p}, r[3] * 1e-9) for p, r in rows if r[1] + r[2]]))
        fam("mf_trace_max_seconds", "gauge", "slowest completed operation", 4, 1e-9)
    hist = _trace_histograms()
    if hist:
        fams.append(("mf_trace_duration_seconds", "histogram", "duration of completed operations (buckets double from 1 us)", hist))
    if _pools:
        per_key: Dict[str, List[Tuple[Dict[str, str], float]]] = {}
        for name, h in list(_pools.items()):
            try:
                st = h.copy_stats()
            except Exception:  # noqa: BLE001 - a destroyed pool must not break the scrape
                continue
            for k, v in st.items():
                per_key.setdefault(k, []).append(({"pool": name}, float(v)))
        for k, vals in per_key.items():
            fams.append((f"mf_pool_{k}_total", "counter", f"copy path counter {k}", vals))
        cap = []
        for name, h in list(_pools.items()):
            try:
                from ..api import bm
                for mem, label in ((bm.BmMemType.DEVICE, "device"), (bm.BmMemType.HOST, "host")):
                    n = int(h.local_mem_size(mem))
                    if n > 0:
                        cap.append(({"pool": name, "mem": label}, float(n)))
            except Exception:  # noqa: BLE001
                continue
        if cap:
            fams.append(("mf_pool_local_bytes", "gauge", "bytes this rank contributes to the pool", cap))
    try:
        from ..zbal import _capi as K
        s = K.SmaStatsC()
        if K.lib().zbal_sma_get_stats(C.byref(s)) == 0:
            gauges = {"heapSize": "bytes of the symmetric heap", "inUseBytes": "bytes handed out", "cachedBytes": "bytes cached per stream",
                      "peakInUseBytes": "peak of bytes handed out", "largestFreeBlock": "largest free block of the heap",
                      "poolCount": "private (CUDA graph) pools", "poolCachedBytes": "bytes parked in private pools"}
            for f, hlp in gauges.items():
                fams.append((f"zbal_heap_{_snake(f)}", "gauge", hlp, [({}, float(getattr(s, f)))]))
            for f in ("mallocCalls", "freeCalls", "cacheHits", "heapCarves", "failedMallocs"):
                fams.append((f"zbal_heap_{_snake(f)}_total", "counter", f"allocator counter {f}", [({}, float(getattr(s, f)))]))
    except Exception:  # noqa: BLE001 - allocator not initialised
        pass
    return fams


def _snake(name: str) -> str:
    return "".join("_" + c.lower() if c.isupper() else c for c in name)


def _esc(v: str) -> str:
    return v.replace("\\", "\\\\").replace('"', '\\"').replace("\n", "\\n")


def render() -> str:
    lines = []
    for name, typ, hlp, samples in collect():
        lines.append(f"# HELP {name} {hlp}")
        lines.append(f"# TYPE {name} {typ}")
        for labels, value in samples:
            labels = dict(labels)
            suffix = labels.pop("__suffix__", "")          # histogram samples: _bucket / _sum / _count
            lab = "{" + ",".join(f'{k}="{_esc(str(v))}"' for k, v in sorted(labels.items())) + "}" if labels else ""
            lines.append(f"{name}{suffix}{lab} {value:.9g}")
    return "\n".join(lines) + "\n"


class _Handler(http.server.BaseHTTPRequestHandler):
    def do_GET(self):  # noqa: N802
        if self.path.split("?")[0] not in ("/metrics", "/"):
            self.send_error(404)
            return
        body = render().encode()
        self.send_response(200)
        self.send_header("Content-Type", "text/plain; version=0.0.4; charset=utf-8")
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def log_message(self, *a):  # scrapes are not worth a log line each
        pass


def serve(port: int, addr: str = "127.0.0.1") -> int:
    """Starts the exporter on a daemon thread; returns the bound port (pass 0 to let the system choose)."""
    global _server
    if _server is not None:
        return _server.server_address[1]
    _server = http.server.ThreadingHTTPServer((addr, port), _Handler)
    threading.Thread(target=_server.serve_forever, name="mf-metrics", daemon=True).start()
    return _server.server_address[1]


def stop() -> None:
    global _server
    if _server is not None:
        _server.shutdown()
        _server.server_close()
        _server = None
