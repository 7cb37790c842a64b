"""The per-process trace table (counts, good/bad ends, min/max/total, periodic file) and the fault points
(activation by call and by config file, hit budgets, the built-in STORE_CONNECT point on a real connect)."""
import ctypes as C
import os
import time

import hooks as H
from conftest import free_port


def test_trace_table(tmp_path):
    l = H.lib()
    assert l.mf_t_trace_count() > 10 and l.mf_t_trace_name(0)
    assert l.mf_t_trace_start(str(tmp_path).encode(), 200) == 0
    try:
        for i in range(5):
            l.mf_t_trace_hit(3, 0 if i < 4 else -7, 1000)
        row = (C.c_uint64 * 6)()
        l.mf_t_trace_row(3, C.byref(row))
        begin, good, bad, mn, mx, total = list(row)
        assert (begin, good, bad) == (5, 4, 1) and 900_000 <= mn <= mx and total >= 5 * mn
        buf = C.create_string_buffer(1 << 16)
        l.mf_t_trace_dump(buf, 1 << 16, 0)
        txt = buf.value.decode()
        name = l.mf_t_trace_name(3).decode()
        assert name in txt
        time.sleep(0.6)                                  # at least one period: the table was appended to the file
        pbuf = C.create_string_buffer(512)
        l.mf_t_trace_file(pbuf, 512)
        path = pbuf.value.decode()
        assert path.startswith(str(tmp_path)) and os.path.getsize(path) > 0 and name in open(path).read()
    finally:
        l.mf_t_trace_stop()
    # stopped: hits are not recorded any more
    l.mf_t_trace_hit(3, 0, 0)


def test_fault_points_by_call_and_by_file(tmp_path):
    l = H.lib()
    conf = tmp_path / "fip.conf"
    l.mf_t_fip_init(str(conf).encode())
    try:
        ret = C.c_int32()
        assert l.mf_t_fip_run(b"MMAP", C.byref(ret)) == 1 and ret.value == 0            # inactive: the block runs
        assert l.mf_t_fip_activate(b"MMAP", 0, 2, -1234) == 0 and l.mf_t_fip_is_active(b"MMAP") == 1
        for _ in range(2):                                                               # two hits are budgeted
            assert l.mf_t_fip_run(b"MMAP", C.byref(ret)) == 0 and ret.value == -1234
        assert l.mf_t_fip_run(b"MMAP", C.byref(ret)) == 1 and l.mf_t_fip_is_active(b"MMAP") == 0
        # a pause point delays and then lets the block run
        l.mf_t_fip_activate(b"IMPORT", 1, 1, 150)
        t0 = time.time()
        assert l.mf_t_fip_run(b"IMPORT", C.byref(ret)) == 1 and time.time() - t0 >= 0.14
        # the config file is picked up while running (checked at most every 200 ms) and cleared when removed
        conf.write_text("# name type hits param\nALLOC_LOCAL_MEMORY callback -1 -55\n")
        time.sleep(0.25)
        l.mf_t_fip_reload()
        assert l.mf_t_fip_run(b"ALLOC_LOCAL_MEMORY", C.byref(ret)) == 0 and ret.value == -55
        conf.unlink()
        time.sleep(0.25)
        l.mf_t_fip_reload()
        assert l.mf_t_fip_run(b"ALLOC_LOCAL_MEMORY", C.byref(ret)) == 1
        # the built-in point in the store client: one refused connect, then the dial succeeds
        port = free_port()
        srv = H.start_server(port, world=2)
        l.mf_t_fip_activate(b"STORE_CONNECT", 0, 1, -1)
        c = H.Store.connect(port, world=2, rank=0, timeout_ms=5000)
        assert c.connected() and l.mf_t_fip_is_active(b"STORE_CONNECT") == 0
        c.close()
        l.mf_t_server_stop(srv)
    finally:
        l.mf_t_fip_exit()


def test_prometheus_exporter_serves_trace_table_and_allocator(tmp_path):
    import urllib.request
    from memfabric_hybrid_b200.utils import metrics
    from memfabric_hybrid_b200.zbal import _capi as K
    l = H.lib()
    assert l.mf_t_trace_start(str(tmp_path).encode(), 60_000) == 0
    try:
        def hist():
            out = {}
            for line in metrics.render().splitlines():
                if line.startswith("mf_trace_duration_seconds") and f'point="{l.mf_t_trace_name(3).decode()}"' in line:
                    key, val = line.rsplit(" ", 1)
                    out[key.replace(f'point="{l.mf_t_trace_name(3).decode()}"', "").replace("{,", "{").replace(",}", "}").replace("{}", "")] = float(val)
            return out
        l.mf_t_trace_hit(3, 0, 1)                            # the point exists in the table from here on
        before = hist()
        for ret in (0, 0, -1):
            l.mf_t_trace_hit(3, ret, 200)
        after = hist()
        d = {k: after[k] - before.get(k, 0) for k in after}
        # three operations of at least 200 us each: none in the buckets up to 128 us, all of them counted at the top
        assert d["mf_trace_duration_seconds_count"] == 3 and d['mf_trace_duration_seconds_bucket{le="+Inf"}'] == 3
        assert d['mf_trace_duration_seconds_bucket{le="0.000128"}'] == 0 and d["mf_trace_duration_seconds_sum"] >= 600e-6
        les = [float(k.split('le="')[1].rstrip('"}')) for k in after if "_bucket" in k and "+Inf" not in k]
        assert les == sorted(les) and les[0] == 1e-6 and len(les) == 24
        vals = [after[k] for k in after if "_bucket" in k]
        assert vals == sorted(vals)                           # cumulative
        l.mf_t_trace_dump(None, 0, 1)                         # the periodic table resets its own columns, not the histogram
        assert hist()["mf_trace_duration_seconds_count"] == after["mf_trace_duration_seconds_count"]
        for ret in (0, 0, -1):
            l.mf_t_trace_hit(3, ret, 200)
        K.lib().zbal_simulate_init(0x7000_0000_0000, 64 << 20)
        p = K.lib().zbal_pluggable_malloc(3 << 20, 0, None)
        text = metrics.render()
        name = l.mf_t_trace_name(3).decode()
        assert f'mf_trace_calls_total{{point="{name}"}} 3' in text
        assert f'mf_trace_failed_total{{point="{name}"}} 1' in text and f'mf_trace_in_flight{{point="{name}"}} 0' in text
        assert "# TYPE mf_trace_duration_seconds histogram" in text
        assert "# TYPE mf_trace_seconds_total counter" in text and "zbal_heap_in_use_bytes 4194304" in text
        port = metrics.serve(0)
        body = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=10).read().decode()
        assert "zbal_heap_heap_size 67108864" in body and body.endswith("\n")
        K.lib().zbal_pluggable_free(p, 0, 0, None)
    finally:
        metrics.stop()
        K.lib().zbal_sma_uninit(0)
        l.mf_t_trace_stop()
