"""Stand-alone config store server: ``python -m memfabric_hybrid_b200.launch_store --url tcp://0.0.0.0:8570``.

Runs until interrupted. Jobs then pass the same URL with ``start_store = False``. ``MF_LOG_LEVEL`` (0-4) sets
the log level. Counterpart of the reference's launcher script (src/smem/python/memfabric_hybrid/launch_ascend_mf_store.py)."""
from __future__ import annotations

import argparse
import os
import signal
import threading


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="MemFabric config store server")
    ap.add_argument("--url", default=os.environ.get("MF_CONFIG_STORE_URL", "tcp://0.0.0.0:8570"))
    ap.add_argument("--flags", type=int, default=0)
    a = ap.parse_args(argv)
    from . import api as mf
    mf.initialize()
    lv = os.environ.get("MF_LOG_LEVEL", "")
    if len(lv) == 1 and lv.isdigit():
        mf.set_log_level(int(lv))
    rc = mf.create_config_store(a.url, a.flags)
    if rc != 0:
        print(f"cannot start the config store at {a.url}: {rc} {mf.get_last_err_msg()}")
        return 1
    print(f"config store serving at {a.url}; Ctrl-C to stop", flush=True)
    stop = threading.Event()
    for s in (signal.SIGINT, signal.SIGTERM):
        signal.signal(s, lambda *_: stop.set())
    stop.wait()
    mf.destroy_config_store(a.url)
    mf.uninitialize()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
