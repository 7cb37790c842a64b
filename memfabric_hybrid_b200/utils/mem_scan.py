"""How much host memory can back a pooled-DRAM slice right now, per NUMA node: free and total bytes, huge pages (2 MiB and
1 GiB, configured and free), and how fragmented the free memory is (free blocks per buddy order: the largest contiguous
free run, and the bytes that sit in runs of at least 2 MiB, which a pool can take without waiting for compaction).

    python -m memfabric_hybrid_b200.utils.mem_scan [--min-mb 2] [--json]

Everything is read from /proc and /sys (``root`` redirects both: tests, or a captured tree of another machine); what a
container hides is reported as absent, not as zero.
Parity of role: script/mem_scan.py of the reference (free physical ranges per NUMA node before a pool is created)."""
from __future__ import annotations

import argparse
import json
import os
import re
from typing import Dict, List, Optional


def _read(path: str) -> Optional[str]:
    try:
        with open(path) as f:
            return f.read()
    except OSError:
        return None


def page_size() -> int:
    return os.sysconf("SC_PAGE_SIZE")


def nodes(root: str = "/") -> List[int]:
    base = os.path.join(root, "sys/devices/system/node")
    try:
        return sorted(int(d[4:]) for d in os.listdir(base) if d.startswith("node") and d[4:].isdigit())
    except OSError:
        return []


def node_meminfo(node: int, root: str = "/") -> Dict[str, int]:
    """{"MemTotal": bytes, "MemFree": bytes, ...} of one node ({} when hidden)."""
    text = _read(os.path.join(root, f"sys/devices/system/node/node{node}/meminfo")) or ""
    out = {}
    for m in re.finditer(r"Node\s+\d+\s+(\w+):\s+(\d+)(\s*kB)?", text):
        out[m.group(1)] = int(m.group(2)) * (1024 if m.group(3) else 1)
    return out


def node_hugepages(node: int, root: str = "/") -> Dict[str, Dict[str, int]]:
    """{"2048kB": {"total": n, "free": n}, "1048576kB": {...}}."""
    base = os.path.join(root, f"sys/devices/system/node/node{node}/hugepages")
    out = {}
    try:
        kinds = sorted(os.listdir(base))
    except OSError:
        return out
    for k in kinds:
        if not k.startswith("hugepages-"):
            continue
        total, free = _read(os.path.join(base, k, "nr_hugepages")), _read(os.path.join(base, k, "free_hugepages"))
        if total is not None and free is not None:
            out[k[len("hugepages-"):]] = {"total": int(total), "free": int(free)}
    return out


def buddy_orders(root: str = "/") -> Dict[int, List[int]]:
    """node -> free blocks per order, summed over the node's zones (order k: blocks of 2^k pages)."""
    out: Dict[int, List[int]] = {}
    for line in (_read(os.path.join(root, "proc/buddyinfo")) or "").splitlines():
        m = re.match(r"Node\s+(\d+),\s+zone\s+\S+\s+(.*)", line)
        if not m:
            continue
        counts = [int(x) for x in m.group(2).split()]
        cur = out.setdefault(int(m.group(1)), [0] * len(counts))
        if len(cur) < len(counts):
            cur.extend([0] * (len(counts) - len(cur)))
        for i, c in enumerate(counts):
            cur[i] += c
    return out


def scan(min_bytes: int = 2 << 20, root: str = "/", page: Optional[int] = None) -> dict:
    """The report as a dict: per node and in total."""
    page = page or page_size()
    buddy = buddy_orders(root)
    ids = nodes(root) or sorted(buddy) or []
    report = {"page_size": page, "min_run_bytes": min_bytes, "nodes": []}
    for n in ids:
        mi = node_meminfo(n, root)
        orders = buddy.get(n)
        entry = {"node": n, "total_bytes": mi.get("MemTotal"), "free_bytes": mi.get("MemFree"), "hugepages": node_hugepages(n, root)}
        if orders is not None:
            largest = max((i for i, c in enumerate(orders) if c), default=None)
            entry["largest_free_run_bytes"] = None if largest is None else page << largest
            entry["free_in_runs_of_min_bytes"] = sum(c * (page << i) for i, c in enumerate(orders) if (page << i) >= min_bytes)
            entry["free_in_buddy_bytes"] = sum(c * (page << i) for i, c in enumerate(orders))
        report["nodes"].append(entry)
    known = [e for e in report["nodes"] if e.get("free_bytes") is not None]
    report["total_free_bytes"] = sum(e["free_bytes"] for e in known) if known else None
    runs = [e["free_in_runs_of_min_bytes"] for e in report["nodes"] if "free_in_runs_of_min_bytes" in e]
    report["total_free_in_runs_of_min_bytes"] = sum(runs) if runs else None
    return report


def render(report: dict) -> str:
    def mb(v):
        return "      n/a" if v is None else f"{v / (1 << 20):9.0f}"
    lines = [f"page {report['page_size']} B; runs of at least {report['min_run_bytes'] >> 20} MiB count as usable without compaction",
             f"{'node':>4} {'total MiB':>10} {'free MiB':>10} {'in runs MiB':>12} {'largest run':>12}  huge pages (free/total)"]
    for e in report["nodes"]:
        hp = ", ".join(f"{k}: {v['free']}/{v['total']}" for k, v in e["hugepages"].items()) or "-"
        lr = e.get("largest_free_run_bytes")
        lines.append(f"{e['node']:>4} {mb(e['total_bytes']):>10} {mb(e['free_bytes']):>10} {mb(e.get('free_in_runs_of_min_bytes')):>12} "
                     f"{('n/a' if lr is None else str(lr >> 10) + ' KiB'):>12}  {hp}")
    if not report["nodes"]:
        lines.append("   (no NUMA information visible here)")
    lines.append(f"free in total: {mb(report['total_free_bytes']).strip()} MiB, of which in runs: {mb(report['total_free_in_runs_of_min_bytes']).strip()} MiB")
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="free host memory per NUMA node, huge pages and fragmentation")
    ap.add_argument("--min-mb", type=int, default=2, help="smallest contiguous run that counts as usable")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--root", default="/", help="tree that holds proc/ and sys/ (default: this machine)")
    a = ap.parse_args(argv)
    rep = scan(a.min_mb << 20, a.root)
    print(json.dumps(rep, indent=1) if a.json else render(rep))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
