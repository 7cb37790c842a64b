"""Drawings and exports of allocator snapshots in the memory visualiser's layout. The drawings are SVG text (returned,
and written to ``output`` when given): one horizontal bar for the address range, segments in grey, blocks in use in
green, cached / inactive blocks in orange, holes between segments hatched in red. No plotting library is needed.
``parse_mem_to_profile`` turns a trace into a Chrome-trace file (chrome://tracing, Perfetto): one bar per allocation's
lifetime in a lane by size class, and a counter of the bytes allocated.
Parity: app/zbal/simulator/python/snapshot_utils/gva_layout_viz.py of the reference (same function names and arguments;
the reference draws with matplotlib)."""
from __future__ import annotations

import json
import pickle
from typing import Dict, List, Optional, Sequence, Tuple

from .gva_layout_analyzer import MemoryAllocatorSimulator

GIB = 1024 ** 3
MIB = 1024 ** 2
_W, _H, _PAD = 1200, 150, 40
_COL = {"range": "#f0f0f0", "segment": "#bdbdbd", "used": "#4caf50", "inactive": "#ff9800", "gap": "#ffcccc"}


def _int(v) -> int:
    return int(v, 16) if isinstance(v, str) else int(v)


class _Canvas:
    """A bar over [base, base + span) bytes, drawn into a fixed-size SVG."""

    def __init__(self, base: int, span: int, title: str):
        self.base, self.span = base, max(1, span)
        self.items: List[str] = [f'<text x="{_PAD}" y="20" font-size="14" font-family="sans-serif">{title}</text>']
        self.rect(base, span, 30, 90, _COL["range"])

    def x(self, addr: int) -> float:
        return _PAD + (addr - self.base) / self.span * (_W - 2 * _PAD)

    def rect(self, addr: int, size: int, y: float, h: float, fill: str, opacity: float = 1.0, stroke: str = "none") -> None:
        lo, hi = max(addr, self.base), min(addr + size, self.base + self.span)
        if hi <= lo:
            return
        w = max(0.5, self.x(hi) - self.x(lo))
        self.items.append(f'<rect x="{self.x(lo):.2f}" y="{y}" width="{w:.2f}" height="{h}" fill="{fill}" fill-opacity="{opacity}" stroke="{stroke}" stroke-width="0.3"/>')

    def label(self, addr: int, y: float, text: str, colour: str = "#000") -> None:
        self.items.append(f'<text x="{self.x(addr):.1f}" y="{y}" font-size="10" font-family="sans-serif" text-anchor="middle" fill="{colour}">{text}</text>')

    def finish(self, legend: Sequence[Tuple[str, str]], output: Optional[str]) -> str:
        for i in range(9):   # ticks: offsets from the base in GiB
            a = self.base + self.span * i // 8
            self.items.append(f'<line x1="{self.x(a):.1f}" y1="120" x2="{self.x(a):.1f}" y2="125" stroke="#000"/>')
            self.label(a, 137, f"+{(a - self.base) / GIB:.2f}G")
        lx = _W - _PAD - 130 * len(legend)
        for i, (name, colour) in enumerate(legend):
            self.items.append(f'<rect x="{lx + 130 * i}" y="8" width="12" height="12" fill="{colour}" stroke="#000" stroke-width="0.3"/>')
            self.items.append(f'<text x="{lx + 130 * i + 16}" y="18" font-size="11" font-family="sans-serif">{name}</text>')
        svg = (f'<svg xmlns="http://www.w3.org/2000/svg" width="{_W}" height="{_H}" viewBox="0 0 {_W} {_H}">' + "".join(self.items) + "</svg>")
        if output:
            with open(output, "w") as f:
                f.write(svg)
        return svg


def visualize_sim_memory(simulator: MemoryAllocatorSimulator, display_segments: bool = False, display_blocks: bool = True,
                         output: Optional[str] = None) -> str:
    """The layout a MemoryAllocatorSimulator holds after ``simulate``."""
    base = simulator.gva_base_addr or 0
    c = _Canvas(base, simulator.gva_size, f"Memory layout (total {simulator.gva_size / GIB:.1f} GiB, base {base:#x})")
    legend = [("unused", _COL["range"])]
    if display_segments:
        for lo, hi in simulator.get_all_segments():
            c.rect(lo, hi - lo, 33, 84, _COL["segment"], 0.5, "#000")
        legend.append(("segment", _COL["segment"]))
    if display_blocks:
        for b in simulator.get_used_blocks():
            c.rect(b.addr, b.size, 38, 74, _COL["used"], 0.85, "#000")
        legend.append(("block in use", _COL["used"]))
    return c.finish(legend, output)


def parser_file_ops(input_file_path: str, device_id: int = 0, get_traces: bool = True):
    """Loads a ``.pkl`` or ``.json`` snapshot in the visualiser's layout -> the trace of one device, or the segment list."""
    if input_file_path.endswith((".pkl", ".pickle")):
        with open(input_file_path, "rb") as f:
            snap = pickle.load(f)
    elif input_file_path.endswith(".json"):
        with open(input_file_path, "r", encoding="utf-8") as f:
            snap = json.load(f)
    else:
        raise ValueError("not support layout file format")
    if "device_traces" not in snap and "blocks" in snap and "heap" in snap:   # the allocator's own JSON layout
        from ..module import memviz_snapshot
        snap = memviz_snapshot(snap)
    return snap["device_traces"][device_id] if get_traces else snap["segments"]


def _live_at_end(operations: Sequence[dict], begin: str, end: str) -> Tuple[Dict[int, int], int]:
    live: Dict[int, int] = {}
    most = 0
    for op in operations:
        if op["action"] == begin:
            live[_int(op["addr"])] = op["size"]
            most = max(most, len(live))
        elif op["action"] == end:
            live.pop(_int(op["addr"]), None)
    return live, most


def visualize_file_memory(total_size_gb: float, start_addr, operations: Sequence[dict], display_segments: bool = True,
                          display_blocks: bool = True, output: Optional[str] = None) -> str:
    """What is alive at the end of a trace (``device_traces[device]``): segments and blocks over a range of
    ``total_size_gb`` GiB that starts at the lowest address seen (or ``start_addr`` if that is lower)."""
    base = _int(start_addr)
    segs, seg_most = _live_at_end(operations, "segment_alloc", "segment_free") if display_segments else ({}, 0)
    blks, blk_most = _live_at_end(operations, "alloc", "free_completed") if display_blocks else ({}, 0)
    for a in list(segs) + list(blks):
        base = min(base, a)
    print(f"blocks info: max num:[{blk_most}], active num:[{len(blks)}]")
    print(f"segments info: max num:[{seg_most}], active num:[{len(segs)}]")
    c = _Canvas(base, int(total_size_gb * GIB), f"Memory layout at the end of the trace (total {total_size_gb} GiB, base {base:#x})")
    for a, n in segs.items():
        c.rect(a, n, 33, 84, _COL["segment"], 0.5, "#000")
    for a, n in blks.items():
        c.rect(a, n, 38, 74, _COL["used"], 0.85, "#000")
    return c.finish([("unused", _COL["range"]), ("segment", _COL["segment"]), ("block in use", _COL["used"])], output)


def visualize_file_snapshot(total_size_gb: float, start_addr, operations: Sequence[dict], output: Optional[str] = None) -> List[dict]:
    """``operations``: the ``segments`` list of a snapshot. Draws segments, their active and inactive blocks and the holes
    between segments; returns the holes, largest first (gap_start, gap_end, size, size_mb). ``total_size_gb`` 0: the
    range is what the segments span. The drawing goes to ``output`` (SVG) when given."""
    segs = sorted(operations, key=lambda s: s["address"])
    gaps = []
    for cur, nxt in zip(segs, segs[1:]):
        end = cur["address"] + cur["total_size"]
        if nxt["address"] > end:
            gaps.append({"gap_start": end, "gap_end": nxt["address"], "size": nxt["address"] - end, "size_mb": (nxt["address"] - end) / MIB})
    if segs:
        base = min(segs[0]["address"], _int(start_addr))
        span = int(total_size_gb * GIB) if total_size_gb > 0 else max(s["address"] + s["total_size"] for s in segs) - base
        c = _Canvas(base, span, f"Memory layout and gaps (base {base:#x})")
        for g in gaps:
            c.rect(g["gap_start"], g["size"], 30, 90, _COL["gap"], 0.6, "#ff5252")
            if g["size_mb"] > 100:
                c.label(g["gap_start"] + g["size"] // 2, 116, f"gap {g['size_mb']:.0f} MB", "#c00")
        for s in segs:
            c.rect(s["address"], s["total_size"], 33, 84, _COL["segment"], 0.5, "#000")
            for b in s.get("blocks", []):
                c.rect(b["address"], b["size"], 42, 60, _COL["used"] if b["state"] == "active_allocated" else _COL["inactive"], 0.85, "#000")
        c.finish([("segment", _COL["segment"]), ("active block", _COL["used"]), ("inactive block", _COL["inactive"]), ("gap", _COL["gap"])], output)
    return sorted(gaps, key=lambda g: g["size"], reverse=True)


def _lane(size: int) -> str:
    mb = size / MIB
    return "< 16MB (Small)" if mb < 16 else ("16MB - 128MB (Medium)" if mb <= 128 else "> 128MB (Large)")


def parse_mem_to_profile(operations: Sequence[dict], output_file: str, export_segments: bool = True, with_unfree: bool = False,
                         process_name: str = "GPU_HBM") -> int:
    """A trace -> Chrome-trace JSON: every segment (``export_segments``) or block lifetime becomes a bar in the lane of
    its size class, a counter follows the bytes allocated; ``with_unfree`` adds what was never released. One logical
    time step (100 us) per trace entry. Returns the number of events written."""
    begin, end = ("segment_alloc", "segment_free") if export_segments else ("alloc", "free_completed")
    lanes = ["> 128MB (Large)", "16MB - 128MB (Medium)", "< 16MB (Small)"]
    events: List[dict] = []
    for i, name in enumerate(lanes):
        events.append({"name": "thread_name", "ph": "M", "pid": process_name, "tid": name, "args": {"name": name}})
        events.append({"name": "thread_sort_index", "ph": "M", "pid": process_name, "tid": name, "args": {"sort_index": i}})
    live: Dict[int, Tuple[int, int]] = {}
    ts = usage = 0

    def counter() -> None:
        events.append({"name": "Memory Usage", "ph": "C", "ts": ts, "pid": process_name, "args": {"Allocated_MB": usage / MIB}})

    def bar(prefix: str, addr: int, start: int, size: int, extra: dict) -> None:
        events.append({"name": f"{prefix}_{size / MIB:.2f}_MB", "ph": "X", "ts": start, "dur": ts - start, "pid": process_name, "tid": _lane(size),
                       "args": {"address": hex(addr), "size": f"{size / MIB:.2f} MB", **extra}})

    for op in operations:
        ts += 100
        action = op["action"]
        if action == begin:
            live[_int(op["addr"])] = (ts, op["size"])
            usage += op["size"]
            counter()
        elif action == end:
            hit = live.pop(_int(op["addr"]), None)
            if hit is not None:
                bar("Block", _int(op["addr"]), hit[0], hit[1], {"alloc_step": hit[0] // 100})
                usage -= hit[1]
                counter()
    if with_unfree:
        for addr, (start, size) in live.items():
            bar("Unfreed", addr, start, size, {"status": "still_allocated"})
    with open(output_file, "w") as f:
        json.dump({"traceEvents": events}, f, indent=2)
    return len(events)
