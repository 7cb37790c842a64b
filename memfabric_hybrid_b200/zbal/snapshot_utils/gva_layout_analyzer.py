"""An address-ordered model of an allocator trace: segments appear and disappear, blocks are carved out of a segment's
free space and merged back with their free neighbours when released. Feeding it the ``device_traces`` of a snapshot
gives the layout at the end of the trace (used / free blocks, the holes between segments); two models compare equal
when their layouts match up to a shift of the base address, which is how a replay is checked against the original.
Parity: app/zbal/simulator/python/snapshot_utils/gva_layout_analyzer.py of the reference (same class and method names)."""
from __future__ import annotations

import bisect
from typing import Dict, Iterable, List, Optional, Tuple


class Block:
    __slots__ = ("addr", "size", "status", "segment_id")

    def __init__(self, addr: int, size: int, status: str, segment_id: int):
        self.addr, self.size, self.status, self.segment_id = addr, size, status, segment_id   # status: 'FREE' | 'USED'

    def __repr__(self) -> str:
        return f"<{self.status} | Addr: {self.addr}, Size: {self.size}>"


class MemoryAllocatorSimulator:
    def __init__(self, gva_base_addr: Optional[int] = None, gva_size: int = 58 * (1024 ** 3)):
        self.gva_base_addr = gva_base_addr      # None: the first segment's address
        self.gva_size = gva_size
        self.segments: Dict[int, int] = {}      # start -> end
        self._addrs: List[int] = []             # block start addresses, ascending
        self._blocks: Dict[int, Block] = {}

    # ---- the ordered block table ----
    def _put(self, b: Block) -> None:
        if b.addr not in self._blocks:
            bisect.insort(self._addrs, b.addr)
        self._blocks[b.addr] = b

    def _drop(self, addr: int) -> Block:
        i = bisect.bisect_left(self._addrs, addr)
        del self._addrs[i]
        return self._blocks.pop(addr)

    def _covering(self, addr: int) -> Optional[Block]:
        i = bisect.bisect_right(self._addrs, addr) - 1
        return self._blocks[self._addrs[i]] if i >= 0 else None

    def _neighbour(self, addr: int, step: int) -> Optional[Block]:
        i = bisect.bisect_left(self._addrs, addr) + step
        return self._blocks[self._addrs[i]] if 0 <= i < len(self._addrs) else None

    # ---- trace actions ----
    def _segment_alloc(self, addr: int, size: int) -> None:
        if self.gva_base_addr is None:
            self.gva_base_addr = addr
        for lo, hi in self.segments.items():
            if addr < hi and lo < addr + size:
                raise ValueError(f"segment [{addr:#x}, {addr + size:#x}) overlaps [{lo:#x}, {hi:#x})")
        self.segments[addr] = addr + size
        self._put(Block(addr, size, "FREE", addr))

    def _segment_free(self, addr: int) -> None:
        if addr not in self.segments:
            raise ValueError("can't free unallocated segment")
        b = self._blocks.get(addr)
        if b is None or b.status != "FREE" or b.size != self.segments[addr] - addr:
            raise ValueError("a segment must be entirely free when it is released")
        self._drop(addr)
        del self.segments[addr]

    def _alloc(self, addr: int, size: int) -> None:
        host = self._covering(addr)
        if host is None:
            raise ValueError("block must belong to a segment")
        if host.status != "FREE" or addr + size > host.addr + host.size:
            raise ValueError("range must be free")
        self._drop(host.addr)
        if addr > host.addr:
            self._put(Block(host.addr, addr - host.addr, "FREE", host.segment_id))
        self._put(Block(addr, size, "USED", host.segment_id))
        tail = host.addr + host.size - (addr + size)
        if tail > 0:
            self._put(Block(addr + size, tail, "FREE", host.segment_id))

    def _free(self, addr: int) -> None:
        b = self._blocks.get(addr)
        if b is None:
            raise ValueError("addr to be free must be allocated")
        if b.status != "USED":
            raise ValueError("status of to be free block must be USED")
        b.status = "FREE"
        nxt = self._neighbour(addr, +1)
        if nxt is not None and nxt.status == "FREE" and nxt.segment_id == b.segment_id and b.addr + b.size == nxt.addr:
            b.size += nxt.size
            self._drop(nxt.addr)
        prv = self._neighbour(addr, -1)
        if prv is not None and prv.status == "FREE" and prv.segment_id == b.segment_id and prv.addr + prv.size == b.addr:
            prv.size += b.size
            self._drop(addr)

    def simulate(self, device_trace_operations: Iterable[dict], progress: bool = False) -> "MemoryAllocatorSimulator":
        ops = device_trace_operations
        if progress:
            try:
                from tqdm import tqdm
                ops = tqdm(list(ops), desc="Processing simulate")
            except ImportError:
                pass
        for te in ops:
            action = te["action"]
            if action == "segment_alloc":
                self._segment_alloc(te["addr"], te["size"])
            elif action == "segment_free":
                self._segment_free(te["addr"])
            elif action == "alloc":
                self._alloc(te["addr"], te["size"])
            elif action == "free_completed":
                self._free(te["addr"])
            # free_requested, empty_cache, snapshot, oom: no change of the layout
        return self

    # ---- queries ----
    def get_all_segments(self) -> List[Tuple[int, int]]:
        return list(self.segments.items())

    def get_all_blocks(self) -> List[Block]:
        return [self._blocks[a] for a in self._addrs]

    def get_free_blocks(self) -> List[Block]:
        return [b for b in self.get_all_blocks() if b.status == "FREE"]

    def get_used_blocks(self) -> List[Block]:
        return [b for b in self.get_all_blocks() if b.status == "USED"]

    def get_free_space(self) -> List[int]:
        """Sizes of the address ranges that belong to no segment, in address order; the last entry is what is left
        behind the highest segment (up to gva_base_addr + gva_size)."""
        base = self.gva_base_addr or 0
        out, pos = [], base
        for start in sorted(self.segments):
            if start > pos:
                out.append(start - pos)
            pos = max(pos, self.segments[start])
        out.append(base + self.gva_size - pos)
        return out

    def used_bytes(self) -> int:
        return sum(b.size for b in self.get_used_blocks())

    def largest_free_block(self) -> int:
        return max((b.size for b in self.get_free_blocks()), default=0)

    def fragmentation(self) -> float:
        """1 - largest free block / all free bytes inside the segments (0: one hole, towards 1: many small ones)."""
        free = sum(b.size for b in self.get_free_blocks())
        return 0.0 if free == 0 else 1.0 - self.largest_free_block() / free

    def __eq__(self, other) -> bool:
        if not isinstance(other, MemoryAllocatorSimulator):
            return NotImplemented
        if self.gva_size != other.gva_size or len(self._addrs) != len(other._addrs) or len(self.segments) != len(other.segments):
            return False
        shift = (other.gva_base_addr or 0) - (self.gva_base_addr or 0)
        return (all(b - a == shift for a, b in zip(self._addrs, other._addrs)) and
                all(b - a == shift for a, b in zip(sorted(self.segments), sorted(other.segments))))

    __hash__ = None
