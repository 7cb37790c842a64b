"""Measurement helpers shared by bench.py and the sweep scripts: clock sampling during the timed
region, device-side timing with CUDA events, max-over-ranks reduction and the KV-block layout."""
from __future__ import annotations

import os
import statistics
import subprocess
import threading
import time

KIB = 1024
# One DeepSeek-R1 KV block: 61 layers x (128 KiB K/V + 16 KiB rope) = 122 discrete segments, 8784 KiB.
KV_LAYERS = 61
KV_SEG_BYTES = (128 * KIB, 16 * KIB)
KV_BLOCK_BYTES = KV_LAYERS * sum(KV_SEG_BYTES)
KV_SEGMENTS = KV_LAYERS * len(KV_SEG_BYTES)


def kv_block_segments(n_blocks: int):
    """(offset, size) of every segment of n_blocks KV blocks laid out per layer, as a serving engine holds
    them: for each layer a K/V array [n_blocks, 128 KiB] and a rope array [n_blocks, 16 KiB]; one block is
    therefore 122 pieces that are NOT adjacent to one another."""
    segs = []
    base = 0
    for _layer in range(KV_LAYERS):
        for seg in KV_SEG_BYTES:
            for b in range(n_blocks):
                segs.append((b, base + b * seg, seg))
            base += n_blocks * seg
    segs.sort(key=lambda t: t[0])  # block-major order, the order a block-wise put walks them
    return [(off, size) for _b, off, size in segs]


class ClockSampler:
    """Reads SM clock and throttle reasons of one GPU while a timed region runs (reads only: nothing is ever set).
    NVML from a thread every 2 ms, so that a region of a few milliseconds still gets samples of its own; nvidia-smi every
    200 ms where NVML cannot be loaded. ``stop()`` -> {"sm_mhz": median, "sm_max_mhz", "reasons": [...], "samples": n}."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    # bits of nvmlDeviceGetCurrentClocksEventReasons (same values as the older ...ThrottleReasons call)
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, gpu_index: int = 0):
        self.gpu = gpu_index
        self.samples = []          # nvidia-smi rows
        self._sm, self._reasons, self._max = [], set(), None
        self._proc = None
        self._thread = None
        self._stop = threading.Event()
        self._nvml = None

    def _nvml_handle(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            # LOCAL_RANK indexes the devices this process may see: honour CUDA_VISIBLE_DEVICES when it lists plain indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v for v in vis.split(",") if v.strip().isdigit()]
            phys = int(ids[self.gpu]) if self.gpu < len(ids) else self.gpu
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self._max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
            return h
        except Exception:  # noqa: BLE001  (no NVML: fall back to nvidia-smi)
            return None

    def _poll_nvml(self, h):
        nv = self._nvml
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self._stop.is_set():
            try:
                self._sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                bits = int(reasons_fn(h))
                for name, bit in self.REASON_BITS.items():
                    if bits & bit:
                        self._reasons.add(name)
            except Exception:  # noqa: BLE001
                break
            time.sleep(0.002)

    def start(self):
        h = self._nvml_handle()
        if h is not None:
            self._thread = threading.Thread(target=self._poll_nvml, args=(h,), daemon=True)
            self._thread.start()
            return self
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()
        return self

    def _read(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self._nvml is not None:
            self._stop.set()
            if self._thread is not None:
                self._thread.join(timeout=1)
            sm = self._sm
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self._max, "reasons": sorted(self._reasons),
                    "samples": len(sm), "source": "nvml, 2 ms"}
        if self._proc is not None:
            time.sleep(0.25)
            self._proc.terminate()
            try:
                self._proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for p in self.samples:
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(names, p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi, 200 ms"}


def max_over_ranks(value: float) -> float:
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier():
    import torch
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    torch.cuda.synchronize()


def env_rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
