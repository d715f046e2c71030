"""Timing helpers: device-timed step loops (CUDA events, max over ranks) and a clock / throttle-reason
sampler that runs ``nvidia-smi`` beside the timed region."""
from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import Callable, Tuple

import torch
import torch.distributed as dist


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU while a region runs: NVML from a
    thread every 20 ms (no start-up delay, so even a sub-second region gets samples), ``nvidia-smi``
    every 200 ms where NVML cannot be loaded."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
    # NVML clocks-event-reason bits, in the order of NAMES
    BITS = (0x8, 0x40, 0x20, 0x4)

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self.samples = []  # (sm MHz, power W, reason mask)
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        try:
            import torch

            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        return pynvml, handle

    def _poll(self, pynvml, handle):
        reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop.is_set():
            try:
                sm = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                power = pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0
                mask = int(reasons_fn(handle))
                self.samples.append((float(sm), power, mask))
            except Exception:
                pass
            self._stop.wait(0.02)

    def start(self):
        try:
            pynvml, handle = self._nvml_handle()
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
            self._thread = threading.Thread(target=self._poll, args=(pynvml, handle), daemon=True)
            self._thread.start()
            return self
        except Exception:
            self._nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self._nvml is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            sm = [s[0] for s in self.samples]
            power = [s[1] for s in self.samples]
            reasons = sorted({n for _, _, m in self.samples for n, b in zip(self.NAMES, self.BITS) if m & b})
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.sm_max,
                    "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": reasons,
                    "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons),
                "source": "nvidia-smi"}


def timed_steps(fn: Callable[[int], object], steps: int, device: torch.device) -> Tuple[float, float, dict, object]:
    """Run ``fn(i)`` for ``steps`` iterations between a barrier + synchronize on both sides.
    Returns (device milliseconds, wall milliseconds, clock record, last return value); both times are
    the maximum over the ranks of the default group."""
    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize(device)
    sampler = ClockSampler(device.index or 0).start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    last = None
    for i in range(steps):
        last = fn(i)
    e1.record()
    torch.cuda.synchronize(device)
    wall = (time.perf_counter() - t0) * 1e3
    if dist.is_initialized():
        dist.barrier()
    clocks = sampler.stop()
    ms = torch.tensor([e0.elapsed_time(e1), wall], device=device, dtype=torch.float64)
    if dist.is_initialized():
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms[0].item(), ms[1].item(), clocks, last
