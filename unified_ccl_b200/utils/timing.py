"""Device-side timing with CUDA events, L2 flushing and clock sampling during a timed region."""
import subprocess
import threading

import torch

_flush_buf = {}


def flush_l2(device=None):
    """Write a buffer larger than the 126 MB L2 so the next kernel starts from HBM."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    if dev not in _flush_buf:
        _flush_buf[dev] = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    _flush_buf[dev].zero_()


def device_time_ms(fn, iters=20, warmup=5, flush=True, pre=None):
    """Median / min / mean of `fn` timed with CUDA events on the current stream."""
    for _ in range(warmup):
        if pre:
            pre()
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        if pre:
            pre()
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return {"median": times[len(times) // 2], "min": times[0], "mean": sum(times) / len(times)}


class ClockSampler:
    """Samples SM clock, power and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0, period_ms=50):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.samples, self._proc, self._thread = [], None, None

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=self._read, daemon=True)
            self._thread.start()
        except OSError:
            self._proc = None
        return self

    def _read(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self._proc:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        return False

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = max(mx, float(s[1]))
            except ValueError:
                continue
            for name, v in zip(names, s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}
