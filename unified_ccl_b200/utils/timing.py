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
    """Samples SM clock, power and throttle reasons while a region runs.

    Reads NVML in a thread of this process every ``period_ms`` (so that even a region of a few
    milliseconds gets samples); falls back to an ``nvidia-smi -lms`` child when the NVML module
    is not importable.  Only reads: no clock, power or mode setting is touched."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    # NVML clocks-event (throttle) reason bits
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, gpu_index=0, period_ms=2):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.samples, self._proc, self._thread = [], None, None
        self._stop = threading.Event()
        self._nvml = None
        self._handle = None

    # ---- NVML path
    def _nvml_open(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = None
            try:
                import torch
                uuid = getattr(torch.cuda.get_device_properties(self.gpu_index), "uuid", None)
                if uuid is not None:
                    u = str(uuid)
                    handle = pynvml.nvmlDeviceGetHandleByUUID(u if u.startswith("GPU-") else "GPU-" + u)
            except Exception:  # noqa: BLE001 - any failure falls back to the plain index
                handle = None
            if handle is None:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self._nvml, self._handle = pynvml, handle
            # constant for the device: read once, so that a sample is two or three NVML calls, not four
            self._max_sm = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            return True
        except Exception:  # noqa: BLE001
            self._nvml = None
            return False

    def _nvml_sample(self):
        n, h = self._nvml, self._handle
        sm = n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)
        mx = self._max_sm
        try:
            watts = n.nvmlDeviceGetPowerUsage(h) / 1000.0
        except Exception:  # noqa: BLE001
            watts = 0.0
        getter = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(
            n, "nvmlDeviceGetCurrentClocksThrottleReasons")
        bits = int(getter(h))
        row = [str(sm), str(mx), "%.1f" % watts]
        for name in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"):
            row.append("Active" if bits & self.REASON_BITS[name] else "Not Active")
        self.samples.append(row)

    def _nvml_loop(self):
        while not self._stop.is_set():
            try:
                self._nvml_sample()
            except Exception:  # noqa: BLE001
                break
            self._stop.wait(self.period_ms / 1000.0)

    # ---- nvidia-smi path
    def _read(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def __enter__(self):
        if self._nvml_open():
            self._thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self._thread.start()
            return self
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(max(self.period_ms, 20))], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=self._read, daemon=True)
            self._thread.start()
        except OSError:
            self._proc = None
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._nvml is not None:
            if self._thread:
                self._thread.join(timeout=1)
            try:
                self._nvml.nvmlShutdown()
            except Exception:  # noqa: BLE001
                pass
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
        for s in list(self.samples):
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
