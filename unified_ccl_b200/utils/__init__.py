"""Benchmark and measurement helpers."""
from .timing import ClockSampler, device_time_ms, flush_l2  # noqa: F401
