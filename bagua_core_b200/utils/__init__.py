"""Measurement helpers: clock sampling during a timed region, device timers, peaks."""
from .clocks import ClockSampler  # noqa: F401
from .timing import cuda_time_ms, flush_l2, load_measured_peaks  # noqa: F401
from .prefetch import DevicePrefetcher, LaggedScalarReader  # noqa: F401
