"""Metrics, tracing, environment flags."""
from .flags import Flags, apply_truncate_layers  # noqa: F401
from .metrics import GLOBAL as METRICS, KernelRoofline, MetricsRegistry, Quantiles  # noqa: F401
from .tracing import ChromeTrace, DeviceTimer, nvtx_range  # noqa: F401
