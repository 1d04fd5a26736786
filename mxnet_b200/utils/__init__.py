"""Small shared helpers (clock sampling for benchmarks, launch helpers)."""
from .clocks import ClockSampler
