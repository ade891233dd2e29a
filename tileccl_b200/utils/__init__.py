"""Utilities: feature gates, topology helpers, profiling, benchmark-result helpers, clocks."""

from . import benchmark_results, clocks, config, feature_gates, profiling, topology
from .config import RuntimeConfig

__all__ = ["benchmark_results", "clocks", "config", "feature_gates", "profiling", "topology",
           "RuntimeConfig"]
