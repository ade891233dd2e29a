"""Utilities: feature gates, topology helpers, profiling, benchmark-result helpers, clocks."""

from . import benchmark_results, clocks, feature_gates, profiling, topology

__all__ = ["benchmark_results", "clocks", "feature_gates", "profiling", "topology"]
