"""Choice of overlap pattern for a problem shape.

The reference hard-codes K / N thresholds measured on H100 PCIe and scales them
by link bandwidth (tileccl/patterns/auto_select.py:41-191).  Here each pattern's
time is estimated from the alpha-beta cost model for the actual machine
(148 SMs, NVLink 5 behind NVSwitch, measured GEMM peak when a peaks file is
present) and the cheapest wins:

  bulk_sync          gemm + push                      (no overlap, two launches)
  producer_consumer  max(gemm, push) + one band       (two launches, two streams)
  fused_sequential   max(gemm, push) + store latency per tile wave
  wg_specialized     max(gemm, push) + one tile       (bulk stores, deferred signals)

``auto_select`` keeps the reference's calling convention: it returns an instance
when ``ctx`` is given, otherwise the class.
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Any, Optional

from ..planning.cost_model import HardwareProfile, TileCostModel

SUPPORTED_OPS = ("gemm_allscatter", "gemm_allgather", "gemm_reducescatter")
_LAUNCH_US = 4.0          # cost of one extra kernel launch on the critical path
_STORE_RTT_US = 3.0       # system-scope fence after plain peer stores
_TILE_M, _TILE_N = 128, 256


@dataclass(frozen=True)
class HardwareInfo:
    """What the selector needs to know about the machine."""

    compute_units: int = 148
    link_bandwidth_gbps: float = 900.0
    gemm_tflops: float = 2250.0
    gemm_efficiency: float = 0.7


def _detect_hardware_info(ctx=None) -> HardwareInfo:
    prof = HardwareProfile.b200_measured(
        peaks_path=os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(
            os.path.abspath(__file__)))), "MEASURED_PEAKS.json"))
    sms, bw = 148, prof.bandwidth_gb_s
    topo = getattr(ctx, "topology", None) if ctx is not None else None
    if topo is not None:
        sms = getattr(topo, "num_compute_units", 0) or sms
        bw = getattr(topo, "bandwidth_gbps", 0.0) or bw
    return HardwareInfo(sms, bw, prof.gemm_tflops_fp16, prof.gemm_efficiency)


def estimate_pattern_times(M: int, N: int, K: int, world_size: int,
                           hw: Optional[HardwareInfo] = None) -> dict:
    """Estimated microseconds per pattern for the full/full all-scatter contract."""
    hw = hw or HardwareInfo()
    ws = max(world_size, 1)
    model = TileCostModel(HardwareProfile(1.0, 1e6 / (hw.link_bandwidth_gbps * 1e9),
                                          hw.gemm_tflops, hw.gemm_efficiency))
    gemm = model.tile_compute_time(M, N, K)
    push_bytes = M * (N // ws) * 2 * (ws - 1)
    push = model.comm_time_bytes(push_bytes) if ws > 1 else 0.0
    tiles = math.ceil(M / _TILE_M) * math.ceil(N / _TILE_N)
    waves = math.ceil(tiles / max(hw.compute_units, 1))
    one_tile = model.tile_compute_time(_TILE_M, _TILE_N, K)
    band = model.comm_time_bytes(_TILE_M * (N // ws) * 2 * max(ws - 1, 1))
    return {
        "bulk_sync": gemm + push + _LAUNCH_US,
        "producer_consumer": max(gemm, push) + band + _LAUNCH_US,
        "fused_sequential": max(gemm, push) + waves * _STORE_RTT_US,
        "wg_specialized": max(gemm, push) + one_tile,
    }


def auto_select(op: str, M: int, N: int, K: int, world_size: int = 1, ctx: Any = None,
                hw_info: Any = None):
    from . import PATTERN_CLASSES

    if op not in SUPPORTED_OPS:
        raise ValueError(f"Unsupported operation {op!r}.  Supported operations: {sorted(SUPPORTED_OPS)}")
    if hw_info is not None:
        hw = HardwareInfo(getattr(hw_info, "compute_units", 148),
                          getattr(hw_info, "link_bandwidth_gbps", 900.0),
                          getattr(hw_info, "gemm_tflops", 2250.0),
                          getattr(hw_info, "gemm_efficiency", 0.7))
    else:
        hw = _detect_hardware_info(ctx)
    if M < 256 or world_size <= 1:
        # too few rows for a persistent overlap to pay / nothing to push
        name = "bulk_sync" if world_size > 1 else "fused_sequential"
    else:
        times = estimate_pattern_times(M, N, K, world_size, hw)
        name = min(times, key=times.get)
    cls = PATTERN_CLASSES[name]
    return cls(ctx) if ctx is not None else cls


def benchmark_all_patterns(ctx, A, B, C, *, warmup: int = 5, iters: int = 20,
                           patterns: Optional[list] = None, **execute_kwargs) -> dict:
    """Time every pattern on the given tensors (CUDA events); failures are recorded, not raised."""
    from . import PATTERN_CLASSES

    results, errors = [], {}
    for name in patterns or list(PATTERN_CLASSES):
        try:
            results.append(PATTERN_CLASSES[name](ctx).benchmark(A, B, C, warmup=warmup, iters=iters,
                                                                **execute_kwargs))
        except Exception as exc:  # keep going: one broken pattern must not hide the others
            errors[name] = f"{type(exc).__name__}: {exc}"
    results.sort(key=lambda r: r["mean_ms"])
    return {"results": results, "errors": errors, "best": results[0]["pattern"] if results else "none",
            "shape": {"M": A.shape[0], "K": A.shape[1], "N": B.shape[1]},
            "world_size": ctx.world_size}
