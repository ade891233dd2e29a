"""alpha-beta cost model for tile pipelines, and its calibrator.

Communication of ``b`` bytes costs ``max(min_comm_us, alpha_us + b * beta_us_per_byte)``;
a GEMM tile costs ``2*M*N*K / (peak * efficiency)``.  A pipeline of ``n`` equal
tiles pays the first tile in full (transfer and compute back to back) and
``max(transfer, compute)`` for each of the rest.  Class and method names follow
the reference (tileccl_v2/cost_model.py:39-593); on top of its four interconnect
presets this module has ``NVLINK_5`` (B200 behind NVSwitch) and
``HardwareProfile.b200_measured`` which takes the GEMM peak from a measured-peaks
file and the link parameters from a calibration file produced on the machine.
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, replace
from enum import Enum, auto
from typing import Optional, Sequence

DTYPE_BYTES = {"float16": 2, "bfloat16": 2, "float32": 4, "float64": 8, "int8": 1, "float8": 1,
               "fp16": 2, "bf16": 2, "fp32": 4}


def _runtime_config():
    from ..utils.config import current

    return current()


class Interconnect(Enum):
    PCIE_GEN4 = auto()
    PCIE_GEN5 = auto()
    NVLINK_3 = auto()
    NVLINK_4 = auto()
    NVLINK_5 = auto()
    CUSTOM = auto()


def _beta_from_gbps(gb_per_s: float) -> float:
    """microseconds per byte at `gb_per_s` GB/s."""
    return 1e6 / (gb_per_s * 1e9)


@dataclass(frozen=True)
class HardwareProfile:
    alpha_us: float
    beta_us_per_byte: float
    gemm_tflops_fp16: float
    gemm_efficiency: float = 0.7
    min_comm_us: float = 0.0
    name: str = "custom"

    @property
    def bandwidth_gb_s(self) -> float:
        if self.beta_us_per_byte <= 0:
            return float("inf")
        return 1e6 / self.beta_us_per_byte / 1e9

    @classmethod
    def from_interconnect(cls, interconnect: Interconnect) -> "HardwareProfile":
        if interconnect is Interconnect.CUSTOM:
            raise ValueError("Use HardwareProfile() directly for custom parameters")
        return _PRESETS[interconnect]

    @classmethod
    def b200_measured(cls, peaks_path: Optional[str] = None,
                      calibration_path: Optional[str] = None) -> "HardwareProfile":
        """NVLINK_5 preset refined by files measured on the machine, when present.

        ``peaks_path``: JSON with ``bf16_tflops`` (cuBLAS burst).  ``calibration_path``:
        JSON with ``alpha_us``, ``beta_us_per_byte`` and optionally ``min_comm_us``
        (written by ``benchmarks/phase0_calibrate.py``); the environment variable
        ``TILECCL_CALIBRATION`` names it, else the ``calibration/b200.json`` that ships
        next to the package (measured on an 8 x B200 NVSwitch machine) is used.
        """
        prof = _PRESETS[Interconnect.NVLINK_5]
        for path, apply in ((peaks_path, _apply_peaks),
                            (globals()["calibration_path"](calibration_path), _apply_calibration)):
            if path and os.path.exists(path):
                try:
                    with open(path) as f:
                        prof = apply(prof, json.load(f))
                except (OSError, ValueError, KeyError):
                    pass
        return prof

    def to_dict(self) -> dict:
        d = dict(self.__dict__)
        d["bandwidth_gb_s"] = self.bandwidth_gb_s
        return d


def _apply_peaks(prof: HardwareProfile, data: dict) -> HardwareProfile:
    return replace(prof, gemm_tflops_fp16=float(data["bf16_tflops"]), gemm_efficiency=0.85,
                   name=prof.name + " + measured GEMM peak")


def _apply_calibration(prof: HardwareProfile, data: dict) -> HardwareProfile:
    """A calibration file may carry two fits.  ``in_kernel`` (preferred): alpha / beta of the
    push phase *inside* the fused kernel, from its %globaltimer trace (fixed in-kernel
    overhead and achieved link rate).  Top level: a whole collective launch per message size
    (includes launch latency and the three-phase protocol)."""
    src = data.get("in_kernel") if isinstance(data.get("in_kernel"), dict) else data
    return replace(prof, alpha_us=float(src["alpha_us"]),
                   beta_us_per_byte=float(src["beta_us_per_byte"]),
                   min_comm_us=float(src.get("min_comm_us", 0.0)),
                   name=prof.name + " (calibrated)")


def calibration_path(explicit: Optional[str] = None) -> str:
    """The link-model file in force: explicit argument, else ``TILECCL_CALIBRATION``, else the
    ``calibration/b200.json`` that ships next to the package."""
    shipped = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__)))), "calibration", "b200.json")
    return explicit or _runtime_config().calibration or shipped


def load_calibration(path: Optional[str] = None) -> dict:
    """Contents of the calibration file (empty dict when it cannot be read)."""
    try:
        with open(calibration_path(path)) as f:
            data = json.load(f)
        return data if isinstance(data, dict) else {}
    except (OSError, ValueError):
        return {}


DEFAULT_TAU_MIN_BYTES = 262144   # the reference's P2P saturation size (tileccl_v2/tile_group.py:22)


def calibrated_tau_min_bytes(path: Optional[str] = None) -> int:
    """Smallest TileGroup worth signalling on its own, from the calibration file: the bytes
    the link moves while one TileGroup signal becomes visible to its consumer
    (``in_kernel.tau_min_bytes``).  Finer groups only add counters that a consumer cannot
    observe any sooner.  Falls back to the reference's constant."""
    data = load_calibration(path)
    ik = data.get("in_kernel")
    if isinstance(ik, dict) and ik.get("tau_min_bytes"):
        return max(1, int(ik["tau_min_bytes"]))
    return DEFAULT_TAU_MIN_BYTES


_PRESETS = {
    Interconnect.PCIE_GEN4: HardwareProfile(5.0, _beta_from_gbps(25), 312.0, 0.6, 0.0,
                                            "PCIe Gen4 (A100)"),
    Interconnect.PCIE_GEN5: HardwareProfile(3.0, _beta_from_gbps(50), 989.0, 0.65, 0.0,
                                            "PCIe Gen5 (H100)"),
    Interconnect.NVLINK_3: HardwareProfile(1.5, _beta_from_gbps(300), 312.0, 0.7, 0.0,
                                           "NVLink 3.0 (A100)"),
    Interconnect.NVLINK_4: HardwareProfile(1.0, _beta_from_gbps(450), 989.0, 0.75, 0.0,
                                           "NVLink 4.0 (H100)"),
    # B200 behind NVSwitch: 900 GB/s per direction nominal; 2250 TFLOPS dense fp16/bf16.
    Interconnect.NVLINK_5: HardwareProfile(1.0, _beta_from_gbps(900), 2250.0, 0.7, 0.0,
                                           "NVLink 5 / NVSwitch (B200)"),
}


@dataclass
class TileCost:
    comm_us: float
    compute_us: float
    tile_bytes: int
    overlap_possible: bool = True

    @property
    def sequential_us(self) -> float:
        return self.comm_us + self.compute_us

    @property
    def overlapped_us(self) -> float:
        return max(self.comm_us, self.compute_us)

    @property
    def compute_bound(self) -> bool:
        return self.compute_us >= self.comm_us


@dataclass
class PipelineCost:
    tile_costs: list
    sequential_us: float
    pipelined_us: float
    overlap_ratio: float
    bottleneck: str

    @property
    def speedup(self) -> float:
        return self.sequential_us / self.pipelined_us if self.pipelined_us > 0 else 1.0

    def summary(self) -> str:
        return (f"Pipeline: {len(self.tile_costs)} tiles, seq={self.sequential_us:.1f}us, "
                f"pipe={self.pipelined_us:.1f}us, speedup={self.speedup:.2f}x, "
                f"overlap={self.overlap_ratio:.1%}, bottleneck={self.bottleneck}")


def _nbytes(tile_M: int, tile_N: int, dtype: str) -> int:
    return tile_M * tile_N * DTYPE_BYTES.get(dtype, 2)


class TileCostModel:
    def __init__(self, profile: HardwareProfile) -> None:
        self.profile = profile

    def comm_time_bytes(self, nbytes: float) -> float:
        p = self.profile
        return max(p.min_comm_us, p.alpha_us + nbytes * p.beta_us_per_byte)

    def tile_comm_time(self, tile_M: int, tile_N: int, dtype: str = "float16") -> float:
        return self.comm_time_bytes(_nbytes(tile_M, tile_N, dtype))

    def tile_compute_time(self, tile_M: int, tile_N: int, tile_K: int,
                          dtype: str = "float16") -> float:
        rate = self.profile.gemm_tflops_fp16 * self.profile.gemm_efficiency  # TFLOP/s
        if rate <= 0:
            return float("inf")
        return 2.0 * tile_M * tile_N * tile_K / (rate * 1e6)

    def tile_cost(self, tile_M: int, tile_N: int, tile_K: int, dtype: str = "float16") -> TileCost:
        return TileCost(self.tile_comm_time(tile_M, tile_N, dtype),
                        self.tile_compute_time(tile_M, tile_N, tile_K, dtype),
                        _nbytes(tile_M, tile_N, dtype))

    def pipeline_cost(self, n_tiles: int, tile_M: int, tile_N: int, tile_K: int,
                      dtype: str = "float16", n_chunks: int = 1) -> PipelineCost:
        tc = self.tile_cost(tile_M, tile_N, tile_K, dtype)
        if n_chunks > 1:
            # Splitting a tile's transfer pays alpha once per chunk.
            per_chunk = self.profile.alpha_us + (tc.tile_bytes // n_chunks) * self.profile.beta_us_per_byte
            tc = TileCost(per_chunk * n_chunks, tc.compute_us, tc.tile_bytes)
        sequential = tc.sequential_us * n_tiles
        pipelined = tc.sequential_us + max(0, n_tiles - 1) * tc.overlapped_us
        ratio = 1.0 - pipelined / sequential if sequential > 0 else 0.0
        return PipelineCost([tc] * n_tiles, sequential, pipelined, ratio,
                            "compute" if tc.compute_bound else "comm")

    def optimal_tile_size(self, M: int, N: int, K: int, dtype: str = "float16",
                          candidates: Optional[Sequence[int]] = None) -> tuple:
        candidates = list(candidates) if candidates is not None else [32, 64, 128, 256, 512]
        best_size, best = candidates[0], None
        for size in candidates:
            if size > M or size > N:
                continue
            n_tiles = math.ceil(M / size) * math.ceil(N / size)
            cost = self.pipeline_cost(n_tiles, size, size, K, dtype)
            if best is None or cost.pipelined_us < best.pipelined_us:
                best_size, best = size, cost
        return best_size, best

    def allreduce_cost(self, M: int, N: int, K: int, world_size: int, tile_size: int = 128,
                       dtype: str = "float16") -> dict:
        per_rank = math.ceil((M // world_size) / tile_size) * math.ceil(N / tile_size)
        phase = self.pipeline_cost(per_rank * (world_size - 1), tile_size, tile_size, K, dtype)
        seq, pipe = 2 * phase.sequential_us, 2 * phase.pipelined_us
        total = PipelineCost(phase.tile_costs + phase.tile_costs, seq, pipe,
                             1.0 - pipe / seq if seq > 0 else 0.0, phase.bottleneck)
        return {"reduce_scatter": phase, "allgather": phase, "total": total}

    def optimal_group_rows(self, rows: int, cols: int, K: int, dtype: str = "float16",
                           block_m: int = 128, max_groups: int = 64) -> tuple:
        """Row-band size (a multiple of ``block_m``) that minimises the pipelined time of
        ``rows x cols`` output produced band by band; returns ``(band_rows, PipelineCost)``."""
        best_rows, best = block_m, None
        tile_rows = math.ceil(rows / block_m)
        for per in range(1, tile_rows + 1):
            n = math.ceil(tile_rows / per)
            if n > max_groups:
                continue
            cost = self.pipeline_cost(n, per * block_m, cols, K, dtype)
            if best is None or cost.pipelined_us < best.pipelined_us:
                best_rows, best = per * block_m, cost
        return best_rows, best


@dataclass
class CalibrationPoint:
    tile_M: int
    tile_N: int
    dtype: str
    measured_comm_us: float
    measured_compute_us: Optional[float] = None

    @property
    def nbytes(self) -> int:
        return _nbytes(self.tile_M, self.tile_N, self.dtype)


class CostModelCalibrator:
    """Least-squares fits of the link parameters from measured transfer times."""

    @staticmethod
    def calibrate_comm(points: Sequence[CalibrationPoint], min_bytes_threshold: int = 0) -> tuple:
        """Ordinary least squares of ``time = alpha + beta * bytes``; both clipped at 0."""
        if len(points) < 2:
            raise ValueError("Need at least 2 calibration points")
        used = [p for p in points if p.nbytes >= min_bytes_threshold]
        if len(used) < 2:
            raise ValueError(f"Need at least 2 points with bytes >= {min_bytes_threshold}, "
                             f"got {len(used)}")
        n = float(len(used))
        sx = sum(float(p.nbytes) for p in used)
        sy = sum(p.measured_comm_us for p in used)
        sxy = sum(p.nbytes * p.measured_comm_us for p in used)
        sxx = sum(float(p.nbytes) ** 2 for p in used)
        det = n * sxx - sx * sx
        if abs(det) < 1e-12:
            raise ValueError("Degenerate calibration data (all same size)")
        beta = (n * sxy - sx * sy) / det
        alpha = (sy - beta * sx) / n
        return max(0.0, alpha), max(0.0, beta)

    @staticmethod
    def calibrate_two_regime(points: Sequence[CalibrationPoint]) -> tuple:
        """``max(floor, alpha + beta * bytes)``: floor = fastest measurement; the line is
        fitted on the larger-and-slower points beyond it (or the two largest points)."""
        if len(points) < 3:
            raise ValueError("Need at least 3 calibration points for two-regime fit")
        ordered = sorted(points, key=lambda p: p.nbytes)
        fastest = min(ordered, key=lambda p: p.measured_comm_us)
        tail = [p for p in ordered
                if p.nbytes > fastest.nbytes and p.measured_comm_us > fastest.measured_comm_us]
        if len(tail) < 2:
            tail = ordered[-2:]
        alpha, beta = CostModelCalibrator.calibrate_comm(tail)
        return alpha, beta, fastest.measured_comm_us

    @staticmethod
    def calibrate_from_measurements(points: Sequence[CalibrationPoint],
                                    base_profile: HardwareProfile,
                                    two_regime: bool = False) -> HardwareProfile:
        if two_regime:
            alpha, beta, floor = CostModelCalibrator.calibrate_two_regime(points)
        else:
            (alpha, beta), floor = CostModelCalibrator.calibrate_comm(points), 0.0
        return HardwareProfile(alpha, beta, base_profile.gemm_tflops_fp16,
                               base_profile.gemm_efficiency, floor,
                               f"{base_profile.name} (calibrated)")

    @staticmethod
    def saturation_bytes(profile: HardwareProfile, fraction: float = 0.9) -> int:
        """Smallest message that reaches ``fraction`` of the link bandwidth under the
        alpha-beta model (this is the tau_min the TileGroup planner should use)."""
        if not 0 < fraction < 1:
            raise ValueError("fraction must be in (0, 1)")
        if profile.beta_us_per_byte <= 0:
            return 0
        return int(math.ceil(fraction / (1 - fraction) * profile.alpha_us / profile.beta_us_per_byte))
