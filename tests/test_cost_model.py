"""alpha-beta cost model and calibrator (CPU only)."""

import math

import pytest

from tileccl_b200.planning import (CalibrationPoint, CostModelCalibrator, HardwareProfile,
                                   Interconnect, TileCostModel)


def test_nvlink4_pipeline_golden():
    m = TileCostModel(HardwareProfile.from_interconnect(Interconnect.NVLINK_4))
    c = m.pipeline_cost(n_tiles=8, tile_M=1024, tile_N=4096, tile_K=1024)
    assert c.sequential_us == pytest.approx(249.78, abs=0.01)
    assert c.pipelined_us == pytest.approx(168.71, abs=0.01)
    assert c.overlap_ratio == pytest.approx(0.325, abs=1e-3)
    assert c.bottleneck == "comm" and c.speedup == pytest.approx(249.78 / 168.71, rel=1e-3)
    assert "8 tiles" in c.summary()


def test_presets_and_custom():
    for ic, gbps in ((Interconnect.PCIE_GEN4, 25), (Interconnect.NVLINK_3, 300),
                     (Interconnect.NVLINK_4, 450), (Interconnect.NVLINK_5, 900)):
        assert HardwareProfile.from_interconnect(ic).bandwidth_gb_s == pytest.approx(gbps)
    with pytest.raises(ValueError):
        HardwareProfile.from_interconnect(Interconnect.CUSTOM)
    assert math.isinf(HardwareProfile(0, 0, 100).bandwidth_gb_s)


def test_two_regime_floor_and_chunking():
    p = HardwareProfile(alpha_us=1.0, beta_us_per_byte=1e-3, gemm_tflops_fp16=100, min_comm_us=37.0)
    m = TileCostModel(p)
    assert m.tile_comm_time(8, 8) == 37.0                       # floor wins for tiny tiles
    assert m.tile_comm_time(256, 256) == pytest.approx(1 + 131072 * 1e-3)
    m = TileCostModel(HardwareProfile(alpha_us=1.0, beta_us_per_byte=1e-3, gemm_tflops_fp16=100))
    one = m.pipeline_cost(4, 128, 128, 64)
    four = m.pipeline_cost(4, 128, 128, 64, n_chunks=4)
    assert four.tile_costs[0].comm_us == pytest.approx(one.tile_costs[0].comm_us + 3 * p.alpha_us)
    assert m.pipeline_cost(1, 128, 128, 64).pipelined_us == one.tile_costs[0].sequential_us


def test_optimal_tile_size_and_allreduce():
    m = TileCostModel(HardwareProfile.from_interconnect(Interconnect.NVLINK_5))
    size, cost = m.optimal_tile_size(4096, 4096, 4096)
    assert size in (32, 64, 128, 256, 512) and cost.pipelined_us > 0
    size2, _ = m.optimal_tile_size(100, 100, 64)
    assert size2 <= 100
    ar = m.allreduce_cost(4096, 4096, 1024, world_size=8)
    assert set(ar) == {"reduce_scatter", "allgather", "total"}
    assert ar["total"].pipelined_us == pytest.approx(2 * ar["allgather"].pipelined_us)
    rows, c = m.optimal_group_rows(2048, 4096, 1024)
    assert rows % 128 == 0 and 128 <= rows <= 2048 and c.pipelined_us > 0


def _pts(alpha, beta, sizes):
    return [CalibrationPoint(n, 1, "int8", alpha + beta * n) for n in sizes]


def test_ols_recovers_alpha_beta():
    a, b = CostModelCalibrator.calibrate_comm(_pts(2.5, 1e-3, [1024, 4096, 65536, 1 << 20]))
    assert a == pytest.approx(2.5, rel=1e-6) and b == pytest.approx(1e-3, rel=1e-6)
    with pytest.raises(ValueError):
        CostModelCalibrator.calibrate_comm(_pts(1, 1, [8]))
    with pytest.raises(ValueError):
        CostModelCalibrator.calibrate_comm(_pts(1, 1, [8, 8]))
    with pytest.raises(ValueError):
        CostModelCalibrator.calibrate_comm(_pts(1, 1, [8, 16]), min_bytes_threshold=1000)


def test_two_regime_fit_finds_floor():
    pts = ([CalibrationPoint(n, 1, "int8", 60.0 - i) for i, n in enumerate([64, 256, 1024])]
           + [CalibrationPoint(1 << 21, 1, "int8", 40.0)]
           + [CalibrationPoint(n, 1, "int8", 5.0 + 2e-5 * n) for n in [1 << 22, 1 << 24, 1 << 26]])
    a, b, floor = CostModelCalibrator.calibrate_two_regime(pts)
    assert floor == 40.0 and b == pytest.approx(2e-5, rel=1e-3) and a == pytest.approx(5.0, rel=1e-2)
    prof = CostModelCalibrator.calibrate_from_measurements(
        pts, HardwareProfile.from_interconnect(Interconnect.NVLINK_5), two_regime=True)
    assert prof.min_comm_us == 40.0 and "calibrated" in prof.name and prof.gemm_tflops_fp16 == 2250.0
    with pytest.raises(ValueError):
        CostModelCalibrator.calibrate_two_regime(pts[:2])


def test_saturation_bytes():
    p = HardwareProfile(alpha_us=1.0, beta_us_per_byte=1e6 / 900e9, gemm_tflops_fp16=2250)
    tau = CostModelCalibrator.saturation_bytes(p, 0.9)
    assert tau == pytest.approx(9 * 900e3, rel=1e-3)            # 9 * alpha / beta
    assert TileCostModel(p).comm_time_bytes(tau) == pytest.approx(10.0, rel=1e-3)


def test_measured_profile_reads_files(tmp_path):
    peaks = tmp_path / "peaks.json"
    peaks.write_text('{"bf16_tflops": 1628.4}')
    cal = tmp_path / "cal.json"
    cal.write_text('{"alpha_us": 2.0, "beta_us_per_byte": 1.4e-6, "min_comm_us": 3.0}')
    p = HardwareProfile.b200_measured(str(peaks), str(cal))
    assert p.gemm_tflops_fp16 == 1628.4 and p.alpha_us == 2.0 and p.min_comm_us == 3.0
    assert HardwareProfile.b200_measured("/nonexistent", "/nonexistent").bandwidth_gb_s == pytest.approx(900)


def test_calibration_file_sizes_the_tile_groups(tmp_path, monkeypatch):
    """tau_min of the calibration file in force decides how many tile rows form a TileGroup."""
    import json

    from tileccl_b200.ops import _fused, _tile_group_info
    from tileccl_b200.planning.cost_model import calibrated_tau_min_bytes

    monkeypatch.delenv("TILECCL_CALIBRATION", raising=False)
    shipped = calibrated_tau_min_bytes()
    assert 256 * 1024 <= shipped <= 2 * 1024 * 1024            # measured: a bit under one 4096-wide tile row
    assert _fused.default_group_m_tiles(64, 16) == 1            # gate shapes: one row per group
    assert _tile_group_info(8192, 4096)["group_m_tiles"] == 1
    coarse = tmp_path / "coarse.json"
    coarse.write_text(json.dumps({"alpha_us": 1.0, "beta_us_per_byte": 1e-6,
                                  "in_kernel": {"alpha_us": 4.0, "beta_us_per_byte": 1.5e-6,
                                                "tau_min_bytes": 8 << 20}}))
    monkeypatch.setenv("TILECCL_CALIBRATION", str(coarse))
    assert calibrated_tau_min_bytes() == 8 << 20
    info = _tile_group_info(8192, 4096)
    assert info["group_m_tiles"] == 8 and info["n_groups"] == 8 and info["calibration"] == str(coarse)
    assert _fused.default_group_m_tiles(4, 16) == 4             # never more rows than there are
    # without an in-kernel section the reference's constant applies
    plain = tmp_path / "plain.json"
    plain.write_text(json.dumps({"alpha_us": 1.0, "beta_us_per_byte": 1e-6}))
    monkeypatch.setenv("TILECCL_CALIBRATION", str(plain))
    assert calibrated_tau_min_bytes() == 262144
    # the in-kernel fit is what the cost model predicts with
    monkeypatch.setenv("TILECCL_CALIBRATION", str(coarse))
    assert HardwareProfile.b200_measured("/nonexistent").alpha_us == 4.0
