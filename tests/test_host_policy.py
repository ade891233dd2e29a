"""Host-side policy objects: contracts, pattern selection, feature gates, support matrix,
profiling helpers, timeline (CPU only)."""

import json
import types

import pytest
import torch

import tileccl_b200
from tileccl_b200.patterns import (PATTERN_CLASSES, auto_select, resolve_dual_role_scheduler,
                                   resolve_pattern_execution, resolve_stage_role_scheduler,
                                   resolve_tile_collective_execution,
                                   resolve_tile_collective_runtime)
from tileccl_b200.patterns.auto_select import HardwareInfo, estimate_pattern_times
from tileccl_b200.planning.runtime import TimelineEvent, TimelineRecorder, events_from_device_trace
from tileccl_b200.utils import feature_gates as fgates
from tileccl_b200.utils.profiling import (CommHeatmap, OverlapTimeline, bandwidth_to_normalized,
                                          format_benchmark_table)


def _t(r, c):
    return torch.empty(r, c)


def test_pattern_contract_full_full_and_shard_shard():
    spec = resolve_pattern_execution(_t(64, 32), _t(32, 128), _t(64, 128), rank=1, world_size=4)
    assert (spec.M, spec.K, spec.full_N, spec.local_N) == (64, 32, 128, 32)
    assert (spec.scatter_src_col_offset, spec.scatter_cols, spec.scatter_dst_leading_dim,
            spec.scatter_dst_col_offset) == (32, 32, 128, 32)
    assert spec.rhs_layout == spec.output_layout == "full"
    sh = resolve_pattern_execution(_t(64, 32), _t(32, 32), _t(64, 32), rank=1, world_size=4,
                                   full_N=128, b_layout="shard", c_layout="shard")
    assert sh.scatter_dst_col_offset == 0 and sh.scatter_dst_leading_dim == 32
    assert json.dumps(sh.to_dict())


@pytest.mark.parametrize("kw", [
    dict(b_layout="full"),                                   # layouts must come together
    dict(b_layout="full", c_layout="shard"),                 # mixed layouts are not a pattern contract
    dict(b_layout="diag", c_layout="full"),
    dict(full_N=130),                                        # not divisible by world size
])
def test_pattern_contract_rejections(kw):
    with pytest.raises(ValueError):
        resolve_pattern_execution(_t(64, 32), _t(32, 128), _t(64, 128), rank=0, world_size=4, **kw)


def test_pattern_contract_shape_errors():
    with pytest.raises(ValueError):
        resolve_pattern_execution(_t(64, 32), _t(31, 128), _t(64, 128), rank=0, world_size=1)
    with pytest.raises(ValueError):
        resolve_pattern_execution(_t(64, 32), _t(32, 128), _t(63, 128), rank=0, world_size=1)
    with pytest.raises(ValueError):
        resolve_pattern_execution(torch.empty(4), _t(32, 128), _t(64, 128), rank=0, world_size=1)


def test_auto_select_rules():
    assert auto_select("gemm_allscatter", 128, 4096, 4096, world_size=8) is PATTERN_CLASSES["bulk_sync"]
    cls = auto_select("gemm_allscatter", 8192, 4096, 4096, world_size=8)
    assert cls in PATTERN_CLASSES.values() and cls is not PATTERN_CLASSES["bulk_sync"]
    with pytest.raises(ValueError):
        auto_select("gemm_everything", 1, 1, 1)
    ctx = types.SimpleNamespace(rank=0, world_size=8, topology=None)
    inst = auto_select("gemm_allscatter", 8192, 4096, 4096, world_size=8, ctx=ctx)
    assert isinstance(inst, tuple(PATTERN_CLASSES.values())) and inst.ctx is ctx
    times = estimate_pattern_times(8192, 4096, 2048, 8, HardwareInfo())
    assert times["bulk_sync"] > times["wg_specialized"] > 0


def test_role_schedulers():
    d = resolve_dual_role_scheduler(148)
    assert d.comm_sms == 0 and d.compute_sms == 148 and d.comm_warps_per_cta == 4
    d2 = resolve_dual_role_scheduler(148, comm_sm_fraction=0.2)
    assert d2.comm_sms == 29 and d2.compute_sms + d2.comm_sms == 148
    assert resolve_dual_role_scheduler(148, compute_sms=100, comm_sms=20).policy == "explicit"
    with pytest.raises(ValueError):
        resolve_dual_role_scheduler(148, compute_sms=140, comm_sms=20)
    s = resolve_stage_role_scheduler(148)
    assert s.gather_sms == s.scatter_sms == 0 and s.compute_sms == 148
    ex = resolve_tile_collective_execution("gemm_reducescatter", total_sms=148, rows=2048, world_size=8)
    assert ex.slot_count == 16 and ex.runtime.wait_mode == "wait_ge"
    assert len(ex.slot_workspace_names(0)) == 8 and json.dumps(ex.to_dict())
    with pytest.raises(ValueError):
        resolve_tile_collective_runtime("nope")


def test_feature_gates(monkeypatch):
    surface = fgates.multiprocess_device_validated_public_surface()
    assert surface["world_sizes"] == [1, 2, 4, 8] and "vmm_fd" in surface["transports"]
    assert fgates.multiprocess_device_collectives_enabled()
    assert fgates.multiprocess_device_remote_access_runtime_supported(transport_strategy="vmm_fd", world_size=8)
    assert not fgates.multiprocess_device_remote_access_runtime_supported(transport_strategy="vmm_fd", world_size=3)
    assert "world_size 3" in fgates.multiprocess_device_remote_access_detail(
        transport_strategy="vmm_fd", world_size=3)
    monkeypatch.delenv(fgates.FORCE_MULTIPROCESS_TRANSPORT_ENV, raising=False)
    assert fgates.forced_multiprocess_transport() is None
    monkeypatch.setenv(fgates.FORCE_MULTIPROCESS_TRANSPORT_ENV, "ctypes_ipc")
    assert fgates.forced_multiprocess_transport() == "vmm_fd"
    monkeypatch.setenv(fgates.FORCE_MULTIPROCESS_TRANSPORT_ENV, "carrier_pigeon")
    with pytest.raises(ValueError):
        fgates.forced_multiprocess_transport()


def test_support_matrix_without_gpu_is_consistent():
    ctx = tileccl_b200.init(rank=0, world_size=1, force_backend=True)
    m = ctx.support_matrix()
    d = m.to_dict()
    assert d["context"]["world_size"] == 1 and not d["context"]["has_heap"]
    assert sum(m.summary().values()) == sum(len(d[k]) for k in
                                            ("ops", "contracts", "execution_paths", "collectives", "memory"))
    assert d["contracts"]["gemm_allscatter.shard/full"]["state"] == "unsupported"
    assert ctx.runtime_metadata()["has_heap"] is False
    with pytest.raises(RuntimeError):
        ctx.require_heap()


def test_profiling_helpers(tmp_path):
    tl = OverlapTimeline()
    tl.record("compute", "gemm", 0.0, 10.0)
    tl.record("comm", "push", 4.0, 12.0)
    o = tl.compute_overlap()
    assert o["overlap_ms"] == pytest.approx(6.0) and o["overlap_ratio"] == pytest.approx(0.75)
    assert o["wall_ms"] == pytest.approx(12.0)
    with pytest.raises(ValueError):
        tl.record("comm", "bad", 2.0, 1.0)
    hm = CommHeatmap(2)
    hm.record(0, 1, 100)
    hm.record(1, 0, 50)
    assert hm.get_traffic_matrix() == [[0, 100], [50, 0]] and hm.balance()["max_min_send_ratio"] == 2.0
    with pytest.raises(ValueError):
        hm.record(0, 2, 1)
    bw = bandwidth_to_normalized(900e9 * 1e-3, 1.0, 900.0)
    assert bw["gbps"] == pytest.approx(900.0) and bw["fraction_of_peak"] == pytest.approx(1.0)
    assert "name" in format_benchmark_table([{"name": "a", "ms": 1.0}])
    tl.export_json(tmp_path / "t.json")
    hm.export_json(tmp_path / "h.json")


def test_timeline_schema_roundtrip(tmp_path):
    rec = TimelineRecorder(benchmark="gate1", path_name="fused", metadata={"ws": 2})
    rec.record_span(name="gemm", lane="rank0/compute", start_ms=0.0, end_ms=1.5, category="compute", rank=0)
    rec.record_marker(name="group0", lane="rank0/signal", at_ms=0.4, rank=0)
    rec.extend(events_from_device_trace([0, 2_000_000, 1_000_000], lane="rank1/tiles", rank=1))
    payload = rec.to_payload()
    assert payload["schema"] == "tileccl.timeline.v1"
    assert payload["authenticity_checks"] == {"event_count": 4, "all_events_have_source": True,
                                              "all_events_have_nonnegative_duration": True}
    assert payload["lane_order"] == ["rank0/compute", "rank0/signal", "rank1/tiles"]
    rec.write_json(tmp_path / "timeline.json")
    again = TimelineRecorder.from_payload(json.loads((tmp_path / "timeline.json").read_text()))
    assert [e.name for e in again.events] == [e.name for e in rec.events]
    with pytest.raises(ValueError):
        TimelineEvent("x", "l", 2.0, 1.0)
    with pytest.raises(ValueError):
        TimelineEvent("x", "l", 0.0, 1.0, source="")
    rec.render_svg(tmp_path / "timeline.svg")
    svg = (tmp_path / "timeline.svg").read_text()
    assert svg.startswith("<svg") and svg.count("<rect") >= 1 + 3 + 1      # background, lanes, one span
    assert "rank1/tiles" in svg and "time (ms)" in svg


def test_only_the_config_module_reads_library_environment_variables():
    """Every TILECCL_* / TileCCL_* switch is read in utils/config.py and nowhere else."""
    import pathlib
    import re

    import tileccl_b200

    root = pathlib.Path(tileccl_b200.__file__).parent
    pat = re.compile(r"(environ|getenv)[^\n]*(TILECCL_|TileCCL_)")
    offenders = []
    for path in list(root.rglob("*.py")) + list(root.rglob("*.cc")) + list(root.rglob("*.cu")):
        if path.name == "config.py" and path.parent.name == "utils":
            continue
        for i, line in enumerate(path.read_text().splitlines(), 1):
            if pat.search(line):
                offenders.append(f"{path.relative_to(root)}:{i}")
    assert not offenders, offenders


def test_runtime_config_snapshot_of_the_environment():
    from tileccl_b200.utils import RuntimeConfig

    cfg = RuntimeConfig.from_env({})
    assert cfg.push_mode == "tma" and cfg.tuning == 1 and cfg.gemm_cta_pairs
    assert cfg.rs_own_lag is None and cfg.wait_budget_us is None and not cfg.disable_nvls
    cfg = RuntimeConfig.from_env({"TILECCL_PUSH_MODE": "Stores", "TILECCL_GEMM_2SM": "0",
                                  "TILECCL_RS_OWN_LAG": "8", "TILECCL_WAIT_BUDGET_US": "2500",
                                  "TILECCL_FORCE_NVLS": "1",
                                  "TileCCL_FORCE_MULTIPROCESS_TRANSPORT": "vmm_fd"})
    assert cfg.push_mode == "stores" and not cfg.gemm_cta_pairs and cfg.rs_own_lag == 8
    assert cfg.wait_budget_us == 2500.0 and cfg.force_nvls
    assert cfg.force_multiprocess_transport == "vmm_fd"
    assert set(cfg.to_dict()) >= {"push_mode", "tuning", "calibration", "native_lib"}
    import pytest

    with pytest.raises(ValueError):
        RuntimeConfig.from_env({"TILECCL_PUSH_MODE": "carrier-pigeon"})
    with pytest.raises(Exception):
        cfg.push_mode = "tma"            # frozen


def test_nvlink_facts_from_a_fake_nvml():
    """Link count, generation and rate come from NVML queries (here: a fake of the API)."""
    from types import SimpleNamespace as NS

    from tileccl_b200.backends.nvml import nvlink_facts

    class FakeNvml:
        NVML_FI_DEV_NVLINK_SPEED_MBPS_COMMON = 90
        calls = []

        def nvmlDeviceGetHandleByIndex(self, i):
            return ("h", i)

        def nvmlDeviceGetNvLinkState(self, h, link):
            self.calls.append(link)
            if link >= 18:
                raise RuntimeError("invalid link")
            return 1

        def nvmlDeviceGetNvLinkVersion(self, h, link):
            return 7

        def nvmlDeviceGetFieldValues(self, h, fields):
            return [NS(nvmlReturn=0, value=NS(uiVal=50000))]

    f = nvlink_facts(0, nvml=FakeNvml())
    assert (f.links_active, f.generation, f.source) == (18, 5, "nvml")
    assert abs(f.gbps_per_direction - 900.0) < 1e-6

    class NoSpeed(FakeNvml):
        def nvmlDeviceGetFieldValues(self, h, fields):
            raise RuntimeError("not supported")

        def nvmlDeviceGetNvLinkState(self, h, link):
            return 1 if link < 12 else 0

    g = nvlink_facts(0, nvml=NoSpeed())
    assert (g.links_active, g.source) == (12, "nvml-partial") and g.gbps_per_direction == 600.0

    class Down(FakeNvml):
        def nvmlDeviceGetNvLinkState(self, h, link):
            return 0

    assert nvlink_facts(0, nvml=Down()) is None


def test_pattern_options_select_the_launch_shape_or_are_rejected():
    """COMM_SMS / COMPUTE_SMS are honoured by the two-kernel patterns and rejected where the
    communication role is a set of warps inside every compute CTA."""
    from types import SimpleNamespace as NS

    from tileccl_b200.patterns import (BulkSyncPattern, FusedSequentialPattern,
                                       ProducerConsumerPattern, WGSpecializedPattern)

    ctx = NS(rank=0, world_size=2, backend=None)
    pc = ProducerConsumerPattern(ctx, COMPUTE_SMS=120, COMM_SMS=24)
    shape = pc.launch_shape()
    assert (shape.compute_sms, shape.comm_sms, shape.policy) == (120, 24, "two_kernels")
    assert BulkSyncPattern(ctx).launch_shape().comm_sms == 32            # default push grid
    wg = WGSpecializedPattern(ctx, COMPUTE_SMS=96, BLOCK_M=128, BLOCK_N=128, BLOCK_K=64)
    assert wg.launch_shape().compute_sms == 96 and wg.launch_shape().comm_sms == 0
    with pytest.raises(ValueError, match="COMM_SMS"):
        WGSpecializedPattern(ctx, COMM_SMS=16)
    with pytest.raises(ValueError, match="COMM_SMS"):
        FusedSequentialPattern(ctx, COMPUTE_SMS=100, COMM_SMS=48)
    with pytest.raises(ValueError, match="128 x 256 x 64"):
        WGSpecializedPattern(ctx, BLOCK_M=64, BLOCK_N=64, BLOCK_K=32)
    with pytest.raises(TypeError):
        WGSpecializedPattern(ctx, FANCY=1)


def test_runtime_config_covers_the_measured_choices():
    from tileccl_b200.utils import RuntimeConfig

    cfg = RuntimeConfig.from_env({})
    assert not cfg.dynamic_tiles and cfg.call_stats and cfg.rs_cta_pairs is None
    assert cfg.ll_max_bytes == 1 << 20 and cfg.stream_run_shares is None and cfg.stream_copy_streams == 1
    cfg = RuntimeConfig.from_env({"TILECCL_DYNAMIC_TILES": "1", "TILECCL_STATS": "0",
                                  "TILECCL_RS_CTA_PAIRS": "1", "TILECCL_LL_MAX_BYTES": "4096",
                                  "TILECCL_STREAM_SHARES": "0.85,0.15"})
    assert cfg.dynamic_tiles and not cfg.call_stats and cfg.rs_cta_pairs is True
    assert cfg.ll_max_bytes == 4096 and cfg.stream_run_shares == (0.85, 0.15)
    assert cfg.wait_budget_ns == 0 and RuntimeConfig.from_env({"TILECCL_WAIT_BUDGET_US": "3"}).wait_budget_ns == 3000


def test_op_state_table_is_bounded_and_keeps_signal_blocks():
    """Plan entries are evicted oldest-first beyond the bound; signal blocks (epochs) never."""
    from types import SimpleNamespace

    from tileccl_b200.ops import _fused

    closed = []

    class FakePlan:
        def __init__(self, i):
            self.i = i

        def close(self):
            closed.append(self.i)

    ctx = SimpleNamespace(_state={})
    sig = _fused.op_state(ctx, ("sig", "gemm_allgather"))
    sig["epoch"] = 7
    for i in range(_fused.MAX_OP_STATES + 5):
        _fused.op_state(ctx, ("push_all", "x", i))["plan"] = FakePlan(i)
    table = ctx._state["ops"]
    assert len(table) <= _fused.MAX_OP_STATES
    assert table[("sig", "gemm_allgather")] is sig and sig["epoch"] == 7
    assert closed == list(range(len(closed))) and len(closed) >= 5
    # the same key gives the same state back
    last = ("push_all", "x", _fused.MAX_OP_STATES + 4)
    assert _fused.op_state(ctx, last) is table[last]


def test_relay_broadcast_policy_and_piece_size(monkeypatch):
    from types import SimpleNamespace

    from tileccl_b200.primitives import collectives as coll

    for nbytes in (8 << 20, (8 << 20) + 16, 256 << 20, 1 << 30, 3 << 30):
        for bulk in (False, True):
            piece = coll.relay_piece_bytes(nbytes, bulk=bulk)
            assert piece % 8192 == 0 and piece >= coll.RELAY_MIN_PIECE
            assert -(-nbytes // piece) <= coll.RELAY_MAX_PIECES
    assert coll.relay_piece_bytes(256 << 20) == 128 << 10               # about 2048 pieces
    assert coll.relay_piece_bytes(8 << 20, bulk=True) == 16 << 10       # about 1024, at least 16 KiB
    assert coll.relay_piece_bytes(256 << 20, bulk=True) == 64 << 10     # capped at the largest piece
    assert coll.relay_piece_bytes(3 << 30, bulk=True) == 192 << 10      # stays within 16384 pieces
    heap3, heap2 = SimpleNamespace(world_size=3), SimpleNamespace(world_size=2)
    monkeypatch.delenv("TILECCL_BCAST_RELAY_MIN_BYTES", raising=False)
    assert coll._relay_ok(heap3, 256 << 20, 4096) and not coll._relay_ok(heap3, 128 << 20, 4096)
    monkeypatch.setenv("TILECCL_BCAST_RELAY_MIN_BYTES", str(64 << 20))
    assert coll._relay_ok(heap3, 64 << 20, 4096)
    assert not coll._relay_ok(heap3, (64 << 20) - 16, 4096)     # below the threshold
    assert not coll._relay_ok(heap2, 256 << 20, 4096)           # one relay only: nothing to gain
    assert not coll._relay_ok(heap3, (64 << 20) + 8, 4096)      # not a multiple of 16
    monkeypatch.setenv("TILECCL_BCAST_RELAY_MIN_BYTES", "0")
    assert not coll._relay_ok(heap3, 256 << 20, 4096)           # switched off


def test_cached_config_follows_the_environment(monkeypatch):
    """current() re-parses only when one of the variables it depends on changed, and the list
    of those variables covers every name from_env() reads."""
    import re

    from tileccl_b200.utils import config

    src = open(config.__file__).read()
    read = set(re.findall(r'"(T[iI][lL][eE]CCL_[A-Za-z_0-9]+)"', src))
    assert read == set(config.ENV_NAMES)
    monkeypatch.delenv("TILECCL_LL_MAX_BYTES", raising=False)
    a = config.current()
    assert config.current() is a                       # unchanged environment: same snapshot
    monkeypatch.setenv("TILECCL_LL_MAX_BYTES", "4096")
    b = config.current()
    assert b is not a and b.ll_max_bytes == 4096
    monkeypatch.delenv("TILECCL_LL_MAX_BYTES")
    assert config.current().ll_max_bytes == 1 << 20


def test_repeat_collective_calls_reuse_the_resolved_launch(monkeypatch):
    """Second call on the same buffers: no validation, no policy, next epoch, same arguments;
    a changed configuration or other buffers take the full path again."""
    from types import SimpleNamespace

    import torch

    from tileccl_b200 import _native
    from tileccl_b200.primitives import collectives as coll

    calls = []

    def fake_launch(*args):
        calls.append(args)
        return 0

    monkeypatch.setattr(_native, "load", lambda *a, **k: SimpleNamespace(
        tccl_collective_launch=fake_launch, tccl_collective_ll_launch=fake_launch))
    monkeypatch.setattr(coll, "_stream_ptr", lambda idx: 0)
    monkeypatch.delenv("TILECCL_DEBUG", raising=False)
    monkeypatch.delenv("TILECCL_DISABLE_NVLS", raising=False)
    monkeypatch.setenv("TILECCL_LL_MAX_BYTES", "0")           # the three-phase kernel's launcher
    dev = torch.device("cpu")
    monkeypatch.setitem(coll._SM_COUNT, dev, 148)
    heap = SimpleNamespace(rank=1, world_size=4, emulated=False, local_group=None, device=dev,
                           multicast_base=0, local_base=1 << 30, stride=1 << 28, has_multicast=False,
                           _state={}, owns_tensor=lambda t: True,
                           allocate_signal_buffer=lambda n: torch.zeros(n, dtype=torch.int32))
    validated = []
    real_validate = coll._validate
    monkeypatch.setattr(coll, "_validate", lambda name, t, h: (validated.append(name),
                                                               real_validate(name, t, h)))
    src = torch.zeros(4 * 65536, dtype=torch.float32)
    out = torch.zeros(65536, dtype=torch.float32)
    coll.reduce_scatter(src, out, heap)
    assert len(calls) == 1 and len(validated) == 2
    coll.reduce_scatter(src, out, heap)
    coll.reduce_scatter(src, out, heap)
    assert len(calls) == 3 and len(validated) == 2              # repeat calls skipped validation
    epochs = [c[8] for c in calls]
    assert epochs == [1, 2, 3]
    assert all(c[:8] == calls[0][:8] and c[9:] == calls[0][9:] for c in calls)
    other = torch.zeros(65536, dtype=torch.float32)
    coll.reduce_scatter(src, other, heap)                       # other buffers: full path
    assert len(validated) == 4 and calls[-1][8] == 4            # same kind, same counter block
    monkeypatch.setenv("TILECCL_WAIT_BUDGET_US", "5000")
    coll.reduce_scatter(src, out, heap)                         # new configuration: full path
    assert len(validated) == 6 and calls[-1][-2] == 5_000_000 and calls[-1][8] == 5
    monkeypatch.setenv("TILECCL_DEBUG", "1")                    # debug mode never remembers
    assert coll._config().debug


def test_low_latency_staging_classes():
    from tileccl_b200.primitives import collectives as coll

    assert coll.ll_slot_bytes(8) == coll.LL_MIN_SLOT_BYTES == 128 * 1024
    assert coll.ll_slot_bytes(65536) == 128 * 1024
    assert coll.ll_slot_bytes(65544) == 256 * 1024
    assert coll.ll_slot_bytes(1 << 20) == 2 << 20
    for n in (8, 4096, 65536, 100_000, 1 << 20):
        assert coll.ll_slot_bytes(n) >= 2 * n


def test_relay_piece_assignment_covers_every_piece_once():
    """Mirror of the device-side assignment (relay_rank_of / the workers' strides in
    csrc/device/tile_collectives.cuh and broadcast_relay_bulk_kernel): the root's workers and
    each relay's workers visit disjoint pieces, and together every piece exactly once."""
    def relay_rank_of(piece, root, ws):
        k = piece % (ws - 1)
        return k if k < root else k + 1

    for ws, root, n_pieces, root_workers, relay_workers in ((3, 0, 17, 4, 5), (4, 2, 1024, 148, 592),
                                                            (8, 7, 1000, 148, 592), (8, 3, 5, 148, 592)):
        sent = []
        for worker in range(root_workers):
            sent += list(range(worker, n_pieces, root_workers))
        assert sorted(sent) == list(range(n_pieces))
        forwarded = []
        for rank in range(ws):
            if rank == root:
                continue
            mine = rank if rank < root else rank - 1
            for worker in range(relay_workers):
                for piece in range(worker * (ws - 1) + mine, n_pieces, relay_workers * (ws - 1)):
                    assert relay_rank_of(piece, root, ws) == rank
                    forwarded.append(piece)
        assert sorted(forwarded) == list(range(n_pieces))


def test_nvls_policy_by_collective_and_size(monkeypatch):
    from types import SimpleNamespace

    from tileccl_b200.primitives import collectives as coll

    for name in ("TILECCL_DISABLE_NVLS", "TILECCL_FORCE_NVLS"):
        monkeypatch.delenv(name, raising=False)
    h8 = SimpleNamespace(world_size=8, has_multicast=True)
    h2 = SimpleNamespace(world_size=2, has_multicast=True)
    assert not coll._use_multimem(h2, 1 << 20, "allgather")             # two ranks: plain stores
    assert coll._use_multimem(h8, 1 << 20, "allgather")                  # 8 MiB in total
    assert not coll._use_multimem(h8, 2 << 20, "allgather")              # 16 MiB in total
    assert coll._use_multimem(h8, 8 << 20, "reduce_scatter")             # 64 MiB in total
    assert not coll._use_multimem(h8, 16 << 20, "reduce_scatter")        # 128 MiB in total
    assert coll._use_multimem(h8, 1 << 30)                               # all-reduce, broadcast
    assert not coll._use_multimem(h8, 1000 * 16 + 8, "allgather")        # not a multiple of 16
    monkeypatch.setenv("TILECCL_FORCE_NVLS", "1")
    assert coll._use_multimem(h8, 16 << 20, "reduce_scatter") and coll._use_multimem(h2, 4096)
    monkeypatch.setenv("TILECCL_DISABLE_NVLS", "1")
    assert not coll._use_multimem(h8, 4096, "allgather")
