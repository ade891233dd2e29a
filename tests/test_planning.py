"""TileGroup planner, collective specs, transport / role plans (CPU only)."""

import pytest
import torch

from tileccl_b200.planning import (CollectiveKind, all_gather_spec, build_group_table,
                                   build_p2p_transport_plan, build_tile_group_plan,
                                   build_tile_groups, build_wg_plan, plan_for_fused_kernel,
                                   reduce_scatter_spec, split_groups_at_row_boundaries,
                                   split_groups_at_row_shards)


def test_readme_snippet_values():
    spec = reduce_scatter_spec(world_size=2)
    plan = build_tile_group_plan(8192, 4096, 128 * 128 * 2)
    transport = build_p2p_transport_plan(comm_mode="push", copy_elems=16384)
    assert spec.kind is CollectiveKind.REDUCE_SCATTER
    assert plan.n_groups == 8
    assert transport.push_mode is True
    assert transport.copy_qwords == 4096


def test_plan_geometry_8192x4096():
    plan = build_tile_group_plan(8192, 4096, 32768)
    assert plan.groups == [(i * 1024, (i + 1) * 1024, 256) for i in range(8)]
    assert plan.p0_min_tiles == 8 and plan.max_rb == 8 and plan.max_cb == 32
    assert plan.max_group_elems == 4_194_304
    assert plan.group_table.dtype == torch.int32 and plan.group_table.shape == (2048,)
    assert torch.equal(plan.group_table, (torch.arange(2048) // 256).to(torch.int32))
    assert plan.row_starts()[0] == 0 and plan.row_ends()[-1] == 8192
    assert sum(plan.tile_counts()) == 64 * 32
    assert plan.min_group_tiles == plan.max_group_tiles == 256 and plan.avg_group_tiles == 256


def test_reduce_scatter_ownership():
    spec = reduce_scatter_spec(world_size=2)
    assert spec.row_split_boundaries(8192) == [4096]
    assert spec.owner_for_row(5000, 8192) == 1
    plan = build_tile_group_plan(8192, 4096, 32768, row_split_boundaries=spec.row_split_boundaries(8192))
    assert plan.n_groups == 8
    spec.validate_tile_groups(8192, plan.groups)
    spec8 = reduce_scatter_spec(world_size=8)
    plan8 = build_tile_group_plan(16384, 4096, 32768,
                                  row_split_boundaries=spec8.row_split_boundaries(16384))
    assert plan8.n_groups == 16 and all(e - s == 1024 for s, e, _ in plan8.groups)
    with pytest.raises(ValueError):
        spec.validate_tile_groups(8192, [(0, 8192, 1)])
    with pytest.raises(ValueError):
        spec.shard_rows(8191)
    assert all_gather_spec(world_size=4).row_split_boundaries(4096) == []
    with pytest.raises(ValueError):
        all_gather_spec().owner_for_row(0, 128)


def test_tail_merge_and_max_groups():
    # 5 tile rows, waves of 2 -> [2, 2, 1]; the ragged wave joins the last full group
    groups = build_tile_groups(5 * 128, 128, 1, group_m=2, tau_min_bytes=1, target_group_tiles=2)
    assert groups == [(0, 256, 2), (256, 640, 3)]
    merged = build_tile_groups(64 * 128, 128, 1, group_m=1, tau_min_bytes=1, max_groups=4)
    assert len(merged) == 4 and merged[0] == (0, 16 * 128, 16) and merged[-1][1] == 64 * 128
    one = build_tile_groups(100, 100, 1, tau_min_bytes=10 ** 9)   # never reaches the minimum
    assert one == [(0, 100, 1)]


def test_split_helpers_and_table_swizzle():
    groups = [(0, 512, 8), (512, 1024, 8)]
    cut = split_groups_at_row_boundaries(1024, 256, groups, [256, 700])
    assert [(s, e) for s, e, _ in cut] == [(0, 256), (256, 512), (512, 700), (700, 1024)]
    shards = split_groups_at_row_shards(1024, 256, groups, num_shards=4)
    assert [(s, e) for s, e, _ in shards] == [(0, 256), (256, 512), (512, 768), (768, 1024)]
    with pytest.raises(ValueError):
        split_groups_at_row_shards(1000, 256, groups, num_shards=3)
    # 4 tile rows x 2 tile cols, waves of 2 rows: ids walk down the rows inside a wave
    table = build_group_table(512, 256, [(0, 128, 2), (128, 512, 6)], group_m=2)
    assert table.tolist() == [0, 1, 0, 1, 1, 1, 1, 1]


@pytest.mark.parametrize("bad", [dict(M=0), dict(N=0), dict(tile_bytes=0), dict(block_m=0),
                                 dict(max_groups=0), dict(group_m=0)])
def test_planner_rejects_bad_arguments(bad):
    kw = dict(M=1024, N=1024, tile_bytes=32768)
    kw.update(bad)
    M, N, tb = kw.pop("M"), kw.pop("N"), kw.pop("tile_bytes")
    with pytest.raises(ValueError):
        build_tile_group_plan(M, N, tb, **kw)


def test_transport_and_wg_plans():
    t = build_p2p_transport_plan(comm_mode="push", copy_elems=16384)
    wg = t.build_wg_plan(total_sms=132, num_comm_wgs=16, max_group_elems=4194304)
    assert wg.num_comp_wgs == 116 and wg.grid == (132,) and wg.copy_tasks_per_group == 256
    assert wg.reduce_tasks_per_group == 0 and wg.tasks_per_group == 256
    pull = build_p2p_transport_plan(comm_mode="pull", copy_elems=1024, reduce_elems=512)
    assert pull.push_mode is False
    assert pull.build_wg_plan(total_sms=148, num_comm_wgs=0, max_group_elems=4096).tasks_per_group == 8
    for kw in (dict(comm_mode="sideways", copy_elems=4), dict(comm_mode="push", copy_elems=0),
               dict(comm_mode="push", copy_elems=4, reduce_elems=0)):
        with pytest.raises(ValueError):
            build_p2p_transport_plan(**kw)
    for kw in (dict(total_sms=0, num_comm_wgs=0), dict(total_sms=8, num_comm_wgs=8),
               dict(total_sms=8, num_comm_wgs=1, copy_elems=6)):
        base = dict(total_sms=8, num_comm_wgs=1, max_group_elems=64, copy_elems=16)
        base.update(kw)
        with pytest.raises(ValueError):
            build_wg_plan(**base)


def test_fused_kernel_plan():
    info = plan_for_fused_kernel(2048, 4096)
    assert info["group_m_tiles"] == 1 and info["n_groups"] == 16
    big = plan_for_fused_kernel(128 * 200, 4096)
    assert big["n_groups"] <= 64 and big["group_m_tiles"] == 4
