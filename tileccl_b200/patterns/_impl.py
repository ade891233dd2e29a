"""How each pattern maps onto the sm_100a kernels (shared by the four pattern modules)."""

from __future__ import annotations

from ..ops import _fused


def _cols(spec):
    return spec.scatter_dst_col_offset, spec.scatter_dst_col_offset + spec.scatter_cols


def run_fused(ctx, name: str, A, B, C, spec, push_mode: int, shape=None) -> None:
    """Single persistent kernel: the epilogue warps push each finished tile.  ``shape``
    (a DualRoleScheduler): its ``compute_sms`` is the grid when it is not the whole device."""
    grid = 0
    if shape is not None and shape.compute_sms < shape.total_sms:
        grid = shape.compute_sms
    if spec.output_layout == "full":
        lo, hi = _cols(spec)
        _fused.all_scatter(ctx, name, A, B, C, col_begin=lo, col_end=hi, push_mode=push_mode,
                           grid=grid)
    else:
        # shard/shard: every rank writes its shard over the peers' shard buffers
        _fused.push_all(ctx, name + ":shard", A, B, C, region_row0=0, region_col0=0,
                        push_mode=push_mode)


def run_two_kernel(ctx, name: str, A, B, C, spec, overlapped: bool, shape=None) -> None:
    """GEMM kernel + region-push kernel, on ``shape.compute_sms`` and ``shape.comm_sms`` CTAs."""
    lo, hi = _cols(spec) if spec.output_layout == "full" else (0, spec.local_N)
    gemm_grid = push_grid = 0
    if shape is not None:
        gemm_grid = shape.compute_sms if shape.compute_sms < shape.total_sms else 0
        push_grid = shape.comm_sms
    _fused.gemm_then_push(ctx, name, A, B, C, col_begin=lo, col_end=hi, overlapped=overlapped,
                          gemm_grid=gemm_grid, push_grid=push_grid)


def pick_push_mode(ctx, preferred: int) -> int:
    """An explicit TILECCL_PUSH_MODE wins over the pattern's own choice."""
    from ..utils.config import current

    if current().push_mode_explicit:
        return _fused.default_push_mode(ctx)
    return preferred
