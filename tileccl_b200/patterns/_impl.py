"""How each pattern maps onto the sm_100a kernels (shared by the four pattern modules)."""

from __future__ import annotations

from ..ops import _fused


def _cols(spec):
    return spec.scatter_dst_col_offset, spec.scatter_dst_col_offset + spec.scatter_cols


def run_fused(ctx, name: str, A, B, C, spec, push_mode: int) -> None:
    """Single persistent kernel: the epilogue warps push each finished tile."""
    if spec.output_layout == "full":
        lo, hi = _cols(spec)
        _fused.all_scatter(ctx, name, A, B, C, col_begin=lo, col_end=hi, push_mode=push_mode)
    else:
        # shard/shard: every rank writes its shard over the peers' shard buffers
        _fused.push_all(ctx, name + ":shard", A, B, C, region_row0=0, region_col0=0,
                        push_mode=push_mode)


def run_two_kernel(ctx, name: str, A, B, C, spec, overlapped: bool) -> None:
    """GEMM kernel + region-push kernel."""
    lo, hi = _cols(spec) if spec.output_layout == "full" else (0, spec.local_N)
    _fused.gemm_then_push(ctx, name, A, B, C, col_begin=lo, col_end=hi, overlapped=overlapped)


def pick_push_mode(ctx, preferred: int) -> int:
    """An explicit TILECCL_PUSH_MODE wins over the pattern's own choice."""
    from ..utils.config import current

    if current().push_mode_explicit:
        return _fused.default_push_mode(ctx)
    return preferred
