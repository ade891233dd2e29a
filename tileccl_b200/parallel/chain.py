"""All-gather -> GEMM chains: the left operand is sharded over ranks and gathered
by the GEMM kernel itself while it computes.

One launch per rank (``csrc/kernels/gemm_sm100.cu``): warp 3 of every CTA pushes
this rank's shard of the operand into every peer's gathered buffer and bumps
their arrival counters; the TMA producer starts with the tiles whose rows are
local and waits on the arrival counter of the owning rank before it touches
rows that come from a peer.  No separate all-gather kernel, no NCCL.

The reference's counterpart is its three-role chained kernel and the host
pipeline around it (tileccl/patterns/chained_ag_gemm_rs.py:201-425,
tileccl/ops.py:2378-2430).
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import fused_gemm as fg
from ..ops import _fused
from ..utils.config import current as _config


def _gate_state(ctx, name: str) -> dict:
    st = _fused.op_state(ctx, ("gate", name))
    if "gate" not in st:
        st["gate"] = ctx.workspace(f"gate:{name}", 8, dtype=torch.int32)
        st["entry"] = ctx.workspace(f"gate_entry:{name}", 8, dtype=torch.int32)
    return st


def rows_allgather_gemm(ctx, name: str, x_full: torch.Tensor, W: torch.Tensor,
                        out: torch.Tensor, *, epilogue: str = "none", b_is_nk: bool = False,
                        use_multimem: Optional[bool] = None) -> torch.Tensor:
    """``out = epilogue(X @ W)`` where ``X`` is the row-wise all-gather of the ranks' shards.

    ``x_full`` is ``[M, K]`` on the symmetric heap; rank ``r`` must have written
    its shard into rows ``[r * M/ws, (r + 1) * M/ws)`` of its own ``x_full``
    before the call.  After the call (stream order) ``x_full`` holds every rank's
    rows and ``out`` the product.  ``epilogue="silu_gate"`` expects ``W`` packed
    as alternating 128-column gate / up blocks and writes ``silu(gate) * up``.
    """
    ws, rank = ctx.world_size, ctx.rank
    M, K = x_full.shape
    Kw, N = (W.shape[1], W.shape[0]) if b_is_nk else (W.shape[0], W.shape[1])
    if K != Kw:
        raise ValueError(f"x_full is {tuple(x_full.shape)} but W is {tuple(W.shape)}")
    if M % ws:
        raise ValueError(f"rows {M} not divisible by world_size {ws}")
    if ws > 1 and not ctx.is_symmetric(x_full):
        raise ValueError("x_full must live on the symmetric heap")
    if not x_full.is_contiguous():
        raise ValueError("x_full must be contiguous")
    epi = {"none": fg.EPI_NONE, "silu_gate": fg.EPI_SILU_GATE}[epilogue]
    n_out = N // 2 if epi == fg.EPI_SILU_GATE else N
    if tuple(out.shape) != (M, n_out):
        raise ValueError(f"out must be {(M, n_out)}, got {tuple(out.shape)}")
    mloc = M // ws
    if ws > 1 and mloc % fg.BLOCK_M:
        raise ValueError(f"rows per rank ({mloc}) must be a multiple of {fg.BLOCK_M} so that no "
                         "tile mixes rows of two ranks")
    if use_multimem is None:
        # Default: unicast bulk copies through the kernel's bounce ring, destinations ordered
        # so that every consumer receives the shard it needs next (a multicast store delivers
        # all shards at the same slow pace, which stalls the GEMM after its own rows).
        # TILECCL_PUSH_MODE=multimem selects one multimem store per 16 bytes instead.
        use_multimem = (ws > 1 and ctx.heap.has_multicast and _config().nvls_allowed
                        and _config().push_mode_explicit
                        and _fused.default_push_mode(ctx) == fg.PUSH_MULTIMEM)
    key = ("ag_gemm", name, x_full.data_ptr(), W.data_ptr(), out.data_ptr(), M, N, K, x_full.dtype,
           epi, b_is_nk, use_multimem)
    st = _fused.op_state(ctx, key)
    gate = _gate_state(ctx, f"{name}:{M}x{K}") if ws > 1 else st
    if "plan" not in st:
        shard_bytes = mloc * K * x_full.element_size()
        region = x_full.data_ptr() + rank * shard_bytes
        spec = fg.FusedGemmSpec(
            mode=fg.MODE_GEMM, dtype=x_full.dtype, a_ptr=x_full.data_ptr(), a_rows=M,
            lda=x_full.stride(0), b_ptr=W.data_ptr(), b_cols=N, ldb=W.stride(0), k=K, sub_m=M,
            sub_n=N, out_ptrs=[out.data_ptr()], ldo=out.stride(0), out_rows=M, out_cols=n_out,
            b_kmajor=b_is_nk, epi_op=epi, rank=rank, world_size=ws,
            rot_m_tiles=(rank * mloc) // fg.BLOCK_M if ws > 1 else 0,
            status_ptr=_fused.status_block(ctx).data_ptr(),
            stats_ptr=_fused.stats_block(ctx).data_ptr(), wait_budget_ns=_fused.wait_budget_ns())
        if ws > 1:
            spec.heap_stride = ctx.heap.stride
            spec.a_gate = gate["gate"].data_ptr()
            spec.a_gate_rows_per_rank = mloc
            spec.entry_local = _fused.entry_ptr(ctx, gate)
            spec.ag_src = region
            spec.ag_dst = region
            spec.ag_bytes = shard_bytes
            spec.ag_mc_dst = ctx.heap.multicast_ptr(region) if use_multimem else 0
        st["plan"] = fg.FusedGemmPlan(spec)
    plan = st["plan"]
    if ws == 1:
        plan.launch()
        return out
    gate["epoch"] += 1
    target = gate["epoch"] * plan.push_grid * fg.AG_PUSH_WARPS
    if ctx.emulated:
        phases = [_fused._on_device(ctx, lambda: plan.launch(a_gate_target=target, tile_begin=0,
                                                             tile_end=0, ag_push=True)),
                  _fused._on_device(ctx, lambda: plan.launch(a_gate_target=target))]
    else:
        phases = [_fused._on_device(ctx, lambda: plan.launch(epoch=gate["epoch"],
                                                             a_gate_target=target, ag_push=True))]
    _fused.run_phases(ctx, ("ag_gemm", name, M, N, K, gate["epoch"]), phases)
    return out


def allgather_gemm(ctx, input_shard: torch.Tensor, W: torch.Tensor, output: torch.Tensor) -> torch.Tensor:
    """``output = cat(column shards over ranks, dim=1) @ W`` on every rank.

    The operand is sharded along K, so each rank multiplies its shard by the
    matching rows of ``W`` and the partial products are summed on every rank:
    ``sum_r shard_r @ W[r*k:(r+1)*k]``, which equals the product with the gathered
    operand.  Uses the fused reduce-scatter kernel followed by the tile all-gather
    (together an all-reduce of the partial products).
    """
    ws, rank = ctx.world_size, ctx.rank
    M, kc = input_shard.shape
    K, N = W.shape
    if kc * ws != K:
        raise ValueError(f"input_shard has {kc} columns, W has {K} rows, world_size is {ws}")
    w_rows = W[rank * kc:(rank + 1) * kc]
    if ws == 1:
        fg.gemm(input_shard, w_rows, output)
        return output
    if M % ws:
        raise ValueError(f"M={M} must be divisible by world_size={ws}")
    if not ctx.is_symmetric(output):
        raise ValueError("output must live on the symmetric heap")
    mloc = M // ws
    local = output[rank * mloc:(rank + 1) * mloc]
    _fused.reduce_scatter(ctx, "ag_gemm_rs", input_shard, w_rows, local, split_axis=0)
    from ..primitives import collectives

    # Gather the reduced row blocks in place: every rank's block already sits at its own
    # position in `output`, so the block itself is the all-gather source.
    collectives.allgather(local.reshape(-1), output.view(-1), ctx.heap)
    return output
