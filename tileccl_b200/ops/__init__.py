"""High-level operators: fused GEMM + collective ops, plain collectives, and
their plan objects.

Signatures follow the reference's ``tileccl.ops`` (tileccl/ops.py:702-1257,
2315-2375).  Every op resolves its tensors into a *contract* (pure shape/layout
facts), wraps it in a frozen *plan* with ``execute`` / ``validate_tensors`` /
``to_dict``, and executes the plan; ``build_*_plan`` returns the plan without
running it.

Two layout families exist for the GEMM + collective ops:

* the reference's column-sharded contracts - ``gemm_allgather(A, B_shard, C)``
  and ``gemm_reducescatter(A, B, C_colshard)``;
* row-sharded variants used by tensor-parallel layers with sequence-sharded
  activations - ``gemm_allgather_rows`` and ``gemm_reducescatter_rows``.

Both run on the same fused tcgen05 kernel (``csrc/kernels/gemm_sm100.cu``); no
library GEMM or NCCL call is involved.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from . import _fused
from ._fused import call_stats, check_status, recover
from ..kernels.fused_gemm import TileCCLTimeoutError
from ..primitives import collectives as _coll

__all__ = [
    "gemm_allscatter", "gemm_allscatter_sharded", "gemm_allgather", "gemm_reducescatter",
    "gemm_allgather_rows", "gemm_reducescatter_rows", "allgather_gemm_reducescatter",
    "allgather", "allreduce", "reduce_scatter", "broadcast", "scatter",
    "build_gemm_allscatter_plan", "build_gemm_allgather_plan", "build_gemm_reducescatter_plan",
    "build_allgather_gemm_reducescatter_plan", "build_allgather_plan", "build_allreduce_plan",
    "build_reduce_scatter_plan",
    "GemmAllScatterPlan", "GemmAllScatterMixedLayoutPlan", "GemmAllGatherPlan",
    "GemmReduceScatterPlan", "AllGatherGemmReduceScatterPlan", "AllGatherPlan", "AllReducePlan",
    "ReduceScatterPlan",
    "GemmAllScatterContract", "GemmAllGatherContract", "GemmReduceScatterContract",
    "AllGatherGemmReduceScatterContract",
    "check_status", "recover", "call_stats", "TileCCLTimeoutError",
]

_STORAGE_KINDS = ("symmetric",)


def _ctx_or_current(ctx):
    if ctx is not None:
        return ctx
    from .. import current_context

    return current_context()


def _mm_key(kind, A, B, C, *extra):
    return (kind, A.data_ptr(), B.data_ptr(), C.data_ptr(), tuple(A.shape), tuple(B.shape),
            tuple(C.shape), A.stride(0), B.stride(0), C.stride(0), A.dtype) + extra


def _cached_plan(ctx, key, build):
    """Plans of the one-call collectives, kept per context: a repeated call on the same
    buffer skips contract resolution (the small-message latency is host time)."""
    cache = ctx.__dict__.setdefault("_collective_plans", {})
    plan = cache.get(key)
    if plan is None:
        if len(cache) >= 512:
            cache.clear()
        plan = cache[key] = build()
    return plan


def _tile_group_info(rows: int, cols: int, elem_bytes: int = 2) -> dict:
    """TileGroup geometry a fused launch over a ``rows x cols`` sub-problem will use: the
    planner's P0 rule with tau_min from the calibration file (see
    ``_fused.default_group_m_tiles``).  Part of the plans' ``to_dict()``."""
    from ..kernels import fused_gemm as fg
    from ..planning.cost_model import calibrated_tau_min_bytes, calibration_path

    m_tiles = -(-rows // fg.BLOCK_M)
    n_tiles = -(-cols // fg.BLOCK_N)
    gm = _fused.default_group_m_tiles(m_tiles, n_tiles, elem_bytes)
    return {"group_m_tiles": gm, "n_groups": -(-m_tiles // gm), "tile": [fg.BLOCK_M, fg.BLOCK_N],
            "tau_min_bytes": calibrated_tau_min_bytes(), "calibration": calibration_path()}


def _check_storage(storage_kind: str) -> None:
    if storage_kind not in _STORAGE_KINDS:
        raise ValueError(f"storage_kind must be one of {_STORAGE_KINDS}, got {storage_kind!r}")


def _check_matrix(name: str, t, ctx, *, on_heap: bool = False) -> None:
    if not isinstance(t, torch.Tensor) or t.dim() != 2:
        raise ValueError(f"{name} must be a 2-D tensor")
    if t.device != ctx.torch_device:
        raise ValueError(f"{name} is on {t.device} but the context is on {ctx.torch_device}")
    if on_heap and ctx.world_size > 1 and not ctx.is_symmetric(t):
        raise ValueError(f"{name} must be allocated from the symmetric heap "
                         "(use ctx.empty / ctx.zeros / ctx.randn)")


def _same_float_dtype(*tensors) -> torch.dtype:
    dt = tensors[0].dtype
    for t in tensors[1:]:
        if t.dtype != dt:
            raise ValueError(f"all operands must share one dtype, got {[x.dtype for x in tensors]}")
    if dt not in (torch.float16, torch.bfloat16):
        raise ValueError(f"fused GEMM operators take float16 or bfloat16 operands, got {dt}")
    return dt


# ==========================================================================
# GEMM + all-scatter
# ==========================================================================
@dataclass(frozen=True)
class GemmAllScatterContract:
    M: int
    K: int
    full_N: int
    rhs_cols: int
    output_cols: int
    rank: int
    world_size: int
    rhs_layout: str
    output_layout: str
    storage_kind: str = "symmetric"

    def to_dict(self) -> dict:
        return dict(self.__dict__)


def _resolve_gemm_allscatter_contract(A, B, C, ctx, full_N, b_layout, c_layout,
                                      storage_kind) -> GemmAllScatterContract:
    _check_storage(storage_kind)
    if (b_layout is None) != (c_layout is None):
        raise ValueError("b_layout and c_layout must be given together (or both omitted)")
    b_layout = b_layout or "full"
    c_layout = c_layout or "full"
    for name, v in (("b_layout", b_layout), ("c_layout", c_layout)):
        if v not in ("full", "shard"):
            raise ValueError(f"{name} must be 'full' or 'shard', got {v!r}")
    if b_layout == "shard" and c_layout == "full":
        raise ValueError("b_layout='shard' with c_layout='full' is gemm_allgather's contract; "
                         "call ops.gemm_allgather(A, B_shard, C) instead")
    for name, t in (("A", A), ("B", B), ("C", C)):
        _check_matrix(name, t, ctx)
    _same_float_dtype(A, B, C)
    M, K = A.shape
    if B.shape[0] != K:
        raise ValueError(f"A is {tuple(A.shape)} but B is {tuple(B.shape)}: inner dimensions differ")
    ws = ctx.world_size
    rhs_cols, out_cols = B.shape[1], C.shape[1]
    if full_N is None:
        full_N = rhs_cols * ws if b_layout == "shard" else rhs_cols
    if full_N % ws:
        raise ValueError(f"full_N={full_N} is not divisible by world_size={ws}")
    want_rhs = full_N if b_layout == "full" else full_N // ws
    want_out = full_N if c_layout == "full" else full_N // ws
    if rhs_cols != want_rhs:
        raise ValueError(f"B has {rhs_cols} columns, expected {want_rhs} for b_layout={b_layout!r}")
    if C.shape[0] != M or out_cols != want_out:
        raise ValueError(f"C is {tuple(C.shape)}, expected {(M, want_out)} for c_layout={c_layout!r}")
    return GemmAllScatterContract(M, K, full_N, rhs_cols, out_cols, ctx.rank, ws, b_layout, c_layout,
                                  storage_kind)


@dataclass(frozen=True)
class GemmAllScatterPlan:
    """full/full or shard/shard: the pattern kernel writes straight into ``C``."""

    ctx: Any = field(repr=False)
    contract: GemmAllScatterContract = None
    pattern_name: str = "fused_sequential"
    pattern_impl: Any = field(default=None, repr=False)
    storage_kind: str = "symmetric"

    @property
    def execution(self):
        from ..patterns.contracts import spec_from_contract

        return spec_from_contract(self.contract)

    def validate_tensors(self, A, B, C) -> None:
        got = _resolve_gemm_allscatter_contract(A, B, C, self.ctx, self.contract.full_N,
                                                self.contract.rhs_layout,
                                                self.contract.output_layout, self.storage_kind)
        if got != self.contract:
            raise ValueError("tensors no longer match this GemmAllScatterPlan; build a new plan")

    def execute(self, A, B, C, *, validate: bool = True):
        if validate:
            self.validate_tensors(A, B, C)
        self.pattern_impl.execute(A, B, C, spec=self.execution)
        return C

    def to_dict(self) -> dict:
        return {"op": "gemm_allscatter", "contract": self.contract.to_dict(),
                "pattern": self.pattern_name, "storage_kind": self.storage_kind,
                "execution": self.execution.to_dict()}


@dataclass(frozen=True)
class GemmAllScatterMixedLayoutPlan:
    """full/shard: ``C_shard = (A @ B)[:, this rank's columns]``.

    Only this rank's own column slice of the full product ends up in the shard
    (peers' pushes land in other slices), so the plan multiplies by that slice of
    ``B`` directly instead of materialising the full product in a workspace.
    """

    ctx: Any = field(repr=False)
    contract: GemmAllScatterContract = None
    pattern_name: str = "local_slice"
    storage_kind: str = "symmetric"

    def validate_tensors(self, A, B, C) -> None:
        got = _resolve_gemm_allscatter_contract(A, B, C, self.ctx, self.contract.full_N, "full",
                                                "shard", self.storage_kind)
        if got != self.contract:
            raise ValueError("tensors no longer match this GemmAllScatterMixedLayoutPlan")

    def execute(self, A, B, C, *, validate: bool = True):
        if validate:
            self.validate_tensors(A, B, C)
        from ..kernels.fused_gemm import gemm

        n = self.contract.output_cols
        gemm(A, B[:, self.ctx.rank * n:(self.ctx.rank + 1) * n], C)
        return C

    def to_dict(self) -> dict:
        return {"op": "gemm_allscatter", "contract": self.contract.to_dict(),
                "pattern": self.pattern_name, "storage_kind": self.storage_kind}


def build_gemm_allscatter_plan(A, B, C, *, ctx=None, full_N=None, b_layout=None, c_layout=None,
                               pattern="auto", hw_info=None, storage_kind="symmetric"):
    ctx = _ctx_or_current(ctx)
    contract = _resolve_gemm_allscatter_contract(A, B, C, ctx, full_N, b_layout, c_layout,
                                                 storage_kind)
    if contract.rhs_layout == "full" and contract.output_layout == "shard":
        return GemmAllScatterMixedLayoutPlan(ctx=ctx, contract=contract, storage_kind=storage_kind)
    if ctx.world_size > 1 and not ctx.is_symmetric(C):
        raise ValueError("C must be allocated from the symmetric heap when world_size > 1")
    from ..patterns import resolve_pattern

    impl = resolve_pattern(pattern, ctx=ctx, M=contract.M, N=contract.full_N, K=contract.K,
                           hw_info=hw_info)
    return GemmAllScatterPlan(ctx=ctx, contract=contract, pattern_name=impl.name,
                              pattern_impl=impl, storage_kind=storage_kind)


def gemm_allscatter(A, B, C, *, ctx=None, full_N=None, b_layout=None, c_layout=None,
                    pattern="auto", hw_info=None, storage_kind="symmetric"):
    """``C = A @ B`` on every rank, with this rank's column slice pushed to all peers.

    Default (full/full) contract: ``A (M, K)``, ``B (K, N)``, ``C (M, N)``; rank
    ``r`` computes the whole product locally and additionally writes columns
    ``[r*N/ws, (r+1)*N/ws)`` into every peer's ``C``.  When the call returns
    (stream order) the peers' slices have arrived in the local ``C`` as well.
    """
    plan = build_gemm_allscatter_plan(A, B, C, ctx=ctx, full_N=full_N, b_layout=b_layout,
                                      c_layout=c_layout, pattern=pattern, hw_info=hw_info,
                                      storage_kind=storage_kind)
    return plan.execute(A, B, C, validate=False)


def gemm_allscatter_sharded(A, B_shard, C_shard, *, full_N, ctx=None, pattern="auto", hw_info=None,
                            storage_kind="symmetric"):
    """shard/shard contract: ``B_shard (K, N/ws)``, ``C_shard (M, N/ws)``."""
    return gemm_allscatter(A, B_shard, C_shard, ctx=ctx, full_N=full_N, b_layout="shard",
                           c_layout="shard", pattern=pattern, hw_info=hw_info,
                           storage_kind=storage_kind)


# ==========================================================================
# GEMM + all-gather
# ==========================================================================
@dataclass(frozen=True)
class GemmAllGatherContract:
    M: int
    K: int
    full_N: int
    shard_cols: int
    rank: int
    world_size: int
    layout: str = "columns"      # "columns" (reference contract) or "rows"
    storage_kind: str = "symmetric"

    def to_dict(self) -> dict:
        return dict(self.__dict__)


@dataclass(frozen=True)
class GemmAllGatherPlan:
    ctx: Any = field(repr=False)
    contract: GemmAllGatherContract = None
    storage_kind: str = "symmetric"
    b_is_nk: bool = False

    def validate_tensors(self, A, B, C) -> None:
        got = _resolve_gemm_allgather_contract(A, B, C, self.ctx, self.contract.layout,
                                               self.storage_kind, self.b_is_nk)
        if got != self.contract:
            raise ValueError("tensors no longer match this GemmAllGatherPlan; build a new plan")

    def execute(self, A, B, C, *, validate: bool = True, wait: bool = True, a_host=None,
                a_host_order: str = "stream"):
        """``a_host``: pinned host tensor shaped like ``A``; when given, ``A`` is filled
        from it on a side stream, run of tile rows by run, while the kernel computes."""
        if validate:
            self.validate_tensors(A, B, C)
        c, ctx = self.contract, self.ctx
        if c.layout == "columns":
            _fused.push_all(ctx, "gemm_allgather_cols", A, B, C, region_row0=0,
                            region_col0=c.rank * c.shard_cols, b_is_nk=self.b_is_nk, wait=wait,
                            a_host=a_host, a_host_order=a_host_order)
        else:
            _fused.push_all(ctx, "gemm_allgather_rows", A, B, C, region_row0=c.rank * A.shape[0],
                            region_col0=0, b_is_nk=self.b_is_nk, wait=wait, a_host=a_host,
                            a_host_order=a_host_order)
        return C

    def to_dict(self) -> dict:
        c = self.contract
        rows = c.M if c.layout == "columns" else c.M // c.world_size
        cols = c.shard_cols if c.layout == "columns" else c.full_N
        d = {"op": "gemm_allgather", "contract": c.to_dict(),
             "storage_kind": self.storage_kind, "kernel": "fused_gemm_sm100/push_all",
             "signal_mode": "counting", "wait_mode": "wait_ge",
             "tile_groups": _tile_group_info(rows, cols)}
        d["group_m_tiles"] = d["tile_groups"]["group_m_tiles"]
        return d


def _resolve_gemm_allgather_contract(A, B, C, ctx, layout, storage_kind, b_is_nk=False):
    _check_storage(storage_kind)
    _check_matrix("A", A, ctx)
    _check_matrix("B", B, ctx)
    _check_matrix("C", C, ctx, on_heap=True)
    _same_float_dtype(A, B, C)
    ws = ctx.world_size
    K, nb = (B.shape[1], B.shape[0]) if b_is_nk else (B.shape[0], B.shape[1])
    if A.shape[1] != K:
        raise ValueError(f"A is {tuple(A.shape)} but B is {tuple(B.shape)}: inner dimensions differ")
    if not C.is_contiguous():
        raise ValueError("C must be contiguous")
    if layout == "columns":
        M, full_N = A.shape[0], nb * ws
        if tuple(C.shape) != (M, full_N):
            raise ValueError(f"C is {tuple(C.shape)}, expected {(M, full_N)} "
                             f"(A rows x world_size * B_shard columns)")
    elif layout == "rows":
        M, full_N = A.shape[0] * ws, nb
        if tuple(C.shape) != (M, full_N):
            raise ValueError(f"C is {tuple(C.shape)}, expected {(M, full_N)} "
                             f"(world_size * A_local rows x B columns)")
    else:
        raise ValueError(f"layout must be 'columns' or 'rows', got {layout!r}")
    return GemmAllGatherContract(M, K, full_N, nb, ctx.rank, ws, layout, storage_kind)


def build_gemm_allgather_plan(A, B_shard, C, *, ctx=None, storage_kind="symmetric",
                              layout="columns", b_is_nk=False) -> GemmAllGatherPlan:
    ctx = _ctx_or_current(ctx)
    contract = _resolve_gemm_allgather_contract(A, B_shard, C, ctx, layout, storage_kind, b_is_nk)
    return GemmAllGatherPlan(ctx=ctx, contract=contract, storage_kind=storage_kind, b_is_nk=b_is_nk)


def gemm_allgather(A, B_shard, C, *, ctx=None, storage_kind="symmetric"):
    """Column-parallel GEMM whose output is gathered on every rank.

    ``A (M, K)`` full, ``B_shard (K, N/ws)``, ``C (M, N)`` on the heap:
    ``C[:, r*N/ws:(r+1)*N/ws] = A_r @ B_shard_r`` for every rank ``r``, on every rank.
    """
    ctx = _ctx_or_current(ctx)
    return _cached_plan(ctx, _mm_key("gemm_allgather", A, B_shard, C, storage_kind),
                        lambda: build_gemm_allgather_plan(A, B_shard, C, ctx=ctx,
                                                          storage_kind=storage_kind)).execute(
        A, B_shard, C, validate=False)


def gemm_allgather_rows(A_local, B, C, *, ctx=None, b_is_nk=False, wait=True, a_host=None,
                        a_host_order="stream"):
    """Row-sharded form: ``A_local (M/ws, K)``, ``B (K, N)``, ``C (M, N)`` on the heap;
    rows ``[r*M/ws, (r+1)*M/ws)`` of ``C`` on every rank come from rank ``r``.

    ``a_host`` (pinned host tensor shaped like ``A_local``): the activations are
    streamed from the host into ``A_local`` while the kernel runs, tile rows in
    the order the kernel consumes them, so only the last run's math is exposed
    after the PCIe copy.  ``a_host_order="plan"``: the caller guarantees that no other
    pending work on the stream touches ``A_local``; the copy then only follows this
    operator's previous call on the same buffers and overlaps whatever else is queued."""
    ctx = _ctx_or_current(ctx)
    plan = _cached_plan(ctx, _mm_key("gemm_allgather_rows", A_local, B, C, b_is_nk),
                        lambda: build_gemm_allgather_plan(A_local, B, C, ctx=ctx, layout="rows",
                                                          b_is_nk=b_is_nk))
    return plan.execute(A_local, B, C, validate=False, wait=wait, a_host=a_host,
                        a_host_order=a_host_order)


# ==========================================================================
# GEMM + reduce-scatter
# ==========================================================================
@dataclass(frozen=True)
class GemmReduceScatterContract:
    M: int
    K: int
    full_N: int
    out_rows: int
    out_cols: int
    rank: int
    world_size: int
    layout: str = "columns"
    storage_kind: str = "symmetric"

    def to_dict(self) -> dict:
        return dict(self.__dict__)


@dataclass(frozen=True)
class GemmReduceScatterPlan:
    ctx: Any = field(repr=False)
    contract: GemmReduceScatterContract = None
    implementation: str = "device"
    storage_kind: str = "symmetric"
    b_is_nk: bool = False

    def validate_tensors(self, A, B, C) -> None:
        got = _resolve_gemm_reducescatter_contract(A, B, C, self.ctx, self.contract.layout,
                                                   self.storage_kind, self.b_is_nk)
        if got != self.contract:
            raise ValueError("tensors no longer match this GemmReduceScatterPlan; build a new plan")

    def execute(self, A, B, C, *, validate: bool = True, a_host=None,
                a_host_order: str = "stream"):
        """``a_host``: pinned host tensor shaped like ``A`` to stream the operand from."""
        if validate:
            self.validate_tensors(A, B, C)
        axis = 1 if self.contract.layout == "columns" else 0
        _fused.reduce_scatter(self.ctx, f"gemm_reducescatter_{self.contract.layout}", A, B, C,
                              split_axis=axis, b_is_nk=self.b_is_nk, a_host=a_host,
                              a_host_order=a_host_order)
        return C

    def to_dict(self) -> dict:
        c = self.contract
        d = {"op": "gemm_reducescatter", "contract": c.to_dict(),
             "implementation": self.implementation, "storage_kind": self.storage_kind,
             "kernel": "fused_gemm_sm100/reduce_scatter", "signal_mode": "counting",
             "wait_mode": "wait_ge", "partials": "16-bit staged, fp32 reduction in rank order",
             "tile_groups": _tile_group_info(c.out_rows, c.out_cols)}
        d["group_m_tiles"] = d["tile_groups"]["group_m_tiles"]
        return d


def _resolve_gemm_reducescatter_contract(A, B, C, ctx, layout, storage_kind, b_is_nk=False):
    _check_storage(storage_kind)
    for name, t in (("A", A), ("B", B), ("C", C)):
        _check_matrix(name, t, ctx)
    _same_float_dtype(A, B, C)
    ws = ctx.world_size
    K, N = (B.shape[1], B.shape[0]) if b_is_nk else (B.shape[0], B.shape[1])
    M = A.shape[0]
    if A.shape[1] != K:
        raise ValueError(f"A is {tuple(A.shape)} but B is {tuple(B.shape)}: inner dimensions differ")
    if not C.is_contiguous():
        raise ValueError("C must be contiguous")
    if layout == "columns":
        if N % ws:
            raise ValueError(f"N={N} is not divisible by world_size={ws}")
        want = (M, N // ws)
    elif layout == "rows":
        if M % ws:
            raise ValueError(f"M={M} is not divisible by world_size={ws}")
        want = (M // ws, N)
    else:
        raise ValueError(f"layout must be 'columns' or 'rows', got {layout!r}")
    if tuple(C.shape) != want:
        raise ValueError(f"C is {tuple(C.shape)}, expected {want} for layout={layout!r}")
    return GemmReduceScatterContract(M, K, N, want[0], want[1], ctx.rank, ws, layout, storage_kind)


def _resolve_rs_implementation(implementation: str) -> str:
    # The reference switches between a host "reference" path and a device path
    # (tileccl/ops.py:2060-2129); here every mode runs the fused device kernel.
    if implementation not in ("auto", "device", "reference"):
        raise ValueError(f"implementation must be 'auto', 'device' or 'reference', got {implementation!r}")
    if implementation == "reference":
        raise ValueError("implementation='reference' (host-side reduction) does not exist in this "
                         "library; use 'auto' or 'device'")
    return "device"


def build_gemm_reducescatter_plan(A, B, C, *, ctx=None, implementation="auto",
                                  storage_kind="symmetric", layout="columns",
                                  b_is_nk=False) -> GemmReduceScatterPlan:
    ctx = _ctx_or_current(ctx)
    impl = _resolve_rs_implementation(implementation)
    contract = _resolve_gemm_reducescatter_contract(A, B, C, ctx, layout, storage_kind, b_is_nk)
    return GemmReduceScatterPlan(ctx=ctx, contract=contract, implementation=impl,
                                 storage_kind=storage_kind, b_is_nk=b_is_nk)


def gemm_reducescatter(A, B, C, *, ctx=None, implementation="auto", storage_kind="symmetric"):
    """Row-parallel GEMM with the partial sums reduce-scattered along columns.

    ``A (M, K)`` is this rank's contribution, ``B (K, N)``, ``C (M, N/ws)``:
    ``C_r = sum_i (A_i @ B_i)[:, r*N/ws:(r+1)*N/ws]``.
    """
    ctx = _ctx_or_current(ctx)
    return _cached_plan(ctx, _mm_key("gemm_reducescatter", A, B, C, implementation, storage_kind),
                        lambda: build_gemm_reducescatter_plan(
                            A, B, C, ctx=ctx, implementation=implementation,
                            storage_kind=storage_kind)).execute(A, B, C, validate=False)


def gemm_reducescatter_rows(A, B, C_local, *, ctx=None, b_is_nk=False, a_host=None,
                            a_host_order="stream"):
    """Row-sharded form: ``A (M, K/ws)``, ``B (K/ws, N)``, ``C_local (M/ws, N)``:
    ``C_local_r = sum_i (A_i @ B_i)[r*M/ws:(r+1)*M/ws, :]``.  ``a_host`` streams ``A``
    from pinned host memory as in :func:`gemm_allgather_rows`."""
    ctx = _ctx_or_current(ctx)
    plan = _cached_plan(ctx, _mm_key("gemm_reducescatter_rows", A, B, C_local, b_is_nk),
                        lambda: build_gemm_reducescatter_plan(A, B, C_local, ctx=ctx, layout="rows",
                                                              b_is_nk=b_is_nk))
    return plan.execute(A, B, C_local, validate=False, a_host=a_host, a_host_order=a_host_order)


# ==========================================================================
# all-gather -> GEMM (-> reduce-scatter)
# ==========================================================================
@dataclass(frozen=True)
class AllGatherGemmReduceScatterContract:
    M: int
    K: int
    shard_cols: int
    N: int
    rank: int
    world_size: int
    reduce_output: bool = False
    storage_kind: str = "symmetric"

    def to_dict(self) -> dict:
        return dict(self.__dict__)


@dataclass(frozen=True)
class AllGatherGemmReduceScatterPlan:
    ctx: Any = field(repr=False)
    contract: AllGatherGemmReduceScatterContract = None
    storage_kind: str = "symmetric"

    def validate_tensors(self, input_shard, W, output) -> None:
        got = _resolve_ag_gemm_rs_contract(input_shard, W, output, self.ctx, self.storage_kind)
        if got != self.contract:
            raise ValueError("tensors no longer match this AllGatherGemmReduceScatterPlan")

    def execute(self, input_shard, W, output, *, validate: bool = True):
        if validate:
            self.validate_tensors(input_shard, W, output)
        from ..parallel.chain import allgather_gemm

        allgather_gemm(self.ctx, input_shard, W, output)
        return output

    def to_dict(self) -> dict:
        return {"op": "allgather_gemm_reducescatter", "contract": self.contract.to_dict(),
                "storage_kind": self.storage_kind,
                "stages": ["tile_allgather(columns)", "fused_gemm_sm100(gated on arrival)"]}


def _resolve_ag_gemm_rs_contract(input_shard, W, output, ctx, storage_kind):
    _check_storage(storage_kind)
    _check_matrix("input_shard", input_shard, ctx, on_heap=True)
    _check_matrix("W", W, ctx)
    _check_matrix("output", output, ctx)
    _same_float_dtype(input_shard, W, output)
    ws = ctx.world_size
    M, kc = input_shard.shape
    K, N = W.shape
    if kc * ws != K:
        raise ValueError(f"input_shard has {kc} columns; W has {K} rows; expected K = columns * "
                         f"world_size = {kc * ws}")
    if tuple(output.shape) != (M, N):
        raise ValueError(f"output is {tuple(output.shape)}, expected {(M, N)}")
    return AllGatherGemmReduceScatterContract(M, K, kc, N, ctx.rank, ws, False, storage_kind)


def build_allgather_gemm_reducescatter_plan(input_shard, W, output, *, ctx=None,
                                            storage_kind="symmetric"):
    ctx = _ctx_or_current(ctx)
    contract = _resolve_ag_gemm_rs_contract(input_shard, W, output, ctx, storage_kind)
    return AllGatherGemmReduceScatterPlan(ctx=ctx, contract=contract, storage_kind=storage_kind)


def allgather_gemm_reducescatter(input_shard, W, output, *, ctx=None, storage_kind="symmetric"):
    """``output = cat(shards over ranks, dim=1) @ W`` on every rank.

    ``input_shard (M, K/ws)`` is a column shard of the left operand.  As in the
    reference (tileccl/ops.py:2348-2430) the product is not reduced across ranks;
    the tensor-parallel chain that does reduce-scatter its output is
    ``tileccl_b200.models.TPMLP`` / ``parallel.chain``.
    """
    return build_allgather_gemm_reducescatter_plan(
        input_shard, W, output, ctx=ctx, storage_kind=storage_kind).execute(
            input_shard, W, output, validate=False)


# ==========================================================================
# plain collectives
# ==========================================================================
def _vector_contract(name: str, t, ctx) -> None:
    if not isinstance(t, torch.Tensor):
        raise ValueError(f"{name} must be a tensor")
    if t.device != ctx.torch_device:
        raise ValueError(f"{name} is on {t.device} but the context is on {ctx.torch_device}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if ctx.world_size > 1 and not ctx.is_symmetric(t):
        raise ValueError(f"{name} must be allocated from the symmetric heap")


@dataclass(frozen=True)
class AllGatherPlan:
    ctx: Any = field(repr=False)
    numel: int = 0
    dtype: Any = None
    storage_kind: str = "symmetric"

    def validate_tensors(self, src, output) -> None:
        _vector_contract("src", src, self.ctx)
        _vector_contract("output", output, self.ctx)
        if src.numel() != self.numel or src.dtype != self.dtype:
            raise ValueError("src no longer matches this AllGatherPlan")
        if output.numel() != self.numel * self.ctx.world_size or output.dtype != self.dtype:
            raise ValueError(f"output must have {self.numel * self.ctx.world_size} elements of {self.dtype}")

    def execute(self, src, output, *, validate: bool = True):
        if validate:
            self.validate_tensors(src, output)
        from ..primitives import collectives

        collectives.allgather(src, output, self.ctx.heap, ctx=self.ctx)
        return output

    def to_dict(self) -> dict:
        return {"op": "allgather", "numel": self.numel, "dtype": str(self.dtype),
                "world_size": self.ctx.world_size, "storage_kind": self.storage_kind}


def build_allgather_plan(src, output, *, ctx=None, storage_kind="symmetric") -> AllGatherPlan:
    ctx = _ctx_or_current(ctx)
    _check_storage(storage_kind)
    plan = AllGatherPlan(ctx=ctx, numel=src.numel(), dtype=src.dtype, storage_kind=storage_kind)
    plan.validate_tensors(src, output)
    return plan


def allgather(src, output, *, ctx=None, storage_kind="symmetric"):
    """Rank-major concatenation of every rank's ``src`` into ``output`` on every rank."""
    ctx = _ctx_or_current(ctx)
    if _coll.try_fast(ctx.heap, "allgather", src, output):
        return output
    key = ("allgather", src.data_ptr(), output.data_ptr(), src.numel(), src.dtype, storage_kind)
    return _cached_plan(ctx, key, lambda: build_allgather_plan(
        src, output, ctx=ctx, storage_kind=storage_kind)).execute(src, output, validate=False)


@dataclass(frozen=True)
class AllReducePlan:
    ctx: Any = field(repr=False)
    numel: int = 0
    dtype: Any = None
    op: str = "sum"
    execution: Any = None
    storage_kind: str = "symmetric"

    # The execution spec's fields are part of the plan's public face.
    def __getattr__(self, name):
        ex = object.__getattribute__(self, "execution")
        if ex is not None and hasattr(ex, name):
            return getattr(ex, name)
        raise AttributeError(name)

    def validate_tensor(self, tensor) -> None:
        _vector_contract("tensor", tensor, self.ctx)
        if tensor.numel() != self.numel or tensor.dtype != self.dtype:
            raise ValueError("tensor no longer matches this AllReducePlan")

    def execute(self, tensor, *, validate: bool = True):
        if validate:
            self.validate_tensor(tensor)
        from ..primitives import collectives

        collectives.allreduce(tensor, self.ctx.heap, op=self.op, ctx=self.ctx,
                              _execution=self.execution)
        return tensor

    def to_dict(self) -> dict:
        d = {"op": "allreduce", "reduce_op": self.op, "numel": self.numel, "dtype": str(self.dtype),
             "world_size": self.ctx.world_size, "storage_kind": self.storage_kind}
        if self.execution is not None:
            d.update(self.execution.to_dict())
        return d


def build_allreduce_plan(tensor, *, ctx=None, op="sum", storage_kind="symmetric") -> AllReducePlan:
    ctx = _ctx_or_current(ctx)
    _check_storage(storage_kind)
    if op != "sum":
        raise ValueError(f"only op='sum' is supported, got {op!r}")
    from ..primitives import collectives

    _vector_contract("tensor", tensor, ctx)
    execution = collectives.resolve_allreduce_execution(tensor, heap=ctx.heap, op=op, ctx=ctx)
    return AllReducePlan(ctx=ctx, numel=tensor.numel(), dtype=tensor.dtype, op=op,
                         execution=execution, storage_kind=storage_kind)


def allreduce(tensor, *, ctx=None, op="sum", storage_kind="symmetric"):
    """In-place sum over ranks."""
    ctx = _ctx_or_current(ctx)
    if op == "sum" and _coll.try_fast(ctx.heap, "allreduce", tensor):
        return tensor
    # (the plan's execution spec depends on the configuration: part of the key)
    key = ("allreduce", tensor.data_ptr(), tensor.numel(), tensor.dtype, op, storage_kind,
           _coll._config_generation())
    return _cached_plan(ctx, key, lambda: build_allreduce_plan(
        tensor, ctx=ctx, op=op, storage_kind=storage_kind)).execute(tensor, validate=False)


@dataclass(frozen=True)
class ReduceScatterPlan:
    ctx: Any = field(repr=False)
    numel_out: int = 0
    dtype: Any = None
    implementation: str = "device"
    storage_kind: str = "symmetric"

    def validate_tensors(self, src, output) -> None:
        _vector_contract("src", src, self.ctx)
        _vector_contract("output", output, self.ctx)
        if output.numel() != self.numel_out or output.dtype != self.dtype:
            raise ValueError("output no longer matches this ReduceScatterPlan")
        if src.numel() != self.numel_out * self.ctx.world_size or src.dtype != self.dtype:
            raise ValueError(f"src must have {self.numel_out * self.ctx.world_size} elements of {self.dtype}")

    def execute(self, src, output, *, validate: bool = True):
        if validate:
            self.validate_tensors(src, output)
        from ..primitives import collectives

        collectives.reduce_scatter(src, output, self.ctx.heap, ctx=self.ctx)
        return output

    def to_dict(self) -> dict:
        return {"op": "reduce_scatter", "numel_out": self.numel_out, "dtype": str(self.dtype),
                "implementation": self.implementation, "world_size": self.ctx.world_size,
                "storage_kind": self.storage_kind}


def build_reduce_scatter_plan(src, output, *, ctx=None, implementation="auto",
                              storage_kind="symmetric") -> ReduceScatterPlan:
    ctx = _ctx_or_current(ctx)
    _check_storage(storage_kind)
    impl = _resolve_rs_implementation(implementation)
    plan = ReduceScatterPlan(ctx=ctx, numel_out=output.numel(), dtype=output.dtype,
                             implementation=impl, storage_kind=storage_kind)
    plan.validate_tensors(src, output)
    return plan


def reduce_scatter(src, output, *, ctx=None, implementation="auto", storage_kind="symmetric"):
    """``output = sum over ranks of src[rank * n:(rank + 1) * n]`` (rank-major chunks)."""
    ctx = _ctx_or_current(ctx)
    if _coll.try_fast(ctx.heap, "reduce_scatter", src, output):
        return output
    key = ("reduce_scatter", src.data_ptr(), output.data_ptr(), src.numel(), src.dtype,
           implementation, storage_kind)
    return _cached_plan(ctx, key, lambda: build_reduce_scatter_plan(
        src, output, ctx=ctx, implementation=implementation,
        storage_kind=storage_kind)).execute(src, output, validate=False)


def broadcast(tensor, *, ctx=None, root: int = 0):
    """Every rank's ``tensor`` becomes ``root``'s."""
    ctx = _ctx_or_current(ctx)
    if _coll.try_fast(ctx.heap, "broadcast", tensor, None, root):
        return tensor
    _vector_contract("tensor", tensor, ctx)
    _coll.broadcast(tensor, ctx.heap, root=root, ctx=ctx)
    return tensor


def scatter(src, output, *, ctx=None, root: int = 0):
    """Rank ``r`` receives chunk ``r`` of ``root``'s ``src``."""
    ctx = _ctx_or_current(ctx)
    if _coll.try_fast(ctx.heap, "scatter", src, output, root):
        return output
    _vector_contract("src", src, ctx)
    _vector_contract("output", output, ctx)
    _coll.scatter(src, output, ctx.heap, root=root, ctx=ctx)
    return output
