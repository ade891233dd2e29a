"""Execution contract shared by the GEMM + all-scatter overlap patterns.

A pattern receives ``A (M, K)``, ``B`` and ``C`` plus one resolved
``PatternExecutionSpec`` saying which layout each tensor has and which column
slice of the output this rank pushes to its peers.  Field names follow the
reference (tileccl/patterns/contracts.py:46-230).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

LAYOUTS = ("full", "shard")


@dataclass(frozen=True)
class PatternTensorSpec:
    rows: int
    cols: int
    layout_kind: str
    world_size: int
    storage_kind: str = "symmetric"

    def to_dict(self) -> dict:
        return {"rows": self.rows, "cols": self.cols, "layout_kind": self.layout_kind,
                "world_size": self.world_size, "storage_kind": self.storage_kind}


@dataclass(frozen=True)
class PatternExecutionSpec:
    M: int
    K: int
    full_N: int
    local_N: int
    rank: int
    world_size: int
    rhs: PatternTensorSpec
    output: PatternTensorSpec
    scatter_src_col_offset: int
    scatter_cols: int
    scatter_dst_leading_dim: int
    scatter_dst_col_offset: int

    @property
    def rhs_layout(self) -> str:
        return self.rhs.layout_kind

    @property
    def output_layout(self) -> str:
        return self.output.layout_kind

    def to_dict(self) -> dict:
        return {"M": self.M, "K": self.K, "full_N": self.full_N, "local_N": self.local_N,
                "rank": self.rank, "world_size": self.world_size, "rhs": self.rhs.to_dict(),
                "output": self.output.to_dict(),
                "scatter": {"src_col_offset": self.scatter_src_col_offset,
                            "cols": self.scatter_cols,
                            "dst_leading_dim": self.scatter_dst_leading_dim,
                            "dst_col_offset": self.scatter_dst_col_offset}}


def _build(M, K, full_N, rhs_cols, out_cols, rank, ws, b_layout, c_layout, storage_kind):
    local_N = full_N // ws
    if b_layout == "full" and c_layout == "full":
        # every rank computes all of C and pushes its own column slice
        src_off, cols, dst_ld, dst_off = rank * local_N, local_N, full_N, rank * local_N
    elif b_layout == "shard" and c_layout == "shard":
        # every rank computes its shard and writes it over the peers' shard buffers
        src_off, cols, dst_ld, dst_off = 0, local_N, local_N, 0
    else:
        raise ValueError(
            f"mixed layouts (b_layout={b_layout!r}, c_layout={c_layout!r}) are not a pattern "
            "contract; full/shard is handled by ops.gemm_allscatter, shard/full is ops.gemm_allgather")
    return PatternExecutionSpec(
        M=M, K=K, full_N=full_N, local_N=local_N, rank=rank, world_size=ws,
        rhs=PatternTensorSpec(K, rhs_cols, b_layout, ws, storage_kind),
        output=PatternTensorSpec(M, out_cols, c_layout, ws, storage_kind),
        scatter_src_col_offset=src_off, scatter_cols=cols, scatter_dst_leading_dim=dst_ld,
        scatter_dst_col_offset=dst_off)


def resolve_pattern_execution(A, B, C, *, rank: int, world_size: int, full_N: Optional[int] = None,
                              b_layout: Optional[str] = None, c_layout: Optional[str] = None,
                              storage_kind: str = "symmetric") -> PatternExecutionSpec:
    """Validate shapes / layouts and return the canonical spec."""
    if A.ndim != 2 or B.ndim != 2 or C.ndim != 2:
        raise ValueError(f"Pattern tensors must all be 2-D: got A.ndim={A.ndim}, B.ndim={B.ndim}, "
                         f"C.ndim={C.ndim}")
    if (b_layout is None) != (c_layout is None):
        raise ValueError("b_layout and c_layout must be given together")
    b_layout, c_layout = b_layout or "full", c_layout or "full"
    for name, v in (("b_layout", b_layout), ("c_layout", c_layout)):
        if v not in LAYOUTS:
            raise ValueError(f"{name} must be one of {LAYOUTS}, got {v!r}")
    M, K = A.shape
    if B.shape[0] != K:
        raise ValueError(f"inner dimensions differ: A is {tuple(A.shape)}, B is {tuple(B.shape)}")
    if C.shape[0] != M:
        raise ValueError(f"C has {C.shape[0]} rows, A has {M}")
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank/world_size: {rank}/{world_size}")
    if full_N is None:
        full_N = B.shape[1] * world_size if b_layout == "shard" else B.shape[1]
    if full_N % world_size:
        raise ValueError(f"full_N={full_N} is not divisible by world_size={world_size}")
    want_b = full_N if b_layout == "full" else full_N // world_size
    want_c = full_N if c_layout == "full" else full_N // world_size
    if B.shape[1] != want_b:
        raise ValueError(f"B has {B.shape[1]} columns, expected {want_b} for b_layout={b_layout!r}")
    if C.shape[1] != want_c:
        raise ValueError(f"C has {C.shape[1]} columns, expected {want_c} for c_layout={c_layout!r}")
    return _build(M, K, full_N, B.shape[1], C.shape[1], rank, world_size, b_layout, c_layout,
                  storage_kind)


def spec_from_contract(contract) -> PatternExecutionSpec:
    """Spec for an already validated ``ops.GemmAllScatterContract``."""
    return _build(contract.M, contract.K, contract.full_N, contract.rhs_cols, contract.output_cols,
                  contract.rank, contract.world_size, contract.rhs_layout, contract.output_layout,
                  contract.storage_kind)
