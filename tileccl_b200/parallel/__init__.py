"""Parallelism building blocks on top of the fused operators: all-gather -> GEMM
chains (sequence-parallel inputs of a tensor-parallel layer)."""

from .chain import allgather_gemm, rows_allgather_gemm

__all__ = ["allgather_gemm", "rows_allgather_gemm"]
