"""CPU emulation of the multi-rank fused operators (``csrc/cpu_emul/fake_device.cc``).

Ranks are threads of this process; the "symmetric heap" is host memory and the
TileGroup counters are ``std::atomic`` words with release / acquire ordering.
Every rank walks the tile order of the GPU kernel.  Used as a GPU-free oracle
(fp32) and for host-side fault injection: a faulty rank makes the others time out
and report, never hang.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .. import _native

FAULTS = {"none": 0, "no_signal": 1, "short_signal": 2, "absent": 3, "late": 4}


@dataclass(frozen=True)
class EmulationStatus:
    code: int
    where: int
    rank: int
    item: int
    expected: int
    observed: int

    @property
    def ok(self) -> bool:
        return self.code == 0

    @property
    def timed_out(self) -> bool:
        return self.code == 2


class EmulatedTimeout(RuntimeError):
    """A rank's bounded wait ran out (the emulated counterpart of TileCCLTimeoutError)."""

    def __init__(self, status: EmulationStatus):
        super().__init__(f"emulated rank {status.rank} gave up waiting: expected {status.expected}, "
                         f"observed {status.observed} (item {status.item}, site {status.where})")
        self.status = status


def _stack(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    return torch.stack([t.detach().to(torch.float32).cpu().contiguous() for t in tensors]).contiguous()


def _run(fn_name: str, ws: int, M: int, N: int, K: int, A: torch.Tensor, B: torch.Tensor,
         out: torch.Tensor, block_m: int, block_n: int, group_m_tiles: int, fault_rank: int,
         fault: str, fault_delay_ms: int, timeout_ms: int, raise_on_timeout: bool) -> EmulationStatus:
    if fault not in FAULTS:
        raise ValueError(f"fault must be one of {sorted(FAULTS)}")
    st = (C.c_int32 * 6)()
    _native.call(fn_name, ws, M, N, K, A.data_ptr(), B.data_ptr(), out.data_ptr(), block_m, block_n,
                 group_m_tiles, fault_rank, FAULTS[fault], fault_delay_ms, timeout_ms, st)
    status = EmulationStatus(*[int(x) for x in st])
    if raise_on_timeout and not status.ok:
        raise EmulatedTimeout(status)
    return status


def gemm_allgather(A_shards: Sequence[torch.Tensor], B_list: Sequence[torch.Tensor], *,
                   block_m: int = 128, block_n: int = 256, group_m_tiles: int = 1,
                   fault_rank: int = -1, fault: str = "none", fault_delay_ms: int = 0,
                   timeout_ms: int = 2000, raise_on_timeout: bool = True):
    """Rank r holds ``A_shards[r] (M/ws, K)`` and ``B_list[r] (K, N)``; returns the list of
    every rank's ``C (M, N)`` (rows ``[r*M/ws, (r+1)*M/ws)`` come from rank r) and the status."""
    ws = len(A_shards)
    mloc, K = A_shards[0].shape
    N = B_list[0].shape[1]
    A, B = _stack(A_shards), _stack(B_list)
    out = torch.zeros(ws, mloc * ws, N, dtype=torch.float32)
    status = _run("tccl_emul_gemm_allgather", ws, mloc * ws, N, K, A, B, out, block_m, block_n,
                  group_m_tiles, fault_rank, fault, fault_delay_ms, timeout_ms, raise_on_timeout)
    return [out[r] for r in range(ws)], status


def gemm_reducescatter(A_list: Sequence[torch.Tensor], B_list: Sequence[torch.Tensor], *,
                       block_m: int = 128, block_n: int = 256, group_m_tiles: int = 1,
                       fault_rank: int = -1, fault: str = "none", fault_delay_ms: int = 0,
                       timeout_ms: int = 2000, raise_on_timeout: bool = True, own_lag: int = 0,
                       signal_delay_tiles: int = 0, flush_before_wait: bool = True):
    """Rank r holds ``A_list[r] (M, K/ws)`` and ``B_list[r] (K/ws, N)``; returns the list of
    ``C_r (M/ws, N) = sum_i (A_i @ B_i)[r*M/ws:(r+1)*M/ws]`` and the status.

    ``own_lag``: rounds by which every rank's own (reducing) tile rows trail its remote
    rows (0 = own rows last), the schedule of the sm_100a kernel.  ``signal_delay_tiles``
    holds every tile's signal back until that many later tiles are done (the kernel signals
    only after a tile's bulk stores have landed); ``flush_before_wait`` sends all held
    signals before a rank blocks at an own tile, which is what keeps that scheme from
    deadlocking."""
    ws = len(A_list)
    M, kloc = A_list[0].shape
    N = B_list[0].shape[1]
    A, B = _stack(A_list), _stack(B_list)
    out = torch.zeros(ws, M // ws, N, dtype=torch.float32)
    st = (C.c_int32 * 6)()
    _native.call("tccl_emul_gemm_reducescatter_ex", ws, M, N, kloc * ws, A.data_ptr(),
                 B.data_ptr(), out.data_ptr(), block_m, block_n, group_m_tiles, own_lag,
                 signal_delay_tiles, 1 if flush_before_wait else 0, fault_rank, FAULTS[fault],
                 fault_delay_ms, timeout_ms, st)
    status = EmulationStatus(*[int(x) for x in st])
    if raise_on_timeout and not status.ok:
        raise EmulatedTimeout(status)
    return [out[r] for r in range(ws)], status


def tile_order(m_tiles_local: int, n_tiles_local: int, *, owners: int = 1, rank: int = 0,
               world_size: int = 1, rot_m_tiles: int = 0, own_lag: int = 0) -> list:
    """``(owner, tile_row, tile_col)`` in the order rank ``rank`` visits its tiles.

    ``own_lag`` (reduce-scatter): rounds by which the rank's own tile rows trail the
    remote rows; 0 keeps all own rows for the end."""
    n = m_tiles_local * n_tiles_local * owners
    buf = (C.c_int32 * (3 * n))()
    _native.call("tccl_plan_tile_order_ex", m_tiles_local, n_tiles_local, owners, rank, world_size,
                 rot_m_tiles, own_lag, buf, n)
    return [(buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]) for i in range(n)]
