"""Python handle on the fused tcgen05 GEMM family (``csrc/kernels/gemm_sm100.cu``).

``FusedGemmPlan`` owns one native plan: the tensor maps for a fixed set of
operand / destination addresses plus the launch geometry.  Building it costs a
dozen driver calls; launching it costs one kernel launch, so callers keep plans
(see ``PlanCache``) and re-launch them every step.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from .. import _native
from ..utils.config import current as _config

MODE_GEMM = 0
MODE_PUSH_ALL = 1
MODE_REDUCE_SCATTER = 2
MODE_ALL_SCATTER = 3

AG_PUSH_WARPS = 2          # warps per CTA that push the A operand (one gate arrival each)
PUSH_STORES = 0
PUSH_TMA = 1
PUSH_MULTIMEM = 2

EPI_NONE = 0
EPI_SILU_GATE = 1

BLOCK_M = 128
BLOCK_N = 256
BLOCK_K = 64
EPILOGUE_SLABS = 4  # one signal increment per 32-row slab of a tile

_DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1}
STATUS_WORDS = 8
STAT_WORDS = 256 * 4       # one row of four counters per CTA

# Kernel launches issued through this module since import (benchmarks report it).
LAUNCH_COUNT = 0

_STATUS_NAMES = {0: "ok", 1: "timeout waiting for an on-chip pipeline barrier",
                 2: "timeout waiting for a peer signal", 3: "bad argument"}


class TileCCLTimeoutError(RuntimeError):
    """A device-side wait ran out of its budget; the kernel returned cleanly."""


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(
            f"the tcgen05 GEMM path handles float16 and bfloat16 operands, got {dtype}"
        ) from None


def decode_status(words: Sequence[int]) -> dict:
    code = int(words[0])
    return {
        "code": code,
        "what": _STATUS_NAMES.get(code, f"unknown({code})"),
        "where": int(words[1]),
        "expected": int(words[2]),
        "observed": int(words[3]),
        "rank": int(words[4]),
        "item": int(words[5]),
    }


def raise_on_status(status: torch.Tensor) -> None:
    """Read a status block back (synchronises) and raise if a wait timed out."""
    words = status.cpu().tolist()
    if words[0] != 0:
        info = decode_status(words)
        status.zero_()
        raise TileCCLTimeoutError(f"device wait gave up: {info}")


@dataclass
class FusedGemmSpec:
    """Everything the native plan builder needs, in Python types."""

    mode: int
    dtype: torch.dtype
    a_ptr: int
    a_rows: int
    lda: int
    b_ptr: int
    b_cols: int
    ldb: int
    k: int
    sub_m: int
    sub_n: int
    out_ptrs: Sequence[int]
    ldo: int
    out_rows: int
    out_cols: int
    b_kmajor: bool = False
    epi_op: int = EPI_NONE
    push_mode: int = PUSH_STORES
    rank: int = 0
    world_size: int = 1
    split_axis: int = 0
    out_mc_ptr: int = 0
    out_slot_elems: int = 0
    out_slots: int = 1
    group_m_tiles: int = 8
    sig_local: int = 0
    heap_stride: int = 0
    sig_stride: int = 0
    rot_m_tiles: int = 0
    stage_local: int = 0
    a_gate: int = 0
    a_gate_rows_per_rank: int = 0
    ag_src: int = 0
    ag_dst: int = 0
    ag_mc_dst: int = 0
    ag_bytes: int = 0
    scatter_col_begin: int = 0
    scatter_col_end: int = 0
    grid: int = 0
    status_ptr: int = 0
    stats_ptr: int = 0          # uint64[8] per-call counters (see ops.call_stats), 0 = off
    trace_ptr: int = 0
    tuning: int = -1            # -1: TILECCL_TUNING from the environment (default 1)
    rs_own_lag: int = 0         # reduce-scatter: rounds the own tile rows trail (0 = all last)
    ident_ptr: int = 0          # reduce-scatter: 128 x 128 identity of `dtype` (see identity_operand)
    wait_budget_ns: int = 0
    entry_local: int = 0        # uint32[world_size] entry-handshake counters on the heap (0 = off)
    cta_pairs: Optional[bool] = None   # kernel form of whole-order launches (None: TILECCL_GEMM_2SM)


def count_launches(n: int) -> None:
    """Launches issued by the native runtime on behalf of a plan (LAUNCH_COUNT bookkeeping)."""
    global LAUNCH_COUNT
    LAUNCH_COUNT += n


_IDENTITY = {}


def identity_operand(dtype: torch.dtype, device) -> torch.Tensor:
    """The 128 x 128 identity a reduce-scatter owner multiplies the peers' staged partial
    tiles with, so that the tensor cores add them to the accumulator (acc += I @ P)."""
    device = torch.device(device)
    key = (dtype, device.index if device.index is not None else torch.cuda.current_device())
    t = _IDENTITY.get(key)
    if t is None:
        t = _IDENTITY[key] = torch.eye(BLOCK_M, dtype=dtype, device=device).contiguous()
    return t


class FusedGemmPlan:
    def __init__(self, spec: FusedGemmSpec):
        self.spec = spec
        d = _native.GemmDesc()
        d.mode = spec.mode
        d.dtype = dtype_code(spec.dtype)
        d.b_kmajor = 1 if spec.b_kmajor else 0
        d.epi_op = spec.epi_op
        d.push_mode = spec.push_mode
        d.rank = spec.rank
        d.world_size = spec.world_size
        d.split_axis = spec.split_axis
        d.a_rows, d.b_cols, d.k = spec.a_rows, spec.b_cols, spec.k
        d.a_ptr, d.lda = spec.a_ptr, spec.lda
        d.b_ptr, d.ldb = spec.b_ptr, spec.ldb
        d.sub_m, d.sub_n = spec.sub_m, spec.sub_n
        for i, ptr in enumerate(spec.out_ptrs):
            d.out_ptr[i] = ptr
        d.out_mc_ptr = spec.out_mc_ptr
        d.ldo = spec.ldo
        d.out_rows, d.out_cols = spec.out_rows, spec.out_cols
        d.out_slot_elems, d.out_slots = spec.out_slot_elems, spec.out_slots
        d.group_m_tiles = spec.group_m_tiles
        d.sig_local, d.heap_stride, d.sig_stride = spec.sig_local, spec.heap_stride, spec.sig_stride
        d.rot_m_tiles = spec.rot_m_tiles
        d.stage_local = spec.stage_local
        d.a_gate, d.a_gate_rows_per_rank = spec.a_gate, spec.a_gate_rows_per_rank
        d.ag_src, d.ag_dst, d.ag_mc_dst, d.ag_bytes = (spec.ag_src, spec.ag_dst, spec.ag_mc_dst,
                                                       spec.ag_bytes)
        d.scatter_col_begin, d.scatter_col_end = spec.scatter_col_begin, spec.scatter_col_end
        d.grid = spec.grid
        d.status = spec.status_ptr
        d.stats = spec.stats_ptr if _config().call_stats else 0
        d.trace = spec.trace_ptr
        d.rs_own_lag = spec.rs_own_lag
        d.ident_ptr = spec.ident_ptr
        cfg = _config()
        d.tuning = spec.tuning if spec.tuning >= 0 else cfg.tuning
        pairs = cfg.gemm_cta_pairs if spec.cta_pairs is None else (spec.cta_pairs and cfg.gemm_cta_pairs)
        d.disable_cta_pairs = 0 if pairs else 1
        d.dynamic_tiles = 1 if cfg.dynamic_tiles else 0
        d.wait_budget_ns = spec.wait_budget_ns
        d.entry_local = spec.entry_local
        handle = C.c_void_p()
        _native.call("tccl_gemm_plan_create", C.byref(d), C.byref(handle))
        self._handle = handle
        self._launch_fn = getattr(_native.load(), "tccl_gemm_plan_launch")
        info = _native.GemmPlanInfo()
        _native.call("tccl_gemm_plan_info", self._handle, C.byref(info))
        self.grid = info.grid
        self.tiles_total = info.tiles_total
        self.tiles_per_owner = info.tiles_per_owner
        self.owners = max(1, info.tiles_total // max(1, info.tiles_per_owner))
        self.m_tiles_local = info.m_tiles_local
        self.n_tiles_local = info.n_tiles_local
        self.groups = info.groups
        self.k_blocks = info.k_blocks
        self.smem_bytes = info.smem_bytes
        self.push_grid = info.push_grid
        self.pair_kernel = bool(info.pair_kernel)
        self.pair_grid = info.pair_grid
        self.trace_words = info.trace_words

    def launch(self, *, epoch: int = 1, a_gate_target: int = 0, tile_begin: int = 0,
               tile_end: int = -1, wait_incoming: bool = False, ag_push: bool = False,
               announce_entry: bool = True,
               stream: Optional[torch.cuda.Stream] = None) -> None:
        global LAUNCH_COUNT
        s = stream if stream is not None else torch.cuda.current_stream()
        LAUNCH_COUNT += 1
        rc = self._launch_fn(self._handle, epoch & 0xFFFFFFFF, a_gate_target & 0xFFFFFFFF,
                             tile_begin, tile_end,
                             (1 if wait_incoming else 0) | (2 if ag_push else 0)
                             | (8 if announce_entry else 0), s.cuda_stream)
        if rc != 0:
            _native.check("tccl_gemm_plan_launch", rc)

    def group_m_count(self, g: int) -> int:
        left = self.m_tiles_local - g * self.spec.group_m_tiles
        return min(left, self.spec.group_m_tiles)

    def close(self) -> None:
        if getattr(self, "_handle", None):
            _native.call("tccl_gemm_plan_destroy", self._handle)
            self._handle = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass


@dataclass
class PlanCache:
    """Keyed store of live plans (key = every address and extent the plan bakes in)."""

    max_entries: int = 256
    _plans: dict = field(default_factory=dict)

    def get(self, key, factory):
        plan = self._plans.get(key)
        if plan is None:
            if len(self._plans) >= self.max_entries:
                old_key = next(iter(self._plans))
                self._plans.pop(old_key).close()
            plan = factory()
            self._plans[key] = plan
        return plan

    def clear(self) -> None:
        for plan in self._plans.values():
            plan.close()
        self._plans.clear()


_GEMM_CACHE = PlanCache()


def _check_operand(name: str, t: torch.Tensor) -> None:
    if t.dim() != 2:
        raise ValueError(f"{name} must be 2-D, got shape {tuple(t.shape)}")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.stride(1) != 1:
        raise ValueError(f"{name} must be row-major with unit column stride")


def gemm(A: torch.Tensor, B: torch.Tensor, C: Optional[torch.Tensor] = None, *,
         b_is_nk: bool = False, epilogue: str = "none",
         stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """``C = A @ B`` on the tcgen05 path (fp16 / bf16 in, fp32 accumulate).

    ``B`` is ``[K, N]`` row-major, or ``[N, K]`` row-major when ``b_is_nk``.
    ``epilogue="silu_gate"`` treats every 256-column tile of the product as
    128 gate columns followed by 128 up columns and writes
    ``silu(gate) * up`` (so ``C`` has ``N / 2`` columns).

    Counterpart of ``tileccl.kernels.gemm.gemm`` (tileccl/kernels/gemm.py:174).
    """
    _check_operand("A", A)
    _check_operand("B", B)
    if A.dtype != B.dtype:
        raise TypeError(f"A and B must share a dtype, got {A.dtype} and {B.dtype}")
    M, K = A.shape
    if b_is_nk:
        N, Kb = B.shape
    else:
        Kb, N = B.shape
    if K != Kb:
        raise ValueError(f"inner dimensions differ: A is {tuple(A.shape)}, B is {tuple(B.shape)}")
    epi = {"none": EPI_NONE, "silu_gate": EPI_SILU_GATE}[epilogue]
    n_out = N // 2 if epi == EPI_SILU_GATE else N
    if C is None:
        C = torch.empty((M, n_out), dtype=A.dtype, device=A.device)
    _check_operand("C", C)
    if tuple(C.shape) != (M, n_out) or C.dtype != A.dtype:
        raise ValueError(f"C must be {(M, n_out)} {A.dtype}, got {tuple(C.shape)} {C.dtype}")
    key = ("gemm", A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, A.stride(0), B.stride(0),
           C.stride(0), A.dtype, b_is_nk, epi, A.device.index)

    def make():
        return FusedGemmPlan(FusedGemmSpec(
            mode=MODE_GEMM, dtype=A.dtype, a_ptr=A.data_ptr(), a_rows=M, lda=A.stride(0),
            b_ptr=B.data_ptr(), b_cols=N, ldb=B.stride(0), k=K, sub_m=M, sub_n=N,
            out_ptrs=[C.data_ptr()], ldo=C.stride(0), out_rows=M, out_cols=n_out,
            b_kmajor=b_is_nk, epi_op=epi))

    with torch.cuda.device(A.device):
        plan = _GEMM_CACHE.get(key, make)
        plan.launch(stream=stream)
    return C
