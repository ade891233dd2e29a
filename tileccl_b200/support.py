"""Runtime support matrix: what works in the current context and why.

Same shape as the reference's matrix (tileccl/support.py:25-401):
``SupportStatus(state, detail)`` entries grouped into ops / contracts /
execution_paths / collectives / memory plus a ``runtime_surface`` summary.  The
entries are derived from capability queries (GPU present? compute capability
10.x? heap attached, which transport, NVLS bound?) instead of being written out
by hand per release.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from .utils.feature_gates import (multiprocess_device_remote_access_detail,
                                  multiprocess_device_remote_access_runtime_supported,
                                  multiprocess_device_validated_public_surface)

SUPPORTED, PARTIAL, UNSUPPORTED = "supported", "partial", "unsupported"


@dataclass(frozen=True)
class SupportStatus:
    state: str
    detail: str

    def __post_init__(self) -> None:
        if self.state not in (SUPPORTED, PARTIAL, UNSUPPORTED):
            raise ValueError(f"state must be supported / partial / unsupported, got {self.state!r}")

    def to_dict(self) -> dict:
        return {"state": self.state, "detail": self.detail}


@dataclass(frozen=True)
class RuntimeSupportMatrix:
    backend: str
    device: str
    rank: int
    world_size: int
    has_heap: bool
    heap_mode: Optional[str]
    transport_strategy: Optional[str]
    runtime_surface: dict
    ops: dict
    contracts: dict
    execution_paths: dict
    collectives: dict
    memory: dict

    def to_dict(self) -> dict:
        dump = lambda table: {k: v.to_dict() for k, v in table.items()}
        return {
            "context": {"backend": self.backend, "device": self.device, "rank": self.rank,
                        "world_size": self.world_size, "has_heap": self.has_heap,
                        "heap_mode": self.heap_mode, "transport_strategy": self.transport_strategy},
            "runtime_surface": self.runtime_surface,
            "ops": dump(self.ops), "contracts": dump(self.contracts),
            "execution_paths": dump(self.execution_paths), "collectives": dump(self.collectives),
            "memory": dump(self.memory),
        }

    def summary(self) -> dict:
        counts = {SUPPORTED: 0, PARTIAL: 0, UNSUPPORTED: 0}
        for table in (self.ops, self.contracts, self.execution_paths, self.collectives, self.memory):
            for st in table.values():
                counts[st.state] += 1
        return counts


def _device_facts(ctx) -> dict:
    facts = {"gpu": False, "sm100": False, "name": None, "sms": 0, "nvls_capable": False}
    try:
        import torch

        if torch.cuda.is_available():
            props = ctx.backend.get_device_properties(torch.device(ctx.device).index or 0)
            facts.update(gpu=True, name=props.name, sms=props.compute_units,
                         sm100=props.compute_capability[0] == 10,
                         nvls_capable=props.multicast_supported)
    except Exception:
        pass
    return facts


def _native_ok() -> tuple:
    try:
        from . import _native

        _native.load()
        return True, f"libtileccl_b200 {_native.version()} loaded"
    except Exception as exc:
        return False, f"native library unavailable: {exc}"


def describe_runtime_support(ctx: Any = None) -> RuntimeSupportMatrix:
    if ctx is None:
        from . import current_context

        ctx = current_context()
    heap = ctx.heap
    has_heap = heap is not None
    heap_mode = heap.mode if has_heap else None
    transport = heap.transport_strategy if has_heap else None
    ws = ctx.world_size
    dev = _device_facts(ctx)
    native, native_detail = _native_ok()

    def gate(needs_heap: bool, what: str) -> SupportStatus:
        if not native:
            return SupportStatus(UNSUPPORTED, native_detail)
        if not dev["gpu"]:
            return SupportStatus(UNSUPPORTED, "no CUDA device visible")
        if not dev["sm100"]:
            return SupportStatus(UNSUPPORTED,
                                 f"{dev['name']} is not compute capability 10.x; kernels are sm_100a only")
        if needs_heap and ws > 1 and not has_heap:
            return SupportStatus(UNSUPPORTED, "world_size > 1 needs a symmetric heap (init(heap_size=...))")
        if needs_heap and ws > 1 and not multiprocess_device_remote_access_runtime_supported(
                transport_strategy=transport, world_size=ws):
            return SupportStatus(PARTIAL, multiprocess_device_remote_access_detail(
                transport_strategy=transport, world_size=ws, operation=what))
        return SupportStatus(SUPPORTED, f"{what}: sm_100a kernel, world_size {ws}"
                             + (f", {transport}" if transport else ""))

    fused = gate(True, "fused tcgen05 GEMM + collective")
    coll = gate(True, "tile collective kernel")
    ops = {
        "gemm_allscatter": fused, "gemm_allscatter_sharded": fused, "gemm_allgather": fused,
        "gemm_allgather_rows": fused, "gemm_reducescatter": fused, "gemm_reducescatter_rows": fused,
        "allgather_gemm_reducescatter": fused, "allgather": coll, "allreduce": coll,
        "reduce_scatter": coll, "broadcast": coll, "scatter": coll,
        "models.TPMLP": fused,
    }
    contracts = {
        "gemm_allscatter.full/full": fused,
        "gemm_allscatter.shard/shard": SupportStatus(
            PARTIAL if fused.state == SUPPORTED else fused.state,
            "every rank writes its shard over the peers' shard buffers (last writer wins), as in "
            "the reference; prefer gemm_allgather for a defined result"),
        "gemm_allscatter.full/shard": fused,
        "gemm_allscatter.shard/full": SupportStatus(UNSUPPORTED, "use ops.gemm_allgather"),
        "gemm_allgather.columns": fused, "gemm_allgather.rows": fused,
        "gemm_reducescatter.columns": fused, "gemm_reducescatter.rows": fused,
        "allreduce.in_place": coll,
        "dtypes.fp16_bf16_gemm": fused,
        "dtypes.fp32_gemm": SupportStatus(UNSUPPORTED, "the tcgen05 path takes fp16 / bf16 operands"),
        "dtypes.collectives_fp16_bf16_fp32": coll,
    }
    nvls = bool(has_heap and heap.has_multicast)
    execution_paths = {
        "pattern.bulk_sync": fused, "pattern.fused_sequential": fused,
        "pattern.producer_consumer": fused, "pattern.wg_specialized": fused,
        "push.stores": fused, "push.tma": fused,
        "push.multimem": (fused if nvls else SupportStatus(
            UNSUPPORTED, "no NVLS multicast mapping bound to the heap"
            + ("" if dev["nvls_capable"] else " (device reports no multicast support)"))),
        "single_process.distinct_gpus": fused,
        "single_process.emulated_ranks": SupportStatus(
            fused.state, "ranks sharing one GPU run phase by phase (no in-kernel peer waits)"),
        "multiprocess.vmm_fd": fused,
        "multiprocess.vmm_fabric": SupportStatus(UNSUPPORTED, "fabric handles need an IMEX domain"),
        "cpu_emulation": SupportStatus(SUPPORTED if native else UNSUPPORTED,
                                       "thread-per-rank CPU executor of the TileGroup schedule"),
    }
    collectives = {f"collectives.{n}_launcher": coll
                   for n in ("allgather", "allreduce", "reduce_scatter", "broadcast", "scatter")}
    collectives["collectives.nvls"] = (coll if nvls else SupportStatus(
        PARTIAL if coll.state == SUPPORTED else coll.state, "NVLS not bound: peer load/store paths are used"))
    collectives["collectives.ops_other_than_sum"] = SupportStatus(UNSUPPORTED, "only op='sum'")
    collectives["collectives.device_functions"] = SupportStatus(
        SUPPORTED, "tile_allreduce / tile_allgather / tile_reduce_scatter / tile_broadcast / "
                   "tile_scatter are __device__ functions (csrc/device/tile_collectives.cuh); user "
                   "kernels are built and launched with tileccl_b200.userkernel")
    collectives["collectives.low_latency"] = SupportStatus(
        coll.state, "all five collectives travel as flag-in-data lines up to TILECCL_LL_MAX_BYTES "
                    "(default 1 MiB) per peer (csrc/device/tile_ll.cuh)")
    collectives["collectives.relay_broadcast"] = SupportStatus(
        coll.state if ws >= 3 or not has_heap else PARTIAL,
        "broadcasts from TILECCL_BCAST_RELAY_MIN_BYTES (default 256 MiB) on three or more ranks are "
        "relayed piece by piece: the root sends every byte once")
    from . import _build

    collectives["debug.recorded_bounds_checks"] = SupportStatus(
        SUPPORTED if _build.DEBUG_LIB_PATH.exists() else PARTIAL,
        "TILECCL_DEBUG=1 loads libtileccl_b200_debug.so (python -m tileccl_b200._build --debug): "
        "device-side bounds checks that record and skip, epoch invariants after every call")
    mem_ok = SupportStatus(SUPPORTED if has_heap else UNSUPPORTED,
                           f"cuMem VMM heap, mode {heap_mode}, transport {transport}" if has_heap
                           else "no heap attached")
    memory = {
        "symmetric_heap.current_runtime": mem_ok,
        "symmetric_heap.device_remote_access": mem_ok if ws == 1 or not has_heap else SupportStatus(
            SUPPORTED if multiprocess_device_remote_access_runtime_supported(
                transport_strategy=transport, world_size=ws) else PARTIAL,
            multiprocess_device_remote_access_detail(transport_strategy=transport, world_size=ws)),
        "symmetric_heap.nvls_multicast": SupportStatus(
            SUPPORTED if nvls else UNSUPPORTED,
            "multicast alias bound" if nvls else "not bound (single rank, shared GPUs, or unsupported)"),
        "symmetric_heap.external_import": SupportStatus(SUPPORTED if has_heap else UNSUPPORTED,
                                                        "as_symmetric() copies into the heap"),
        "symmetric_heap.external_mapping": SupportStatus(UNSUPPORTED, "no zero-copy adoption of foreign memory"),
        "symmetric_heap.fd_passing": SupportStatus(SUPPORTED, "POSIX fd handles over Unix sockets"),
        "symmetric_heap.segment_metadata": mem_ok,
        "symmetric_heap.peer_mapping_metadata": mem_ok,
    }
    surface = {
        "policy": "capability_derived",
        "validated_public_surface": multiprocess_device_validated_public_surface(),
        "current_runtime": {"world_size": ws, "heap_mode": heap_mode, "transport_strategy": transport,
                            "nvls_bound": nvls, "device": dev},
        "in_validated_public_surface": bool(ws == 1 or (has_heap and
            multiprocess_device_remote_access_runtime_supported(transport_strategy=transport,
                                                                world_size=ws))),
        "native": native_detail,
    }
    return RuntimeSupportMatrix(ctx.backend_name, ctx.device, ctx.rank, ws, has_heap, heap_mode,
                                transport, surface, ops, contracts, execution_paths, collectives,
                                memory)
