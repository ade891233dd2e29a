"""Host launchers of the tile collectives (``csrc/kernels/collectives.cu``).

Same entry points as the reference (tileccl/primitives/collectives.py:1882-2632):
``allreduce``, ``allgather``, ``broadcast``, ``scatter``, ``reduce_scatter``,
``resolve_allreduce_execution`` / ``AllReduceExecutionSpec``.  Buffers live on the
symmetric heap; no NCCL call is made.

Algorithms (all direct, one NVLink hop, any world size 1..8):

=============== =========================================================
all-gather      push own chunk into every rank's output (multimem.st if NVLS)
reduce-scatter  pull own chunk from every rank and sum in fp32
                (multimem.ld_reduce if NVLS); chunks up to 64 KiB: every rank
                sends chunk d to rank d as flag-in-data lines, the owner sums
all-reduce      small (up to 1 MiB at two to four ranks, 512 KiB at eight): one-shot over
                flag-in-data lines; <= 256 KiB otherwise: one-shot through a
                double-buffered staging copy; larger: pull-reduce own chunk, push
                it to every rank
broadcast       root pushes to everyone (multimem.st if NVLS); from 256 MiB on three or
                more ranks: pipelined relay (root sends every byte once, to the other
                ranks in turn, and each forwards its pieces to the rest)
scatter         root pushes chunk r to rank r
=============== =========================================================
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Optional

import torch

from .. import _native
from ..utils.config import current as _config
from ..utils.config import generation as _config_generation
from ..kernels.fused_gemm import STATUS_WORDS, raise_on_status

OP_ALLGATHER = 0
OP_REDUCE_SCATTER = 1
OP_ALLREDUCE_TWO_SHOT = 2
OP_ALLREDUCE_ONE_SHOT = 3
OP_BROADCAST = 4
OP_SCATTER = 5

_DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
_COUNTER_WORDS = 32
_THREADS = 512
MAX_WORLD_SIZE = 8

# Message regimes of the all-reduce policy (bytes).
LATENCY_MAX_BYTES = 8 * 1024
ONE_SHOT_MAX_BYTES = 256 * 1024


@dataclass(frozen=True)
class AllReduceExecutionSpec:
    """How one all-reduce call will run; part of ``AllReducePlan.to_dict()``."""

    implementation: str       # "noop" | "device_one_shot" | "device_two_shot"
    protocol: str             # "local_identity" | "staged_snapshot_epoch" | "pull_reduce_push_epoch"
    kernel_family: str        # "local_identity" | "generic_multi_peer"
    message_regime: str       # "latency" | "throughput" | "bandwidth"
    message_bytes: int
    chunk_elems: int          # elements each rank reduces (two-shot) or the whole message (one-shot)
    num_chunks: int
    pipeline_slots: int       # staging parities (one-shot) / 1
    grid_size: int
    num_warps: int
    workspace_bytes: int
    reuse_handshake: str      # "epoch_parity_double_buffer" | "completion_counter" | "none"
    cta_policy: str
    epoch_policy: str
    use_multimem: bool

    def to_dict(self) -> dict:
        return asdict(self)


# --------------------------------------------------------------------------
# per-heap state
# --------------------------------------------------------------------------
_SM_COUNT: dict = {}


def _sm_count(device: torch.device) -> int:
    n = _SM_COUNT.get(device)
    if n is None:
        n = _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_ptr(device_index: int) -> int:
    """Handle of the current stream of ``device_index`` (the cheap way when torch has it)."""
    if _raw_stream is not None:
        return _raw_stream(device_index)
    return torch.cuda.current_stream(device_index).cuda_stream


# --------------------------------------------------------------------------
# Repeat calls.  A call on buffers that were seen before (same addresses, sizes, dtype,
# root, and the same configuration snapshot) skips validation and policy and re-issues the
# launch through a closure that has everything resolved: for small messages the host side of
# a call is as long as the device side.  One-process-per-GPU heaps only (emulated ranks
# replay phases through `_run`), never in debug mode (which checks every call).
# --------------------------------------------------------------------------
_FAST_MAX = 4096


def _fast_key(kind: str, a: torch.Tensor, b: Optional[torch.Tensor], root: int) -> tuple:
    if b is None:
        return (kind, a.data_ptr(), a.numel(), a.dtype, a.is_contiguous(), root,
                _config_generation())
    return (kind, a.data_ptr(), b.data_ptr(), a.numel(), b.numel(), a.dtype, b.dtype,
            a.is_contiguous() and b.is_contiguous(), root, _config_generation())


def try_fast(heap, kind: str, a: torch.Tensor, b: Optional[torch.Tensor] = None,
             root: int = 0) -> bool:
    """Re-issue a remembered launch; False when this call has to take the full path."""
    table = heap._state.get("coll_fast")
    if not table:
        return False
    fn = table.get(_fast_key(kind, a, b, root))
    if fn is None:
        return False
    fn()
    return True


def _remember(heap, kind: str, a, b, root: int, relaunch) -> None:
    if relaunch is None:
        return
    table = heap._state.setdefault("coll_fast", {})
    if len(table) >= _FAST_MAX:
        table.clear()
    table[_fast_key(kind, a, b, root)] = relaunch


def _counters(heap, kind: str) -> dict:
    st = heap._state.setdefault(("coll", kind), None)
    if st is None:
        st = {"counters": heap.allocate_signal_buffer(_COUNTER_WORDS), "epoch": 0}
        heap._state[("coll", kind)] = st
    return st


def _status(heap) -> torch.Tensor:
    st = heap._state.get("status")
    if st is None:
        st = torch.zeros(STATUS_WORDS, dtype=torch.int32, device=heap.device)
        heap._state["status"] = st
    return st


def check_status(heap) -> None:
    """Synchronise and raise if a collective kernel gave up waiting for a peer."""
    st = heap._state.get("status")
    if st is not None:
        torch.cuda.synchronize(heap.device)
        raise_on_status(st)


def _budget_ns() -> int:
    return _config().wait_budget_ns


def _grid_for(nbytes: int, device: torch.device) -> int:
    vecs = max(1, nbytes // 16)
    return max(1, min(_sm_count(device), -(-vecs // (_THREADS * 2))))


# Total message size from which the plain peer path replaces NVLS (bytes; measured at 8 ranks).
# A multicast store or a switch-side reduction also moves the caller's own share through the
# switch (1 / world_size of the traffic on the link for nothing), which costs more than the
# saved instructions once a call is bandwidth-bound; the all-reduce keeps NVLS at every size
# (one multimem.ld_reduce + one multimem.st per 16 bytes instead of 2 (n - 1) accesses).
NVLS_MAX_TOTAL_BYTES = {"allgather": 16 << 20, "reduce_scatter": 128 << 20}


def _use_multimem(heap, nbytes: int, kind: str = "") -> bool:
    """NVLS (multimem) path?  With two ranks a multicast store also loops the data back
    to the sender through the switch and measures slower than plain peer stores
    (about 500 vs 700 GB/s), so the default is NVLS only from three ranks on, and for
    all-gather / reduce-scatter only below ``NVLS_MAX_TOTAL_BYTES``;
    ``TILECCL_FORCE_NVLS=1`` uses it whenever it is bound, ``TILECCL_DISABLE_NVLS=1`` never.
    ``nbytes`` is the per-rank chunk for all-gather / reduce-scatter."""
    cfg = _config()
    if not heap.has_multicast or cfg.disable_nvls:
        return False
    if nbytes % 16 != 0 or nbytes < 16:
        return False
    if cfg.force_nvls:
        return True
    if heap.world_size <= 2:
        return False
    limit = NVLS_MAX_TOTAL_BYTES.get(kind)
    return limit is None or nbytes * heap.world_size < limit


def _validate(name: str, t: torch.Tensor, heap) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if heap.world_size > MAX_WORLD_SIZE:
        raise ValueError(f"world_size {heap.world_size} exceeds the supported maximum {MAX_WORLD_SIZE}")
    if heap.world_size > 1 and not heap.owns_tensor(t):
        raise ValueError(f"{name} must live on the symmetric heap of rank {heap.rank}")
    if t.data_ptr() % 16:
        raise ValueError(f"{name} must be 16-byte aligned")


def _run(heap, key, phases) -> None:
    """Launch now, or (emulated ranks) park until all ranks have called and replay by phase."""
    group = heap.local_group
    if group is None or not group.emulated or heap.world_size == 1:
        for ph in phases:
            ph()
        return
    slot = group.pending.setdefault(key, {})
    if heap.rank in slot:
        raise RuntimeError(f"rank {heap.rank} entered collective {key[0]!r} twice before its peers")
    slot[heap.rank] = phases
    if len(slot) < heap.world_size:
        return
    del group.pending[key]
    for i in range(max(len(p) for p in slot.values())):
        for r in range(heap.world_size):
            if i < len(slot[r]):
                slot[r][i]()


def _launch(heap, kind: str, op: int, dtype_code: int, src: int, dst: int, nbytes: int, *,
            elem_size: int, root: int = 0, staging: int = 0, stage_slot: int = 0,
            use_multimem: bool = False, grid: Optional[int] = None, rv_extra=()):
    """Launch one call; returns a closure that repeats it (next epoch, same arguments) on a
    one-process-per-GPU heap, else None."""
    st = _counters(heap, kind)
    grid = grid or _grid_for(nbytes, heap.device)
    if "status_ptr" not in st:
        st["status_ptr"] = _status(heap).data_ptr()
        st["counters_ptr"] = st["counters"].data_ptr()
        st["fn"] = getattr(_native.load(), "tccl_collective_launch")
    status, counters = st["status_ptr"], st["counters_ptr"]
    if not heap.emulated and heap.local_group is None:
        # One process per GPU: a single launch with all three phases, on the current stream
        # of the current device (the heap's device).  This is the latency path: no device
        # switch, everything but the epoch and the stream resolved once.
        fn, rank, ws, mc = st["fn"], heap.rank, heap.world_size, 1 if use_multimem else 0
        mc_base, local_base, stride = heap.multicast_base, heap.local_base, heap.stride
        budget, dev_index = _budget_ns(), heap.device.index

        def relaunch():
            st["epoch"] = e = st["epoch"] + 1
            rc = fn(op, dtype_code, rank, ws, root, mc, 7, elem_size, e & 0xFFFFFFFF, src, dst,
                    staging, stage_slot, counters, mc_base, local_base, stride, nbytes, grid,
                    status, budget, _stream_ptr(dev_index))
            if rc != 0:
                _native.check("tccl_collective_launch", rc)

        relaunch()
        if _config().debug:
            if op != OP_ALLREDUCE_ONE_SHOT:
                from .. import debug as _debug

                _debug.after_collective(heap, st, st["epoch"],
                                        root=root if op in (OP_BROADCAST, OP_SCATTER) else None)
            return None
        return relaunch

    st["epoch"] += 1
    epoch = st["epoch"]

    def make(mask: int):
        def go():
            with torch.cuda.device(heap.device):
                _native.call(
                    "tccl_collective_launch", op, dtype_code, heap.rank, heap.world_size, root,
                    1 if use_multimem else 0, mask, elem_size, epoch & 0xFFFFFFFF, src, dst, staging,
                    stage_slot, counters,
                    heap.multicast_base, heap.local_base, heap.stride, nbytes, grid, status,
                    _budget_ns(), torch.cuda.current_stream().cuda_stream)
        return go

    if heap.emulated and heap.world_size > 1:
        phases = [make(1), make(2), make(4)] if op != OP_ALLREDUCE_ONE_SHOT else [make(1), make(2)]
    else:
        phases = [make(7)]
    _run(heap, (kind, nbytes, epoch) + tuple(rv_extra), phases)
    return None


LL_MIN_SLOT_BYTES = 128 * 1024  # staging per (parity, source): 64 KiB of payload as 16-byte lines
LL_MAX_BYTES = 1024 * 1024      # what the kernel accepts; the policy limit is RuntimeConfig.ll_max_bytes


def ll_slot_bytes(per_peer_bytes: int) -> int:
    """Staging slot of the message class of ``per_peer_bytes``: two bytes of staging per
    payload byte, sized for the next power of two so that neighbouring sizes share staging."""
    cls = 1 << max(0, (max(1, per_peer_bytes) - 1).bit_length())
    return max(LL_MIN_SLOT_BYTES, 2 * cls)


def _ll_ok(heap, per_peer_bytes: int, *ptrs: int) -> bool:
    """Low-latency path?  Small per-peer messages that are multiples of 8 bytes."""
    limit = min(LL_MAX_BYTES, _config().ll_max_bytes)
    return (heap.world_size > 1 and 0 < per_peer_bytes <= limit and per_peer_bytes % 8 == 0
            and all(p % 8 == 0 for p in ptrs))


LL_ALLREDUCE_MAX_INGRESS = 4 << 20   # payload bytes a rank receives in a low-latency all-reduce


def _ll_allreduce_ok(heap, nbytes: int, ptr: int) -> bool:
    """One-shot all-reduce over flag-in-data lines?  Every rank receives the whole vector
    from every peer (twice the bytes on the wire), which pays while that stays small."""
    return (_ll_ok(heap, nbytes, ptr)
            and nbytes * (heap.world_size - 1) <= LL_ALLREDUCE_MAX_INGRESS)


def _launch_ll(heap, kind: str, op: int, src: int, dst: int, per_peer_bytes: int, *,
               root: int = 0, dtype_code: int = 3):
    """One low-latency copy collective (``ll_copy_kernel``): payload and flag share a store.
    Returns a closure that repeats the call (see ``_launch``) or None."""
    slot_bytes = ll_slot_bytes(per_peer_bytes)
    st = heap._state.get(("coll_ll", kind, slot_bytes))
    if st is None:
        slots = heap.world_size if op in (OP_ALLGATHER, OP_REDUCE_SCATTER,
                                           OP_ALLREDUCE_ONE_SHOT) else 1
        st = {"stage": heap.allocate_zeroed((2 * slots * slot_bytes,), torch.uint8),
              "counters": heap.allocate_signal_buffer(_COUNTER_WORDS), "epoch": 0,
              "status_ptr": _status(heap).data_ptr(), "fn": getattr(_native.load(),
                                                                   "tccl_collective_ll_launch")}
        st["stage_ptr"], st["counters_ptr"] = st["stage"].data_ptr(), st["counters"].data_ptr()
        heap._state[("coll_ll", kind, slot_bytes)] = st
    lines = per_peer_bytes // 8 * (heap.world_size - 1)      # lines this rank sends or receives
    grid = max(1, min(8 if per_peer_bytes <= 65536 else 64, lines // 2048))
    if not heap.emulated and heap.local_group is None:
        fn, rank, ws, stride = st["fn"], heap.rank, heap.world_size, heap.stride
        stage_ptr, counters_ptr, status = st["stage_ptr"], st["counters_ptr"], st["status_ptr"]
        budget, dev_index = _budget_ns(), heap.device.index

        def relaunch():
            st["epoch"] = e = st["epoch"] + 1
            rc = fn(op, dtype_code, rank, ws, root, 3, e & 0xFFFFFFFF, src, dst, stage_ptr,
                    counters_ptr, stride, per_peer_bytes, slot_bytes, grid, status, budget,
                    _stream_ptr(dev_index))
            if rc != 0:
                _native.check("tccl_collective_ll_launch", rc)

        relaunch()
        return None if _config().debug else relaunch

    st["epoch"] += 1
    epoch = st["epoch"]

    def go(mask: int):
        rc = st["fn"](op, dtype_code, heap.rank, heap.world_size, root, mask, epoch & 0xFFFFFFFF,
                      src, dst, st["stage_ptr"], st["counters_ptr"], heap.stride, per_peer_bytes,
                      slot_bytes, grid,
                      st["status_ptr"], _budget_ns(), torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            _native.check("tccl_collective_ll_launch", rc)

    def on_dev(mask):
        def run():
            with torch.cuda.device(heap.device):
                go(mask)
        return run

    phases = [on_dev(1), on_dev(2)] if heap.emulated else [on_dev(3)]
    _run(heap, ("ll:" + kind, per_peer_bytes, slot_bytes, epoch, root), phases)
    return None


RELAY_MAX_PIECES = 16384
RELAY_MIN_PIECE = 16 * 1024


def relay_piece_bytes(nbytes: int, max_piece: int = 64 * 1024, bulk: bool = False) -> int:
    """Piece size of the relay broadcast.  A piece is the unit of pipelining: a relay can
    forward a piece only when all of it has arrived, so the relays start one piece time after
    the root and finish one piece time after it.  Every piece also costs its sender a
    system-scope fence.  Register-copy form (the default): about 2048 pieces per message, at
    least 16 KiB each (a CTA-wide fence per piece wants few, large pieces).  Bulk-copy form:
    about 1024 pieces between 16 KiB and ``max_piece`` (a fence per pipeline), larger only
    where the piece count would exceed the flag block (16384).  Multiples of 8 KiB."""
    if bulk:
        piece = min(max(RELAY_MIN_PIECE, -(-nbytes // 1024)), max(RELAY_MIN_PIECE, max_piece))
        piece = max(piece, -(-nbytes // RELAY_MAX_PIECES))
    else:
        piece = max(RELAY_MIN_PIECE, -(-nbytes // 2048))
    return -(-piece // 8192) * 8192


def _relay_ok(heap, nbytes: int, ptr: int) -> bool:
    limit = _config().bcast_relay_min_bytes
    return (heap.world_size >= 3 and limit > 0 and nbytes >= limit and nbytes % 16 == 0
            and ptr % 16 == 0)


def _launch_relay(heap, root: int, ptr: int, nbytes: int):
    """Large broadcast as a pipelined relay (``broadcast_relay_kernel``).  Returns a closure
    that repeats the call (see ``_launch``) or None."""
    kind = f"broadcast_relay:{root}"
    st = heap._state.get(("coll_relay", kind))
    if st is None:
        st = {"flags": heap.allocate_signal_buffer(RELAY_MAX_PIECES),
              "counters": heap.allocate_signal_buffer(_COUNTER_WORDS), "epoch": 0,
              "status_ptr": _status(heap).data_ptr(),
              "fn": getattr(_native.load(), "tccl_broadcast_relay_launch")}
        st["flags_ptr"], st["counters_ptr"] = st["flags"].data_ptr(), st["counters"].data_ptr()
        heap._state[("coll_relay", kind)] = st
    cfg = _config()
    piece = relay_piece_bytes(nbytes, cfg.bcast_relay_piece_kib * 1024, cfg.bcast_relay_bulk)
    n_pieces = -(-nbytes // piece)
    # The root's workers take pieces in turn; a relay owns every (ws - 1)-th piece.  The root
    # runs few workers: the link is shared by the pieces in flight, so with fewer of them each
    # piece completes sooner and the relays idle less at the start and at the end (148
    # pipelines with two 16 KiB slots each still keep well over the 2 MB in flight that the
    # link needs).  A relay runs as many as it has pieces for.
    own = n_pieces if heap.rank == root else -(-n_pieces // (heap.world_size - 1))
    bulk = 1 if cfg.bcast_relay_bulk else 0
    workers_per_cta = 4 if bulk else 1               # the bulk form runs four pipelines per CTA
    if heap.rank == root:
        own = min(own, cfg.bcast_relay_root_workers)
    grid = max(1, min(_sm_count(heap.device) * cfg.bcast_relay_ctas_per_sm,
                      -(-own // workers_per_cta)))
    if not heap.emulated and heap.local_group is None:
        fn, rank, ws = st["fn"], heap.rank, heap.world_size
        flags_ptr, counters_ptr, status = st["flags_ptr"], st["counters_ptr"], st["status_ptr"]
        local_base, stride = heap.local_base, heap.stride
        budget, dev_index = _budget_ns(), heap.device.index

        def relaunch():
            st["epoch"] = e = st["epoch"] + 1
            rc = fn(rank, ws, root, 15, e & 0xFFFFFFFF, ptr, nbytes, piece, flags_ptr,
                    counters_ptr, local_base, stride, grid, bulk, status, budget,
                    _stream_ptr(dev_index))
            if rc != 0:
                _native.check("tccl_broadcast_relay_launch", rc)

        relaunch()
        if _config().debug:
            from .. import debug as _debug

            _debug.after_collective(heap, st, st["epoch"])
            return None
        return relaunch

    st["epoch"] += 1
    epoch = st["epoch"]

    def go(mask: int):
        rc = st["fn"](heap.rank, heap.world_size, root, mask, epoch & 0xFFFFFFFF, ptr, nbytes,
                      piece, st["flags_ptr"], st["counters_ptr"], heap.local_base, heap.stride,
                      grid, bulk, st["status_ptr"], _budget_ns(),
                      torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            _native.check("tccl_broadcast_relay_launch", rc)

    def on_dev(mask):
        def run():
            with torch.cuda.device(heap.device):
                go(mask)
        return run

    phases = [on_dev(1), on_dev(2), on_dev(8), on_dev(4)] if heap.emulated else [on_dev(15)]
    _run(heap, (kind, nbytes, epoch, root), phases)
    return None


def _heap_of(heap, ctx):
    if heap is None and ctx is not None:
        heap = ctx.heap
    if heap is None:
        raise ValueError("a symmetric heap is required")
    return heap


# --------------------------------------------------------------------------
# launchers
# --------------------------------------------------------------------------
def resolve_allreduce_execution(tensor: torch.Tensor, *, heap, op: str = "sum",
                                ctx=None) -> AllReduceExecutionSpec:
    heap = _heap_of(heap, ctx)
    if op != "sum":
        raise ValueError(f"only op='sum' is supported, got {op!r}")
    if tensor.dtype not in _DTYPE_CODE:
        raise TypeError(f"allreduce supports float16, bfloat16 and float32, got {tensor.dtype}")
    nbytes = tensor.numel() * tensor.element_size()
    ws = heap.world_size
    regime = ("latency" if nbytes <= LATENCY_MAX_BYTES
              else "throughput" if nbytes <= ONE_SHOT_MAX_BYTES else "bandwidth")
    if ws == 1:
        return AllReduceExecutionSpec("noop", "local_identity", "local_identity", regime, nbytes,
                                      tensor.numel(), 1, 1, 0, 0, 0, "none", "none", "none", False)
    grid = _grid_for(nbytes, heap.device) if tensor.is_cuda else 1
    if _ll_allreduce_ok(heap, nbytes, tensor.data_ptr()):
        return AllReduceExecutionSpec(
            "device_one_shot_ll", "flag_in_data_parity_ack", "generic_multi_peer", regime, nbytes,
            tensor.numel(), 1, 2, max(1, min(64, nbytes // 8 * (ws - 1) // 2048)), _THREADS // 32,
            2 * ws * ll_slot_bytes(nbytes) + 4 * _COUNTER_WORDS, "epoch_parity_double_buffer",
            "grid_stride_multi_cta", "monotonic_counter", False)
    if nbytes <= ONE_SHOT_MAX_BYTES:
        slot = (nbytes + 15) // 16 * 16
        return AllReduceExecutionSpec(
            "device_one_shot", "staged_snapshot_epoch", "generic_multi_peer", regime, nbytes,
            tensor.numel(), 1, 2, grid, _THREADS // 32, 2 * slot + 4 * _COUNTER_WORDS,
            "epoch_parity_double_buffer", "grid_stride_multi_cta", "monotonic_counter", False)
    chunk_bytes = (-(-nbytes // ws) + 15) // 16 * 16
    return AllReduceExecutionSpec(
        "device_two_shot", "pull_reduce_push_epoch", "generic_multi_peer", regime, nbytes,
        chunk_bytes // tensor.element_size(), ws, 1, grid, _THREADS // 32, 4 * _COUNTER_WORDS,
        "completion_counter", "grid_stride_multi_cta", "monotonic_counter",
        _use_multimem(heap, chunk_bytes))


def allreduce(tensor: torch.Tensor, heap=None, op: str = "sum", *, ctx=None,
              _execution: Optional[AllReduceExecutionSpec] = None) -> torch.Tensor:
    """In-place sum of ``tensor`` over all ranks."""
    heap = _heap_of(heap, ctx)
    if op == "sum" and try_fast(heap, "allreduce", tensor):
        return tensor
    _validate("tensor", tensor, heap)
    ex = _execution or resolve_allreduce_execution(tensor, heap=heap, op=op)
    if ex.implementation == "noop":
        return tensor
    nbytes = ex.message_bytes
    code = _DTYPE_CODE[tensor.dtype]
    ptr = tensor.data_ptr()
    if ex.implementation == "device_one_shot_ll":
        again = _launch_ll(heap, "allreduce", OP_ALLREDUCE_ONE_SHOT, ptr, ptr, nbytes,
                           dtype_code=code)
    elif ex.implementation == "device_one_shot":
        # One staging area (two parities of the largest one-shot message) and one counter
        # block serve every message size: the parity halves sit at fixed offsets, so calls
        # of different sizes alternate between them just like calls of one size.
        stage = heap._state.get("coll_stage")
        if stage is None:
            stage = heap.allocate_tensor((2 * ONE_SHOT_MAX_BYTES,), torch.uint8)
            heap._state["coll_stage"] = stage
        again = _launch(heap, "allreduce1", OP_ALLREDUCE_ONE_SHOT, code, ptr, ptr, nbytes,
                        staging=stage.data_ptr(), stage_slot=ONE_SHOT_MAX_BYTES,
                        grid=ex.grid_size, elem_size=tensor.element_size())
    else:
        again = _launch(heap, "allreduce2", OP_ALLREDUCE_TWO_SHOT, code, ptr, ptr, nbytes,
                        use_multimem=ex.use_multimem, grid=ex.grid_size,
                        elem_size=tensor.element_size())
    _remember(heap, "allreduce", tensor, None, 0, again)
    return tensor


def allgather(tensor: torch.Tensor, output: torch.Tensor, heap=None, *, ctx=None) -> torch.Tensor:
    """``output[r * n:(r + 1) * n] = rank r's tensor`` on every rank."""
    heap = _heap_of(heap, ctx)
    if try_fast(heap, "allgather", tensor, output):
        return output
    _validate("tensor", tensor, heap)
    _validate("output", output, heap)
    if output.numel() != tensor.numel() * heap.world_size or output.dtype != tensor.dtype:
        raise ValueError(f"output must hold world_size * {tensor.numel()} elements of {tensor.dtype}")
    nbytes = tensor.numel() * tensor.element_size()
    if heap.world_size == 1:
        output.view(-1).copy_(tensor.view(-1))
        return output
    if _ll_ok(heap, nbytes, tensor.data_ptr(), output.data_ptr()):
        again = _launch_ll(heap, "allgather", OP_ALLGATHER, tensor.data_ptr(), output.data_ptr(),
                           nbytes)
    else:
        again = _launch(heap, "allgather", OP_ALLGATHER, 3, tensor.data_ptr(), output.data_ptr(),
                        nbytes, use_multimem=_use_multimem(heap, nbytes, "allgather"),
                        elem_size=tensor.element_size())
    _remember(heap, "allgather", tensor, output, 0, again)
    return output


def reduce_scatter(tensor: torch.Tensor, output: torch.Tensor, heap=None, op: str = "sum",
                   implementation: str = "auto", *, ctx=None) -> torch.Tensor:
    """``output = sum over ranks of tensor[rank * n:(rank + 1) * n]``."""
    heap = _heap_of(heap, ctx)
    if op != "sum":
        raise ValueError(f"only op='sum' is supported, got {op!r}")
    if implementation not in ("auto", "device"):
        raise ValueError("implementation must be 'auto' or 'device' (there is no host reference path)")
    if try_fast(heap, "reduce_scatter", tensor, output):
        return output
    _validate("tensor", tensor, heap)
    _validate("output", output, heap)
    if tensor.dtype not in _DTYPE_CODE:
        raise TypeError(f"reduce_scatter supports float16, bfloat16 and float32, got {tensor.dtype}")
    if tensor.numel() != output.numel() * heap.world_size or output.dtype != tensor.dtype:
        raise ValueError(f"tensor must hold world_size * {output.numel()} elements of {output.dtype}")
    nbytes = output.numel() * output.element_size()
    if heap.world_size == 1:
        output.view(-1).copy_(tensor.view(-1))
        return output
    if _ll_ok(heap, nbytes, tensor.data_ptr(), output.data_ptr()):
        again = _launch_ll(heap, "reduce_scatter", OP_REDUCE_SCATTER, tensor.data_ptr(),
                           output.data_ptr(), nbytes, dtype_code=_DTYPE_CODE[tensor.dtype])
    else:
        again = _launch(heap, "reduce_scatter", OP_REDUCE_SCATTER, _DTYPE_CODE[tensor.dtype],
                        tensor.data_ptr(), output.data_ptr(), nbytes,
                        use_multimem=_use_multimem(heap, nbytes, "reduce_scatter"),
                        elem_size=tensor.element_size())
    _remember(heap, "reduce_scatter", tensor, output, 0, again)
    return output


def broadcast(tensor: torch.Tensor, heap=None, root: int = 0, *, ctx=None) -> torch.Tensor:
    """Every rank's ``tensor`` becomes ``root``'s (in place)."""
    heap = _heap_of(heap, ctx)
    if try_fast(heap, "broadcast", tensor, None, root):
        return tensor
    _validate("tensor", tensor, heap)
    if not 0 <= root < heap.world_size:
        raise ValueError(f"root={root} out of range for world_size={heap.world_size}")
    if heap.world_size == 1:
        return tensor
    nbytes = tensor.numel() * tensor.element_size()
    if _ll_ok(heap, nbytes, tensor.data_ptr()):
        again = _launch_ll(heap, f"broadcast:{root}", OP_BROADCAST, tensor.data_ptr(),
                           tensor.data_ptr(), nbytes, root=root)
    elif _relay_ok(heap, nbytes, tensor.data_ptr()):
        again = _launch_relay(heap, root, tensor.data_ptr(), nbytes)
    else:
        # The rooted handshake only advances the counters between the root and the others, so
        # every root has its own counter block and epoch (roots may alternate call by call).
        again = _launch(heap, f"broadcast:{root}", OP_BROADCAST, 3, tensor.data_ptr(),
                        tensor.data_ptr(), nbytes, root=root,
                        use_multimem=_use_multimem(heap, nbytes), rv_extra=(root,),
                        elem_size=tensor.element_size())
    _remember(heap, "broadcast", tensor, None, root, again)
    return tensor


def scatter(tensor: torch.Tensor, output: torch.Tensor, heap=None, *, root: int = 0,
            ctx=None) -> torch.Tensor:
    """Rank ``r`` receives ``root``'s ``tensor[r * n:(r + 1) * n]`` in ``output``."""
    heap = _heap_of(heap, ctx)
    if try_fast(heap, "scatter", tensor, output, root):
        return output
    _validate("tensor", tensor, heap)
    _validate("output", output, heap)
    if not 0 <= root < heap.world_size:
        raise ValueError(f"root={root} out of range for world_size={heap.world_size}")
    if tensor.numel() != output.numel() * heap.world_size or output.dtype != tensor.dtype:
        raise ValueError(f"tensor must hold world_size * {output.numel()} elements of {output.dtype}")
    nbytes = output.numel() * output.element_size()
    if heap.world_size == 1:
        output.view(-1).copy_(tensor.view(-1))
        return output
    if _ll_ok(heap, nbytes, tensor.data_ptr(), output.data_ptr()):
        again = _launch_ll(heap, f"scatter:{root}", OP_SCATTER, tensor.data_ptr(),
                           output.data_ptr(), nbytes, root=root)
    else:
        again = _launch(heap, f"scatter:{root}", OP_SCATTER, 3, tensor.data_ptr(),
                        output.data_ptr(), nbytes, root=root, rv_extra=(root,),
                        elem_size=tensor.element_size())
    _remember(heap, "scatter", tensor, output, root, again)
    return output
