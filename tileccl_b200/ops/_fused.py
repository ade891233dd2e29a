"""Engine behind the fused GEMM + collective operators.

Turns tensors and a context into native plans (``kernels/fused_gemm.py``), owns
the per-operator symmetric workspaces (TileGroup counters, reduce-scatter
staging), advances epochs, and decides how the launches of one call are ordered:

* one process per GPU: a single launch per call; waiting for peers happens
  inside the kernel (bounded);
* one process driving one GPU per rank: the same launches, issued rank after
  rank; kernels on different GPUs overlap, so in-kernel waits are still fine;
* several ranks emulated on one GPU: kernels of different ranks must not wait
  on each other inside a launch, so the calls of all ranks are collected and
  then replayed phase by phase (all producers, then all consumers).  The
  reference has the same rendezvous for its single-process mode
  (tileccl/ops.py:85-92, 1572-1658).
"""

from __future__ import annotations

import ctypes as C
from typing import Callable, Optional, Sequence

import torch

from .. import _native
from ..kernels import fused_gemm as fg
from ..utils.config import current as _config

MAX_GROUPS = 64           # TileGroup counters per source rank in a signal block
_DEFAULT_PUSH = {"stores": fg.PUSH_STORES, "tma": fg.PUSH_TMA, "multimem": fg.PUSH_MULTIMEM}


# --------------------------------------------------------------------------
# per-context state
# --------------------------------------------------------------------------
MAX_OP_STATES = 512
_PINNED_STATE_KINDS = ("sig", "h2d_stream")   # signal blocks carry epochs: never evicted


def op_state(ctx, key) -> dict:
    """Mutable state of one (operator, shapes, buffers) combination on one rank.

    A plan bakes addresses, extents, strides and the dtype into its tensor maps, and all of
    those are part of its key, so an equal key always means equal descriptors (a freed
    tensor whose address is reused by one of the same geometry gets the same plan, which is
    then also the right one).  The table is bounded: beyond ``MAX_OP_STATES`` entries the
    oldest plan entry is dropped (its native plan is destroyed with it; the signal blocks
    and their epochs stay)."""
    table = ctx._state.setdefault("ops", {})
    st = table.get(key)
    if st is None:
        if len(table) >= MAX_OP_STATES:
            for old in table:
                if old[0] not in _PINNED_STATE_KINDS:
                    dropped = table.pop(old)
                    plan = dropped.get("plan")
                    dropped.clear()
                    if plan is not None and hasattr(plan, "close"):
                        plan.close()
                    break
        st = {"epoch": 0}
        table[key] = st
    return st


def status_block(ctx) -> torch.Tensor:
    """uint32[8] device words a kernel writes when one of its waits gives up."""
    st = ctx._state.get("status")
    if st is None:
        st = torch.zeros(fg.STATUS_WORDS, dtype=torch.int32, device=ctx.torch_device)
        ctx._state["status"] = st
    return st


def stats_block(ctx) -> torch.Tensor:
    """uint64[256][4] device table: CTA b of every fused launch adds its counters to row b."""
    st = ctx._state.get("stats")
    if st is None:
        st = torch.zeros(fg.STAT_WORDS, dtype=torch.int64, device=ctx.torch_device)
        ctx._state["stats"] = st
    return st


def call_stats(ctx, reset: bool = True) -> dict:
    """Counters accumulated by the fused kernels of this context since the last reset
    (synchronises the device): bytes stored into peers' memory, TileGroup signals sent,
    SM cycles spent waiting for peers (summed over the waiting threads) and tiles computed."""
    st = ctx._state.get("stats")
    if st is None:
        return {"bytes_pushed": 0, "signals_sent": 0, "peer_wait_cycles": 0, "tiles": 0}
    torch.cuda.synchronize(ctx.torch_device)
    w = st.view(-1, 4).sum(0).cpu().tolist()
    if reset:
        st.zero_()
    return {"bytes_pushed": w[0], "signals_sent": w[1], "peer_wait_cycles": w[2], "tiles": w[3]}


def check_status(ctx) -> None:
    """Synchronise and raise :class:`TileCCLTimeoutError` if any kernel gave up waiting."""
    st = ctx._state.get("status")
    if st is None:
        return
    torch.cuda.synchronize(ctx.torch_device)
    fg.raise_on_status(st)


def recover(ctx) -> None:
    """Bring the fused operators of this context back to a clean state after a device wait
    gave up (``TileCCLTimeoutError``): a call that was cut short leaves its TileGroup
    counters between two epochs, so later calls would wait for counts that never come.

    Collective: every rank calls it at the same point, with none of its kernels in flight.
    All ranks meet, every counter block and arrival counter of this context is zeroed, the
    epochs restart at zero, and the ranks meet again before anyone launches.
    """
    ctx.barrier()
    for st in ctx._state.get("ops", {}).values():
        if not isinstance(st, dict):
            continue
        for name in ("sig", "entry", "gate", "counters", "bands"):
            t = st.get(name)
            if isinstance(t, torch.Tensor):
                t.zero_()
        if "epoch" in st:
            st["epoch"] = 0
    status = ctx._state.get("status")
    if status is not None:
        status.zero_()
    heap = ctx.heap
    if heap is not None:
        # the stand-alone collectives keep their counter blocks and epochs on the heap object
        for key, st in heap._state.items():
            if (isinstance(key, tuple) and key and key[0] in ("coll", "coll_ll", "coll_relay")
                    and isinstance(st, dict)):
                st["counters"].zero_()
                if "stage" in st:
                    st["stage"].zero_()      # stale low-latency lines carry old flags
                if "flags" in st:
                    st["flags"].zero_()      # piece flags of the relay broadcast hold call numbers
                st["epoch"] = 0
        hs = heap._state.get("status")
        if hs is not None:
            hs.zero_()
    ctx.barrier()


def wait_budget_ns() -> int:
    return _config().wait_budget_ns


def default_push_mode(ctx) -> int:
    cfg = _config()
    if cfg.push_mode_explicit:
        mode = _DEFAULT_PUSH[cfg.push_mode]
        if mode == fg.PUSH_MULTIMEM and not (ctx.heap is not None and ctx.heap.has_multicast):
            raise RuntimeError("TILECCL_PUSH_MODE=multimem but no NVLS multicast mapping is bound")
        return mode
    # Bulk (TMA) stores straight from the staged tile: measured fastest on NVLink 5.
    return fg.PUSH_TMA


def default_rs_own_lag(ws: int, m_tiles: int, n_tiles: int) -> int:
    """Rounds by which a reduce-scatter rank's own tile rows trail its remote rows.

    A round sends one tile row to every peer.  The own row j is reduced once the
    peers' row j has arrived, so it trails by the time a pushed row needs to land
    under load.  Measured at two ranks (16384 x 4096 x 2048: lag 0 / 8 / 16 / 32 rounds
    -> 0.174 / 0.166 / 0.154 / 0.161 ms): about 24 us of link time is the sweet spot.
    0 means "own rows last" (nothing to overlap, or too few rows).
    """
    env = _config().rs_own_lag
    if env is not None:
        return max(0, env)
    if ws < 2 or m_tiles < 2:
        return 0
    round_bytes = (ws - 1) * n_tiles * fg.BLOCK_M * fg.BLOCK_N * 2
    round_us = round_bytes / 690e3            # measured NVLink 5 push rate, bytes per us
    lag = int(-(-24.0 // round_us))
    return lag if 1 <= lag < m_tiles else 0


def rs_uses_cta_pairs(ws: int) -> bool:
    """Kernel form of a reduce-scatter.  With peers the one-CTA form measured faster at 2, 4
    and 8 GPUs (its owner-side reduction multiplies a 128 x 128 identity, the CTA-pair form a
    256 x 256 one of which half is zero blocks, and an own pair-tile waits for two tile rows
    of every peer instead of one); a single rank runs a plain GEMM, where pairs win."""
    forced = _config().rs_cta_pairs
    if forced is not None:
        return forced
    return ws <= 1


def default_group_m_tiles(m_tiles: int, n_tiles: Optional[int] = None, elem_bytes: int = 2) -> int:
    """Tile rows per TileGroup: the planner's P0 rule (a group carries at least tau_min bytes,
    tileccl_v2/tile_group.py:116-117 in the reference) with tau_min taken from the calibration
    file, and never more than MAX_GROUPS groups.  For the 4096-column gate shapes one tile row
    (1 MiB) already exceeds the calibrated tau_min, so groups are single rows."""
    finest = max(1, -(-m_tiles // MAX_GROUPS))
    if not n_tiles:
        return finest
    from ..planning.cost_model import calibrated_tau_min_bytes

    row_bytes = n_tiles * fg.BLOCK_M * fg.BLOCK_N * elem_bytes
    need = -(-calibrated_tau_min_bytes() // row_bytes)
    return max(1, min(m_tiles, max(finest, need)))


# --------------------------------------------------------------------------
# launch ordering
# --------------------------------------------------------------------------
def run_phases(ctx, key, phases: Sequence[Callable[[], None]]) -> None:
    """Run this rank's launches now, or park them until every emulated rank has called."""
    group = ctx.local_group
    if group is None or not group.emulated or ctx.world_size == 1:
        for ph in phases:
            ph()
        return
    slot = group.pending.setdefault(key, {})
    if ctx.rank in slot:
        raise RuntimeError(
            f"rank {ctx.rank} called the same collective operator twice before the other emulated "
            "ranks called it once")
    slot[ctx.rank] = list(phases)
    if len(slot) < ctx.world_size:
        return
    del group.pending[key]
    n = max(len(p) for p in slot.values())
    for i in range(n):
        for r in range(ctx.world_size):
            if i < len(slot[r]):
                slot[r][i]()


def _on_device(ctx, fn: Callable[[], None]) -> Callable[[], None]:
    dev = ctx.torch_device

    def wrapped():
        with torch.cuda.device(dev):
            fn()

    return wrapped


def _in_kernel_waits_ok(ctx) -> bool:
    """Whether a kernel of this rank may spin on flags written by other ranks' kernels."""
    return not ctx.emulated


# --------------------------------------------------------------------------
# workspaces
# --------------------------------------------------------------------------
def _signal_state(ctx, signame: str) -> dict:
    """Counter block + epoch shared by every plan with the same operator name and shapes.

    The epoch belongs to the counters (they only grow), not to a plan: two plans
    over different buffers of the same shape take turns on one block.
    """
    st = op_state(ctx, ("sig", signame))
    if "sig" not in st:
        st["sig"] = ctx.workspace(f"sig:{signame}", ctx.world_size * MAX_GROUPS, dtype=torch.int32)
        # "calls entered" counters of the entry handshake (see entry_ptr)
        st["entry"] = ctx.workspace(f"entry:{signame}", 8, dtype=torch.int32)
    return st


def entry_ptr(ctx, st: dict) -> int:
    """Address of the entry-handshake counters of a signal state, or 0 when the handshake is
    not needed.  A kernel that stores into its peers' copy of a buffer (the all-gathered C, the
    gathered A operand) first waits until those peers have entered the same call: their
    streams have then finished whatever read the previous call's data, so back-to-back calls
    on one buffer need no barrier from the caller.  Ranks that share a GPU are launched phase
    by phase on one stream and need none of this."""
    if ctx.world_size <= 1 or not _in_kernel_waits_ok(ctx):
        return 0
    return st["entry"].data_ptr()


def _heap_offset_ptrs(ctx, tensor: torch.Tensor, extra_bytes: int = 0) -> list:
    """Address of `tensor` (+ byte offset) in every rank's heap, as mapped in this process."""
    heap = ctx.require_heap()
    off = heap.get_offset(tensor.data_ptr()) + extra_bytes
    return [heap.peer_base(r) + off for r in range(ctx.world_size)]


def _require_2d(name: str, t: torch.Tensor, ctx) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be a row-major 2-D tensor, got shape {tuple(t.shape)} "
                         f"strides {tuple(t.stride())}")
    if t.device != ctx.torch_device:
        raise ValueError(f"{name} is on {t.device}, expected {ctx.torch_device}")


def _b_dims(B: torch.Tensor, b_is_nk: bool) -> tuple:
    return (B.shape[1], B.shape[0]) if b_is_nk else (B.shape[0], B.shape[1])  # (K, N)


# --------------------------------------------------------------------------
# A operand streamed from pinned host memory while the kernel runs
# --------------------------------------------------------------------------
def visit_rows(m_tiles: int, owners: int, rank: int, world_size: int, own_lag: int = 0) -> list:
    """``(owner, tile_row)`` of every tile row in the order the kernel visits them
    (the row-level view of csrc/plan/tile_order.h; rot_m_tiles = 0)."""
    if owners <= 1:
        return [(rank, r) for r in range(m_tiles)]
    lag = m_tiles if own_lag <= 0 or own_lag > m_tiles else own_lag
    rows = []
    for r in range(m_tiles):
        rows += [((rank + d) % world_size, r) for d in range(1, owners)]
        if r >= lag:
            rows.append((rank, r - lag))
    rows += [(rank, j) for j in range(m_tiles - lag, m_tiles)]
    return rows


# Shares of the rank's tile rows given to successive runs of a host-streamed launch.  Every
# extra cudaMemcpyAsync costs several microseconds of copy-engine set-up (measured: 24 copies
# instead of 6 per step added about 0.2 ms), so there are few runs; the falling sizes leave
# little math behind the last byte of the transfer.
STREAM_RUN_SHARES = (0.50, 0.35, 0.15)


def _tile_row_chunks(plan, min_tiles: int = 148, shares: Sequence[float] = STREAM_RUN_SHARES) -> list:
    """Split the rank's tile order into runs of whole tile rows.

    Returns ``[(tile_begin, tile_end, [(row0, row1), ...]), ...]`` where the row
    ranges are the rows of A the run reads.  Runs follow the kernel's visiting
    order (rounds over the owners for reduce-scatter, see csrc/plan/tile_order.h),
    so the host copy of run i only has to stay ahead of the launch of run i.
    Run sizes follow ``shares``; runs smaller than ``min_tiles`` tiles are merged
    into their predecessor.
    """
    n_t = plan.n_tiles_local
    spec = plan.spec
    order = visit_rows(plan.m_tiles_local, plan.owners, spec.rank, spec.world_size,
                       getattr(spec, "rs_own_lag", 0))
    rows_total = len(order)
    min_rows = max(1, -(-min_tiles // n_t))
    bounds, acc = [0], 0.0
    for share in shares[:-1]:
        acc += share
        b = min(rows_total, round(acc * rows_total))
        if b - bounds[-1] >= min_rows and rows_total - b >= min_rows:
            bounds.append(b)
    bounds.append(rows_total)
    chunks = []
    for i in range(len(bounds) - 1):
        r0, r1 = bounds[i], bounds[i + 1]
        if r1 <= r0:
            continue
        ranges = []
        for owner, lm in order[r0:r1]:
            base = owner * spec.sub_m if plan.owners > 1 and spec.split_axis == 0 else 0
            limit = spec.sub_m if plan.owners > 1 else spec.a_rows
            lo = base + lm * fg.BLOCK_M
            hi = min(base + min(limit, (lm + 1) * fg.BLOCK_M), spec.a_rows)
            ranges.append((lo, hi))
        # rows of one owner are contiguous across rounds: sort and merge into few large copies
        merged = []
        for lo, hi in sorted(ranges):
            if merged and merged[-1][1] == lo:
                merged[-1] = (merged[-1][0], hi)
            else:
                merged.append((lo, hi))
        chunks.append((r0 * n_t, r1 * n_t, merged))
    return chunks


def launch_streamed(ctx, plan, A: torch.Tensor, a_host: torch.Tensor, *,
                    order: str = "stream", **launch_kw) -> None:
    """Run ``plan`` while its A operand is still arriving from pinned host memory.

    The rows of ``a_host`` are copied to ``A`` on a side stream in the order the
    kernel consumes them; every run of tile rows is launched as soon as its rows
    are on the device, so all but the last run's math hides under the PCIe copy.
    Everything is stream-ordered: the host never blocks.

    ``order="stream"``: the copies start after everything queued on the current
    stream (anything there may still read ``A``).  ``order="plan"``: the caller
    guarantees that no other pending work touches ``A``; the copies then only follow
    this operator's previous call on the same buffers, and the transfer for one
    problem overlaps the kernels of the one before it.
    """
    if order not in ("stream", "plan"):
        raise ValueError("order must be 'stream' or 'plan'")
    if a_host.shape != A.shape or a_host.dtype != A.dtype:
        raise ValueError(f"a_host must match A: {tuple(a_host.shape)} {a_host.dtype} vs "
                         f"{tuple(A.shape)} {A.dtype}")
    if not a_host.is_pinned():
        raise ValueError("a_host must be pinned host memory (tensor.pin_memory())")
    if (plan.owners > 1 and plan.spec.split_axis != 0) or plan.spec.rot_m_tiles != 0:
        # column-split reduce-scatter reads every row of A for every owner
        A.copy_(a_host, non_blocking=True)
        plan.launch(**launch_kw)
        return
    st = op_state(ctx, ("h2d_stream",))
    if "stream" not in st:
        st["stream"] = torch.cuda.Stream(device=ctx.torch_device)
        st["stream2"] = torch.cuda.Stream(device=ctx.torch_device)
    side, cur = st["stream"], torch.cuda.current_stream()
    key = (A.data_ptr(), a_host.data_ptr(), A.stride(0))
    prepared = getattr(plan, "_stream_chunks", None)
    if prepared is None or prepared[0] != key:
        chunks = _tile_row_chunks(plan, shares=_config().stream_run_shares or STREAM_RUN_SHARES)
        if not A.is_contiguous() or any(len(r) > _native.STREAM_MAX_RANGES for _, _, r in chunks):
            prepared = (key, None, chunks)
        else:
            row_bytes = A.shape[1] * A.element_size()
            arr = (_native.StreamChunk * len(chunks))()
            for c, (t0, t1, ranges) in zip(arr, chunks):
                c.tile_begin, c.tile_end, c.n_ranges = t0, t1, len(ranges)
                for i, (lo, hi) in enumerate(ranges):
                    c.dst[i] = A.data_ptr() + lo * row_bytes
                    c.src[i] = a_host.data_ptr() + lo * row_bytes
                    c.bytes[i] = (hi - lo) * row_bytes
            prepared = (key, arr, chunks)
        plan._stream_chunks = prepared
    _, arr, chunks = prepared
    wait_incoming = launch_kw.pop("wait_incoming", False)
    ag_push = launch_kw.pop("ag_push", False)
    if arr is not None:
        # Copies, events and launches are issued by the native runtime: a few microseconds
        # of host time per run instead of a Python round trip each.
        fg.count_launches(len(chunks))
        if getattr(plan, "_stream_fast", None) is None or plan._stream_fast[0] != (key, order):
            fn = getattr(_native.load(), "tccl_gemm_plan_launch_streamed")
            handle, n_chunks, side_ptr = plan._handle, len(chunks), side.cuda_stream
            side2_ptr = st["stream2"].cuda_stream if _config().stream_copy_streams == 2 else 0
            order_bit = 4 if order == "plan" else 0

            def stream_fast(epoch, a_gate_target, flags, _arr=arr):
                """Repeat of this streamed launch on the same buffers: one native call."""
                fg.count_launches(n_chunks)
                rc = fn(handle, epoch & 0xFFFFFFFF, a_gate_target & 0xFFFFFFFF,
                        flags | order_bit | 8, _arr, n_chunks, side_ptr, side2_ptr,
                        torch.cuda.current_stream().cuda_stream)
                if rc != 0:
                    _native.check("tccl_gemm_plan_launch_streamed", rc)

            plan._stream_fast = ((key, order), stream_fast)
        _native.call("tccl_gemm_plan_launch_streamed", plan._handle,
                     launch_kw.get("epoch", 1) & 0xFFFFFFFF,
                     launch_kw.get("a_gate_target", 0) & 0xFFFFFFFF,
                     (1 if wait_incoming else 0) | (2 if ag_push else 0)
                     | (4 if order == "plan" else 0) | 8, arr, len(chunks),
                     side.cuda_stream,
                     st["stream2"].cuda_stream if _config().stream_copy_streams == 2 else 0,
                     cur.cuda_stream)
        return
    side.wait_stream(cur)                       # earlier readers of A are done
    events = st.setdefault("events", [torch.cuda.Event() for _ in range(16)])
    for i, (t0, t1, ranges) in enumerate(chunks):
        ev = events[i % 16]
        with torch.cuda.stream(side):
            for lo, hi in ranges:
                A[lo:hi].copy_(a_host[lo:hi], non_blocking=True)
            ev.record(side)
        cur.wait_event(ev)
        last = i == len(chunks) - 1
        plan.launch(tile_begin=t0, tile_end=t1, wait_incoming=wait_incoming and last,
                    ag_push=ag_push and i == 0, announce_entry=i == 0, **launch_kw)


# --------------------------------------------------------------------------
# push-all: C_d[region of this rank] = A @ B for every rank d
# --------------------------------------------------------------------------
def push_all(ctx, name: str, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, *,
             region_row0: int, region_col0: int, b_is_nk: bool = False,
             group_m_tiles: Optional[int] = None, push_mode: Optional[int] = None,
             wait: bool = True, a_host: Optional[torch.Tensor] = None,
             a_host_order: str = "stream") -> None:
    """Product of the local operands, written into the same region of ``C`` on every rank.

    ``C`` must live on the symmetric heap.  ``region_*`` is where this rank's
    ``[A.rows, N_b]`` block goes inside ``C``.  With ``wait`` the call also
    makes sure (on the stream) that every peer's block has arrived in the local
    ``C``.  ``a_host`` (pinned, same shape as ``A``): the operand is first brought
    to ``A`` from the host, overlapped with the kernel (see ``launch_streamed``).
    """
    _require_2d("A", A, ctx)
    _require_2d("B", B, ctx)
    _require_2d("C", C, ctx)
    K, N = _b_dims(B, b_is_nk)
    Mloc = A.shape[0]
    if A.shape[1] != K:
        raise ValueError(f"inner dimensions differ: A {tuple(A.shape)}, B {tuple(B.shape)}")
    ws, rank = ctx.world_size, ctx.rank
    if ws > 1 and not ctx.is_symmetric(C):
        raise ValueError("C must be allocated from the symmetric heap (ctx.zeros / ctx.empty)")
    push_mode = default_push_mode(ctx) if push_mode is None else push_mode
    key = ("push_all", name, A.data_ptr(), B.data_ptr(), C.data_ptr(), Mloc, N, K, A.stride(0),
           B.stride(0), C.stride(0), A.dtype, b_is_nk, region_row0, region_col0, push_mode)
    st = op_state(ctx, key)
    fast = st.get("fast")
    if fast is not None and a_host is None:
        fast(wait)              # repeated call on the same buffers: epoch + launch only
        return
    if a_host is not None:
        fh = st.get("fast_host")
        if fh is not None and fh[0] == (a_host.data_ptr(), a_host_order):
            fh[1](wait)         # the same, with the operand streamed from the same host buffer
            return
    m_tiles = -(-Mloc // fg.BLOCK_M)
    gm = group_m_tiles or default_group_m_tiles(m_tiles, -(-N // fg.BLOCK_N), A.element_size())
    sigst = _signal_state(ctx, f"push_all:{name}:{Mloc}x{N}x{K}:g{gm}") if ws > 1 else st
    if "plan" not in st:
        region_bytes = (region_row0 * C.stride(0) + region_col0) * C.element_size()
        if ws > 1:
            sig = sigst["sig"]
            dests = _heap_offset_ptrs(ctx, C, region_bytes)
            mc = 0
            if push_mode == fg.PUSH_MULTIMEM:
                mc = ctx.heap.multicast_ptr(C.data_ptr()) + region_bytes
            sig_ptr, stride = sig.data_ptr(), ctx.heap.stride
        else:
            dests = [C.data_ptr() + region_bytes]
            mc, sig_ptr, stride = 0, 0, 0
        st["plan"] = fg.FusedGemmPlan(fg.FusedGemmSpec(
            mode=fg.MODE_PUSH_ALL if ws > 1 else fg.MODE_GEMM, dtype=A.dtype, a_ptr=A.data_ptr(),
            a_rows=Mloc, lda=A.stride(0), b_ptr=B.data_ptr(), b_cols=N, ldb=B.stride(0), k=K,
            sub_m=Mloc, sub_n=N, out_ptrs=dests, ldo=C.stride(0), out_rows=Mloc, out_cols=N,
            b_kmajor=b_is_nk, push_mode=push_mode, rank=rank, world_size=ws, out_mc_ptr=mc,
            group_m_tiles=gm, sig_local=sig_ptr, heap_stride=stride, sig_stride=MAX_GROUPS,
            entry_local=entry_ptr(ctx, sigst) if ws > 1 else 0,
            status_ptr=status_block(ctx).data_ptr(), stats_ptr=stats_block(ctx).data_ptr(), wait_budget_ns=wait_budget_ns()))
        plan = st["plan"]
        if ws > 1:
            per_epoch = [plan.group_m_count(g) * plan.n_tiles_local * fg.EPILOGUE_SLABS
                         for g in range(plan.groups)]
            st["per_epoch"] = torch.tensor(per_epoch, dtype=torch.int32, device=ctx.torch_device)
            st["sig"] = sig
    plan = st["plan"]
    if ctx.local_group is None and "fast" not in st:
        # One process per GPU (or a single rank): nothing to rendezvous with on the host.
        in_kernel = ws > 1 and _in_kernel_waits_ok(ctx)

        def fast(wait_flag, _plan=plan, _sig=sigst, _ws=ws, _ik=in_kernel):
            _sig["epoch"] += 1
            if _ws == 1:
                _plan.launch()
            else:
                _plan.launch(epoch=_sig["epoch"], wait_incoming=wait_flag and _ik)

        st["fast"] = fast
    sigst["epoch"] += 1
    epoch = sigst["epoch"]
    def remember_streamed(in_kernel_wait: bool) -> None:
        """After a streamed call went through the checked path once, later calls with the
        same host buffer take one native call (host time matters: the first copy of a step
        cannot start before the host has issued it)."""
        sf = getattr(plan, "_stream_fast", None)
        if sf is None or ctx.local_group is not None:
            return
        launcher = sf[1]

        def fast_host(wait_flag, _sig=sigst):
            _sig["epoch"] += 1
            launcher(_sig["epoch"], 0, 1 if (wait_flag and in_kernel_wait) else 0)

        st["fast_host"] = ((a_host.data_ptr(), a_host_order), fast_host)

    if ws == 1:
        if a_host is not None:
            launch_streamed(ctx, plan, A, a_host, order=a_host_order)
            remember_streamed(False)
        else:
            plan.launch()
        return
    fused_wait = wait and _in_kernel_waits_ok(ctx) and not ctx.is_single_process
    if a_host is not None and not ctx.is_single_process:
        phases = [_on_device(ctx, lambda: launch_streamed(ctx, plan, A, a_host, epoch=epoch,
                                                          order=a_host_order,
                                                          wait_incoming=fused_wait))]
    else:
        if a_host is not None:
            A.copy_(a_host, non_blocking=True)
        phases = [_on_device(ctx, lambda: plan.launch(epoch=epoch, wait_incoming=fused_wait))]
    if wait and not fused_wait:
        phases.append(_on_device(ctx, lambda: wait_groups(ctx, st["sig"], plan.groups,
                                                          st["per_epoch"], epoch)))
    run_phases(ctx, ("push_all", name, Mloc, N, K, epoch), phases)
    if a_host is not None and not ctx.is_single_process:
        remember_streamed(True)


def wait_groups(ctx, sig: torch.Tensor, n_groups: int, per_epoch: torch.Tensor, epoch: int) -> None:
    """Stream-ordered wait until every peer's TileGroups of `epoch` have been signalled."""
    _native.call("tccl_wait_groups", sig.data_ptr(), MAX_GROUPS, ctx.world_size, n_groups,
                 per_epoch.data_ptr(), epoch & 0xFFFFFFFF, ctx.rank,
                 status_block(ctx).data_ptr(), wait_budget_ns(), ctx.rank,
                 torch.cuda.current_stream().cuda_stream)


# --------------------------------------------------------------------------
# reduce-scatter: C_local = sum over ranks of (A_r @ B_r)[this rank's block]
# --------------------------------------------------------------------------
def reduce_scatter(ctx, name: str, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, *,
                   split_axis: int, b_is_nk: bool = False, group_m_tiles: Optional[int] = None,
                   push_mode: Optional[int] = None, a_host: Optional[torch.Tensor] = None,
                   a_host_order: str = "stream") -> None:
    """Every rank multiplies its operands; block ``r`` of the summed product lands on rank ``r``.

    ``split_axis=0``: ``A`` is ``[ws * Mloc, K]``, ``C`` is ``[Mloc, N]`` (row blocks).
    ``split_axis=1``: ``B`` has ``ws * Nloc`` columns, ``C`` is ``[M, Nloc]`` (column blocks).
    Partials travel as 16-bit values into a staging area on the owner's heap and are summed
    there in fp32, in rank order, by the epilogue of the owner's own tiles.
    """
    _require_2d("A", A, ctx)
    _require_2d("B", B, ctx)
    _require_2d("C", C, ctx)
    K, N = _b_dims(B, b_is_nk)
    M = A.shape[0]
    ws, rank = ctx.world_size, ctx.rank
    if A.shape[1] != K:
        raise ValueError(f"inner dimensions differ: A {tuple(A.shape)}, B {tuple(B.shape)}")
    if split_axis == 0:
        if M % ws:
            raise ValueError(f"M={M} is not divisible by world_size={ws}")
        sub_m, sub_n = M // ws, N
    else:
        if N % ws:
            raise ValueError(f"N={N} is not divisible by world_size={ws}")
        sub_m, sub_n = M, N // ws
    if tuple(C.shape) != (sub_m, sub_n):
        raise ValueError(f"C must be {(sub_m, sub_n)}, got {tuple(C.shape)}")
    if not C.is_contiguous():
        raise ValueError("C must be contiguous")
    push_mode = default_push_mode(ctx) if push_mode is None else push_mode
    if push_mode == fg.PUSH_MULTIMEM:
        push_mode = fg.PUSH_STORES  # partials go to one owner, not to everyone
    key = ("reduce_scatter", name, A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, A.stride(0),
           B.stride(0), C.stride(0), A.dtype, b_is_nk, split_axis, push_mode)
    st = op_state(ctx, key)
    fast = st.get("fast")
    if fast is not None and a_host is None:
        fast()
        return
    if a_host is not None:
        fh = st.get("fast_host")
        if fh is not None and fh[0] == (a_host.data_ptr(), a_host_order):
            fh[1]()
            return
    m_tiles = -(-sub_m // fg.BLOCK_M)
    gm = group_m_tiles or default_group_m_tiles(m_tiles, -(-sub_n // fg.BLOCK_N), A.element_size())
    sigst = (_signal_state(ctx, f"reduce_scatter:{name}:{M}x{N}x{K}:a{split_axis}:g{gm}:{A.dtype}")
             if ws > 1 else st)
    if "plan" not in st:
        if ws > 1:
            sig = sigst["sig"]
            if "stage" not in sigst:
                sigst["stage"] = ctx.workspace(f"stage:{name}:{sub_m}x{sub_n}:{A.dtype}",
                                               2 * ws * sub_m * sub_n, dtype=A.dtype)
            stage = sigst["stage"]
            dests = _heap_offset_ptrs(ctx, stage)
            dests[rank] = C.data_ptr()
            sig_ptr, stride, stage_ptr = sig.data_ptr(), ctx.heap.stride, stage.data_ptr()
            st["sig"], st["stage"] = sig, stage
        else:
            dests = [C.data_ptr()]
            sig_ptr = stride = stage_ptr = 0
        st["plan"] = fg.FusedGemmPlan(fg.FusedGemmSpec(
            mode=fg.MODE_REDUCE_SCATTER if ws > 1 else fg.MODE_GEMM, dtype=A.dtype,
            a_ptr=A.data_ptr(), a_rows=M, lda=A.stride(0), b_ptr=B.data_ptr(), b_cols=N,
            ldb=B.stride(0), k=K, sub_m=sub_m, sub_n=sub_n, out_ptrs=dests, ldo=sub_n,
            out_rows=sub_m, out_cols=sub_n, b_kmajor=b_is_nk, push_mode=push_mode, rank=rank,
            world_size=ws, split_axis=split_axis, out_slot_elems=sub_m * sub_n, out_slots=2 * ws,
            ident_ptr=fg.identity_operand(A.dtype, A.device).data_ptr() if ws > 1 else 0,
            rs_own_lag=(default_rs_own_lag(ws, m_tiles, -(-sub_n // fg.BLOCK_N))
                        if ws > 1 and _in_kernel_waits_ok(ctx) else 0),
            cta_pairs=rs_uses_cta_pairs(ws),
            group_m_tiles=gm, sig_local=sig_ptr, heap_stride=stride, sig_stride=MAX_GROUPS,
            stage_local=stage_ptr, status_ptr=status_block(ctx).data_ptr(), stats_ptr=stats_block(ctx).data_ptr(),
            wait_budget_ns=wait_budget_ns()))
    plan = st["plan"]
    if ctx.local_group is None and "fast" not in st:
        def fast(_plan=plan, _sig=sigst):
            _sig["epoch"] += 1
            _plan.launch(epoch=_sig["epoch"])

        st["fast"] = fast
    sigst["epoch"] += 1
    epoch = sigst["epoch"]
    if a_host is not None and (ws == 1 or (_in_kernel_waits_ok(ctx) and not ctx.is_single_process)):
        phases = [_on_device(ctx, lambda: launch_streamed(ctx, plan, A, a_host, epoch=epoch,
                                                          order=a_host_order))]
    elif ws == 1 or _in_kernel_waits_ok(ctx):
        if a_host is not None:
            A.copy_(a_host, non_blocking=True)
        phases = [_on_device(ctx, lambda: plan.launch(epoch=epoch))]
    else:
        if a_host is not None:
            A.copy_(a_host, non_blocking=True)
        # Emulated ranks: peers' tiles for everybody first, then each owner's own (reducing) tiles.
        n_remote = plan.tiles_per_owner * (ws - 1)
        phases = [_on_device(ctx, lambda: plan.launch(epoch=epoch, tile_begin=0, tile_end=n_remote)),
                  _on_device(ctx, lambda: plan.launch(epoch=epoch, tile_begin=n_remote))]
    run_phases(ctx, ("reduce_scatter", name, M, N, K, split_axis, epoch), phases)
    sf = getattr(plan, "_stream_fast", None)
    if (a_host is not None and sf is not None and ctx.local_group is None
            and (ws == 1 or _in_kernel_waits_ok(ctx))):
        launcher = sf[1]

        def fast_host(_sig=sigst):
            _sig["epoch"] += 1
            launcher(_sig["epoch"], 0, 0)

        st["fast_host"] = ((a_host.data_ptr(), a_host_order), fast_host)


# --------------------------------------------------------------------------
# all-scatter: full product kept locally, this rank's column slice pushed to all
# --------------------------------------------------------------------------
def all_scatter(ctx, name: str, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, *,
                col_begin: int, col_end: int, b_is_nk: bool = False,
                push_mode: Optional[int] = None, wait: bool = True, grid: int = 0) -> None:
    _require_2d("A", A, ctx)
    _require_2d("B", B, ctx)
    _require_2d("C", C, ctx)
    K, N = _b_dims(B, b_is_nk)
    M = A.shape[0]
    ws, rank = ctx.world_size, ctx.rank
    if ws > 1 and not ctx.is_symmetric(C):
        raise ValueError("C must be allocated from the symmetric heap (ctx.zeros / ctx.empty)")
    push_mode = default_push_mode(ctx) if push_mode is None else push_mode
    key = ("all_scatter", name, A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, A.stride(0),
           B.stride(0), C.stride(0), A.dtype, b_is_nk, col_begin, col_end, push_mode, grid)
    st = op_state(ctx, key)
    m_tiles = -(-M // fg.BLOCK_M)
    gm = default_group_m_tiles(m_tiles, -(-N // fg.BLOCK_N), A.element_size())
    sigst = _signal_state(ctx, f"all_scatter:{name}:{M}x{N}x{K}:g{gm}") if ws > 1 else st
    if "plan" not in st:
        if ws > 1:
            sig = sigst["sig"]
            dests = _heap_offset_ptrs(ctx, C)
            mc = ctx.heap.multicast_ptr(C.data_ptr()) if push_mode == fg.PUSH_MULTIMEM else 0
            sig_ptr, stride = sig.data_ptr(), ctx.heap.stride
            st["sig"] = sig
        else:
            dests, mc, sig_ptr, stride = [C.data_ptr()], 0, 0, 0
        st["plan"] = fg.FusedGemmPlan(fg.FusedGemmSpec(
            mode=fg.MODE_ALL_SCATTER if ws > 1 else fg.MODE_GEMM, dtype=A.dtype,
            a_ptr=A.data_ptr(), a_rows=M, lda=A.stride(0), b_ptr=B.data_ptr(), b_cols=N,
            ldb=B.stride(0), k=K, sub_m=M, sub_n=N, out_ptrs=dests, ldo=C.stride(0), out_rows=M,
            out_cols=N, b_kmajor=b_is_nk, push_mode=push_mode, rank=rank, world_size=ws,
            out_mc_ptr=mc, group_m_tiles=gm, sig_local=sig_ptr, heap_stride=stride,
            sig_stride=MAX_GROUPS, scatter_col_begin=col_begin, scatter_col_end=col_end,
            entry_local=entry_ptr(ctx, sigst) if ws > 1 else 0, grid=grid,
            status_ptr=status_block(ctx).data_ptr(), stats_ptr=stats_block(ctx).data_ptr(), wait_budget_ns=wait_budget_ns()))
        plan = st["plan"]
        if ws > 1:
            # A tile signals once per slab whether or not it overlaps the pushed slice, so the
            # count per group is the same as for push-all.
            per_epoch = [plan.group_m_count(g) * plan.n_tiles_local * fg.EPILOGUE_SLABS
                         for g in range(plan.groups)]
            st["per_epoch"] = torch.tensor(per_epoch, dtype=torch.int32, device=ctx.torch_device)
    plan = st["plan"]
    sigst["epoch"] += 1
    epoch = sigst["epoch"]
    phases = [_on_device(ctx, lambda: plan.launch(epoch=epoch))]
    if ws > 1 and wait:
        phases.append(_on_device(ctx, lambda: wait_groups(ctx, st["sig"], plan.groups,
                                                          st["per_epoch"], epoch)))
    run_phases(ctx, ("all_scatter", name, M, N, K, epoch), phases)


# --------------------------------------------------------------------------
# two-kernel all-scatter: GEMM kernel + region-push kernel
# --------------------------------------------------------------------------
_COLL_COUNTER_WORDS = 32


def _comm_stream(ctx) -> torch.cuda.Stream:
    s = ctx._state.get("comm_stream")
    if s is None:
        with torch.cuda.device(ctx.torch_device):
            s = torch.cuda.Stream()
        ctx._state["comm_stream"] = s
    return s


def gemm_then_push(ctx, name: str, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, *,
                   col_begin: int, col_end: int, overlapped: bool, b_is_nk: bool = False,
                   use_multimem: Optional[bool] = None, gemm_grid: int = 0,
                   push_grid: int = 0) -> None:
    """All-scatter as two kernels: ``C = A @ B`` locally, then columns
    ``[col_begin, col_end)`` of ``C`` are copied to every peer.

    ``overlapped=False``: the push kernel follows the GEMM in stream order (bulk-synchronous).
    ``overlapped=True``: the GEMM publishes each finished band of 128 rows on a local counter
    and the push kernel, on a second stream, sends a band as soon as its counter is complete
    (producer / consumer).
    """
    _require_2d("A", A, ctx)
    _require_2d("B", B, ctx)
    _require_2d("C", C, ctx)
    K, N = _b_dims(B, b_is_nk)
    M = A.shape[0]
    ws, rank = ctx.world_size, ctx.rank
    if ws > 1 and not ctx.is_symmetric(C):
        raise ValueError("C must be allocated from the symmetric heap (ctx.zeros / ctx.empty)")
    width = col_end - col_begin
    if ws > 1 and (width <= 0 or (width * C.element_size()) % 16 or (col_begin * C.element_size()) % 16):
        raise ValueError("the pushed column slice must start and end on 16-byte boundaries")
    key = ("gemm_then_push", name, A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, A.stride(0),
           B.stride(0), C.stride(0), A.dtype, b_is_nk, col_begin, col_end, overlapped, gemm_grid)
    st = op_state(ctx, key)
    m_tiles = -(-M // fg.BLOCK_M)
    shared = op_state(ctx, ("gemm_then_push:sig", name, M, N, K, overlapped))
    if "plan" not in st:
        if ws > 1 and "counters" not in shared:
            shared["counters"] = ctx.workspace(f"push:{name}:{M}x{N}x{K}:{overlapped}",
                                               _COLL_COUNTER_WORDS, dtype=torch.int32)
            shared["bands"] = (torch.zeros(m_tiles, dtype=torch.int32, device=ctx.torch_device)
                               if overlapped else None)
        bands = shared.get("bands")
        st["plan"] = fg.FusedGemmPlan(fg.FusedGemmSpec(
            mode=fg.MODE_GEMM, dtype=A.dtype, a_ptr=A.data_ptr(), a_rows=M, lda=A.stride(0),
            b_ptr=B.data_ptr(), b_cols=N, ldb=B.stride(0), k=K, sub_m=M, sub_n=N,
            out_ptrs=[C.data_ptr()], ldo=C.stride(0), out_rows=M, out_cols=N, b_kmajor=b_is_nk,
            rank=rank, world_size=ws, group_m_tiles=1, grid=gemm_grid,
            sig_local=bands.data_ptr() if (bands is not None and ws > 1) else 0,
            sig_stride=m_tiles, status_ptr=status_block(ctx).data_ptr(), stats_ptr=stats_block(ctx).data_ptr(),
            wait_budget_ns=wait_budget_ns()))
    plan = st["plan"]
    if ws == 1:
        plan.launch()
        return
    shared["epoch"] += 1
    epoch = shared["epoch"]
    if use_multimem is None:
        use_multimem = default_push_mode(ctx) == fg.PUSH_MULTIMEM
    region = C.data_ptr() + col_begin * C.element_size()
    mc_region = ctx.heap.multicast_ptr(region) if use_multimem else 0
    bands = shared.get("bands")
    band_ready = bands.data_ptr() if bands is not None else 0
    per_band = plan.n_tiles_local * fg.EPILOGUE_SLABS
    grid = max(1, min(m_tiles, push_grid or 32))
    counters = shared["counters"].data_ptr()
    status = status_block(ctx).data_ptr()

    def push(mask: int, stream=None):
        def go():
            s = stream if stream is not None else torch.cuda.current_stream()
            _native.call("tccl_push_region", region, mc_region, C.stride(0) * C.element_size(), M,
                         width * C.element_size(), fg.BLOCK_M, rank, ws, ctx.heap.stride,
                         band_ready, per_band, counters, epoch & 0xFFFFFFFF, mask, grid, status,
                         wait_budget_ns(), s.cuda_stream)
        return go

    gemm_launch = _on_device(ctx, lambda: plan.launch(epoch=epoch))
    if ctx.emulated:
        phases = [gemm_launch, _on_device(ctx, push(1)), _on_device(ctx, push(2)),
                  _on_device(ctx, push(4))]
    elif overlapped:
        def both():
            main = torch.cuda.current_stream()
            comm = _comm_stream(ctx)
            comm.wait_stream(main)          # operands and C are ready for this call
            plan.launch(epoch=epoch)        # producer first ...
            push(7, comm)()                 # ... consumer second, on its own stream
            main.wait_stream(comm)
        phases = [_on_device(ctx, both)]
    else:
        phases = [gemm_launch, _on_device(ctx, push(7))]
    run_phases(ctx, ("gemm_then_push", name, M, N, K, overlapped, epoch), phases)
