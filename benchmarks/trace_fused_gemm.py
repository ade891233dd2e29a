#!/usr/bin/env python
"""Per-tile timeline of the fused GEMM + collective kernel on real ranks.

The kernel can stamp %globaltimer four times per tile and epilogue warp
(accumulator ready / stores issued / older bulk stores complete / signalled)
and four times per CTA (kernel entry / roles start / incoming TileGroups seen /
exit).  This script runs all-gather and reduce-scatter shapes with the stamps
on, in the kernel form the operators use (CTA pairs), and prints where the time
of one call goes: launch latency, the head before the first bulk store, the
link-bound body, the tail after the last store, plus the median time an
epilogue warp spends in each section.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/trace_fused_gemm.py --ag 16384,4096,1024 --rs 16384,4096,2048

Several shapes: separate them with ';'.  ``--one-cta`` traces the one-CTA form.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _slots_of_cta(plan, pair, b, n_slots):
    """Trace slots (128-row tiles) that CTA `b` works on, in its visiting order."""
    if pair:
        pairs = plan.pair_grid // 2
        return [2 * t + (b & 1) for t in range(b >> 1, n_slots // 2, pairs)]
    return list(range(b, n_slots, plan.grid))


def _write_timeline(path, label, plan, pair, t, rank, n_slots, max_ctas=16):
    """Device-clock timeline (one lane per CTA, epilogue warp 0): a span per tile from
    "accumulator ready" to "signalled", written with planning.runtime.TimelineRecorder."""
    from tileccl_b200.planning.runtime.timeline import TimelineRecorder

    grid = plan.pair_grid if pair else plan.grid
    rec = TimelineRecorder(benchmark="trace_fused_gemm", path_name=label,
                           metadata={"clock": "%globaltimer", "rank": rank, "grid": grid})
    t0 = t[:, :, 0][t[:, :, 0] > 0].min()
    for b in range(min(grid, max_ctas)):
        for i in _slots_of_cta(plan, pair, b, n_slots):
            a, s3 = t[i, 0, 0], t[i, 0, 3]
            if a > 0 and s3 > 0:
                rec.record_span(name=f"tile{i}", lane=f"cta{b}", start_ms=(a - t0) / 1e6,
                                end_ms=(s3 - t0) / 1e6, category="epilogue", rank=rank,
                                source="device_globaltimer", tile_range={"tile": i})
    rec.write_json(path)


def summarize(label, plan, pair, trace, ms, rank, timeline=None):
    """Reduce one traced launch to a dict of microsecond figures (and print it on rank 0)."""
    grid = plan.pair_grid if pair else plan.grid
    raw = trace.cpu().numpy().astype(np.int64)
    n_slots = (2 * ((plan.m_tiles_local + 1) // 2) * plan.n_tiles_local * plan.owners if pair
               else plan.tiles_total)
    t = raw[:n_slots * 16].reshape(n_slots, 4, 4)
    cta = raw[n_slots * 16:n_slots * 16 + grid * 8].reshape(grid, 8)
    if timeline and rank == 0:
        _write_timeline(timeline, label, plan, pair, t, rank, n_slots)
    entry0 = cta[:, 0][cta[:, 0] > 0].min()
    rel = (t - entry0) / 1e3
    rel[t == 0] = np.nan
    crel = (cta - entry0) / 1e3
    crel[cta == 0] = np.nan
    acc_wait, issue, compl, sig = [], [], [], []
    from tileccl_b200.utils.config import current

    dynamic = current().dynamic_tiles
    if dynamic:
        # tiles are handed out at run time: no fixed per-CTA sequence to walk, so only the
        # per-tile sections are summarised (not the wait between a CTA's consecutive tiles)
        for i in range(n_slots):
            for w in range(4):
                a, s1, s2, s3 = rel[i, w]
                if np.isnan(a):
                    continue
                issue.append(s1 - a)
                if not np.isnan(s2):
                    compl.append(s2 - s1)
                    sig.append(s3 - s2)
                else:
                    sig.append(s3 - s1)
    for b in range(0 if dynamic else grid):
        for w in range(4):
            prev = None
            for i in _slots_of_cta(plan, pair, b, n_slots):
                a, s1, s2, s3 = rel[i, w]
                if np.isnan(a):
                    continue
                if prev is not None:
                    acc_wait.append(a - prev)
                issue.append(s1 - a)
                if not np.isnan(s2):
                    compl.append(s2 - s1)
                    sig.append(s3 - s2)
                else:
                    sig.append(s3 - s1)
                prev = s3

    def med(x):
        return round(float(np.median(x)), 2) if len(x) else None

    out = {
        "label": label, "event_us": round(ms * 1e3, 1), "grid": grid, "pair": pair,
        "dynamic_tiles": dynamic,
        "cta_entry_spread_us": round(float(np.nanmax(crel[:, 0])), 2),
        "roles_start_us": round(float(np.nanmedian(crel[:, 1])), 2),
        "first_acc_ready_us": round(float(np.nanmin(rel[:, :, 0])), 2),
        "median_first_acc_ready_us": round(float(np.nanmedian(
            np.sort(np.nanmin(rel[:, :, 0], axis=1))[:max(1, grid // (2 if pair else 1))])), 2),
        "last_acc_ready_us": round(float(np.nanmax(rel[:, :, 0])), 2),
        "last_stores_issued_us": round(float(np.nanmax(rel[:, :, 1])), 2),
        "last_signal_us": round(float(np.nanmax(rel[:, :, 3])), 2),
        "incoming_seen_us": (round(float(np.nanmax(crel[:, 2])), 2)
                             if not np.all(np.isnan(crel[:, 2])) else None),
        "epilogue_done_us": round(float(np.nanmax(crel[:, 4:8])), 2),
        "epilogue_done_min_us": round(float(np.nanmin(np.nanmax(crel[:, 4:8], axis=1))), 2),
        "median_wait_acc_us": med(acc_wait), "median_issue_us": med(issue),
        "median_wait_older_stores_us": med(compl), "median_signal_us": med(sig),
    }
    end = max(out["epilogue_done_us"], out["incoming_seen_us"] or 0.0)
    out["event_minus_kernel_span_us"] = round(out["event_us"] - end, 1)
    # how long this rank sat waiting for its peers' data after its own pushes were done
    out["wait_for_peers_us"] = (round(out["incoming_seen_us"] - out["epilogue_done_us"], 2)
                                if out["incoming_seen_us"] is not None else None)
    if dist.is_initialized() and dist.get_world_size() > 1:
        rows = [None] * dist.get_world_size()
        dist.all_gather_object(rows, {k: out[k] for k in ("event_us", "epilogue_done_us",
                                                          "incoming_seen_us", "wait_for_peers_us",
                                                          "first_acc_ready_us")})
        for k in ("event_us", "epilogue_done_us", "incoming_seen_us", "wait_for_peers_us"):
            vals = [r[k] for r in rows if r[k] is not None]
            if vals:
                out[f"{k}_ranks_min_max"] = [min(vals), max(vals)]
    if rank == 0:
        print(json.dumps(out), flush=True)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ag", default="16384,4096,1024", help="M,N,K of the GEMM + all-gather (';'-separated list)")
    ap.add_argument("--rs", default="16384,4096,2048", help="M,N,K of the GEMM -> reduce-scatter (';'-separated list)")
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--one-cta", action="store_true", help="trace the one-CTA form of the kernel")
    ap.add_argument("--steady", action="store_true",
                    help="launch the iterations back to back (flush, launch, flush, launch ...) "
                         "without a barrier in between, as a training loop would, and trace the last")
    ap.add_argument("--timeline", default=None,
                    help="write rank 0's per-CTA timeline of the first all-gather run to this JSON file")
    args = ap.parse_args()
    if args.one_cta:
        os.environ["TILECCL_GEMM_2SM"] = "0"
    rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import tileccl_b200 as tccl
    from tileccl_b200.kernels import fused_gemm as fg
    from tileccl_b200.ops import _fused

    ctx = tccl.init(heap_size=3 << 30)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    status = _fused.status_block(ctx).data_ptr()

    def timed(plan, trace, **kw):
        ep = 0
        if args.steady:
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            for _ in range(max(args.iters, 2)):
                ep += 1
                flush.zero_()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                plan.launch(epoch=ep, **kw)
                e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e)
        for _ in range(args.iters):
            ep += 1
            flush.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            trace.zero_()
            torch.cuda.synchronize()
            flush[:64 << 20].zero_()
            s.record()
            plan.launch(epoch=ep, **kw)
            e.record()
            torch.cuda.synchronize()
        return s.elapsed_time(e)

    def trace_buffer(m_tiles, n_tiles, owners):
        words = 2 * ((m_tiles + 1) // 2) * n_tiles * owners * 16 + 8 * 1024
        return torch.zeros(words, dtype=torch.int64, device=dev)

    first = True
    for shape in [s for s in args.ag.split(";") if s]:
        M, N, K = (int(x) for x in shape.split(","))
        mloc = M // ws
        A = (torch.randn(mloc, K, device=dev) / K ** 0.5).half()
        B = torch.randn(K, N, device=dev).half()
        C = ctx.zeros(M, N, dtype=torch.float16)
        sig = ctx.zeros(ws * _fused.MAX_GROUPS, dtype=torch.int32)
        m_tiles, n_tiles = -(-mloc // fg.BLOCK_M), -(-N // fg.BLOCK_N)
        trace = trace_buffer(m_tiles, n_tiles, 1)
        region = rank * mloc * N * 2
        plan = fg.FusedGemmPlan(fg.FusedGemmSpec(
            mode=fg.MODE_PUSH_ALL, dtype=torch.float16, a_ptr=A.data_ptr(), a_rows=mloc, lda=K,
            b_ptr=B.data_ptr(), b_cols=N, ldb=N, k=K, sub_m=mloc, sub_n=N,
            out_ptrs=_fused._heap_offset_ptrs(ctx, C, region), ldo=N, out_rows=mloc, out_cols=N,
            push_mode=_fused.default_push_mode(ctx), rank=rank, world_size=ws,
            group_m_tiles=_fused.default_group_m_tiles(m_tiles), sig_local=sig.data_ptr(),
            heap_stride=ctx.heap.stride, sig_stride=_fused.MAX_GROUPS, trace_ptr=trace.data_ptr(),
            status_ptr=status))
        ms = timed(plan, trace, wait_incoming=True)
        summarize(f"GEMM+AG {M}x{N}x{K} ws={ws}", plan, plan.pair_kernel, trace, ms, rank,
                  args.timeline if first else None)
        first = False
        dist.barrier()
        del plan

    for shape in [s for s in args.rs.split(";") if s]:
        M, N, K = (int(x) for x in shape.split(","))
        kloc, sub_m = K // ws, M // ws
        A = (torch.randn(M, kloc, device=dev) / K ** 0.5).half()
        B = torch.randn(kloc, N, device=dev).half()
        C = torch.zeros(sub_m, N, device=dev, dtype=torch.float16)
        sig = ctx.zeros(ws * _fused.MAX_GROUPS, dtype=torch.int32)
        stage = ctx.zeros(2 * ws * sub_m * N, dtype=torch.float16)
        dests = _fused._heap_offset_ptrs(ctx, stage)
        dests[rank] = C.data_ptr()
        m_tiles, n_tiles = -(-sub_m // fg.BLOCK_M), -(-N // fg.BLOCK_N)
        trace = trace_buffer(m_tiles, n_tiles, ws)
        lag = _fused.default_rs_own_lag(ws, m_tiles, n_tiles)
        plan = fg.FusedGemmPlan(fg.FusedGemmSpec(
            mode=fg.MODE_REDUCE_SCATTER, dtype=torch.float16, a_ptr=A.data_ptr(), a_rows=M, lda=kloc,
            b_ptr=B.data_ptr(), b_cols=N, ldb=N, k=kloc, sub_m=sub_m, sub_n=N, out_ptrs=dests, ldo=N,
            out_rows=sub_m, out_cols=N, push_mode=_fused.default_push_mode(ctx), rank=rank,
            world_size=ws, split_axis=0, out_slot_elems=sub_m * N, out_slots=2 * ws,
            group_m_tiles=_fused.default_group_m_tiles(m_tiles), sig_local=sig.data_ptr(),
            heap_stride=ctx.heap.stride, sig_stride=_fused.MAX_GROUPS, stage_local=stage.data_ptr(),
            rs_own_lag=lag, ident_ptr=fg.identity_operand(torch.float16, dev).data_ptr(),
            trace_ptr=trace.data_ptr(), status_ptr=status))
        ms = timed(plan, trace)
        summarize(f"GEMM->RS {M}x{N}x{K} ws={ws} own_lag={lag}", plan, plan.pair_kernel, trace, ms,
                  rank)
        dist.barrier()
        del plan
    _fused.check_status(ctx)
    dist.barrier()
    ctx.heap.cleanup()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
