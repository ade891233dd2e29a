#!/usr/bin/env python
"""Per-tile timeline of the fused GEMM + collective kernel on real ranks.

The kernel can stamp %globaltimer four times per tile and epilogue warp
(accumulator ready / stores issued / older bulk stores complete / signalled).
This script runs one all-gather shape and one reduce-scatter shape with the
stamps on and prints, per phase, the median and mean time an epilogue warp
spends in each section, plus when the CTAs finish: enough to see whether a run
is bound by the tensor cores (long waits for the accumulator), by NVLink (long
waits for bulk-store completion) or by signalling.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/trace_fused_gemm.py --ag 16384,4096,1024 --rs 16384,4096,2048
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _write_timeline(path, label, plan, t, rank, max_ctas=16):
    """Device-clock timeline (one lane per CTA, epilogue warp 0): a span per tile from
    "accumulator ready" to "signalled", written with planning.runtime.TimelineRecorder."""
    from tileccl_b200.planning.runtime.timeline import TimelineRecorder

    rec = TimelineRecorder(benchmark="trace_fused_gemm", path_name=label,
                           metadata={"clock": "%globaltimer", "rank": rank, "grid": plan.grid})
    t0 = t[:, :, 0][t[:, :, 0] > 0].min()
    for b in range(min(plan.grid, max_ctas)):
        for i in range(b, t.shape[0], plan.grid):
            a, s3 = t[i, 0, 0], t[i, 0, 3]
            if a > 0 and s3 > 0:
                rec.record_span(name=f"tile{i}", lane=f"cta{b}", start_ms=(a - t0) / 1e6,
                                end_ms=(s3 - t0) / 1e6, category="epilogue", rank=rank,
                                source="device_globaltimer", tile_range={"tile": i})
    rec.write_json(path)


def _summary(label, plan, trace, tiles, ms, rank, timeline=None):
    t = trace.cpu().numpy().astype(np.int64).reshape(tiles, 4, 4)
    if timeline and rank == 0:
        _write_timeline(timeline, label, plan, t, rank)
    t0 = t[:, :, 0][t[:, :, 0] > 0].min()
    rel = (t - t0) / 1e3
    grid = plan.grid
    acc_wait, issue, compl, sig = [], [], [], []
    for b in range(grid):
        for w in range(4):
            prev = None
            for i in range(b, tiles, grid):
                a, s1, s2, s3 = rel[i, w]
                if prev is not None:
                    acc_wait.append(a - prev)
                issue.append(s1 - a)
                if t[i, w, 2] > 0:
                    compl.append(s2 - s1)
                    sig.append(s3 - s2)
                else:
                    sig.append(s3 - s1)
                prev = s3
    ends = np.array([rel[b::grid][:, :, 3].max() for b in range(grid)])

    def mm(x):
        return (float(np.median(x)), float(np.mean(x))) if len(x) else (-1.0, -1.0)

    if rank == 0:
        print(f"{label}: event time {ms * 1e3:.1f} us | last stamp {rel[:, :, 3].max():.1f} us | "
              f"CTA end min/med/max {ends.min():.1f}/{np.median(ends):.1f}/{ends.max():.1f} us")
        print("   per tile and epilogue warp, median/mean us: wait for accumulator %.2f/%.2f, "
              "TMEM->smem->stores issued %.2f/%.2f, wait for older bulk stores %.2f/%.2f, "
              "signal %.2f/%.2f" % (*mm(acc_wait), *mm(issue), *mm(compl), *mm(sig)), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ag", default="16384,4096,1024", help="M,N,K of the GEMM + all-gather")
    ap.add_argument("--rs", default="16384,4096,2048", help="M,N,K of the GEMM -> reduce-scatter")
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--timeline", default=None,
                    help="write rank 0's per-CTA timeline of the all-gather run to this JSON file")
    args = ap.parse_args()
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

    M, N, K = (int(x) for x in args.ag.split(","))
    mloc = M // ws
    A = (torch.randn(mloc, K, device=dev) / K ** 0.5).half()
    B = torch.randn(K, N, device=dev).half()
    C = ctx.zeros(M, N, dtype=torch.float16)
    sig = ctx.zeros(ws * _fused.MAX_GROUPS, dtype=torch.int32)
    m_tiles, n_tiles = -(-mloc // fg.BLOCK_M), -(-N // fg.BLOCK_N)
    tiles = m_tiles * n_tiles
    trace = torch.zeros(tiles * 16, dtype=torch.int64, device=dev)
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
    _summary(f"GEMM+AG {M}x{N}x{K} ws={ws}", plan, trace, tiles, ms, rank, args.timeline)
    dist.barrier()

    M, N, K = (int(x) for x in args.rs.split(","))
    kloc, sub_m = K // ws, M // ws
    A = (torch.randn(M, kloc, device=dev) / K ** 0.5).half()
    B = torch.randn(kloc, N, device=dev).half()
    C = torch.zeros(sub_m, N, device=dev, dtype=torch.float16)
    sig = ctx.zeros(ws * _fused.MAX_GROUPS, dtype=torch.int32)
    stage = ctx.zeros(2 * ws * sub_m * N, dtype=torch.float16)
    dests = _fused._heap_offset_ptrs(ctx, stage)
    dests[rank] = C.data_ptr()
    m_tiles, n_tiles = -(-sub_m // fg.BLOCK_M), -(-N // fg.BLOCK_N)
    tiles = m_tiles * n_tiles * ws
    trace = torch.zeros(tiles * 16, dtype=torch.int64, device=dev)
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
    _summary(f"GEMM->RS {M}x{N}x{K} ws={ws} own_lag={lag}", plan, trace, tiles, ms, rank)
    _fused.check_status(ctx)
    dist.barrier()
    ctx.heap.cleanup()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
