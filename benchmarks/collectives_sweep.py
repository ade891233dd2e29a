#!/usr/bin/env python
"""Tile-collective sweep: allreduce(sum), allgather, reduce_scatter, broadcast(root 0),
scatter on symmetric-heap buffers, 4 KiB .. 1 GiB in powers of two, fp16 and fp32, values
U(-1, 1) seeded per rank.  Columns: this library, NCCL on the same buffers, and (separate
run, ``--impl reference``) the reference's Triton collectives.  One process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/collectives_sweep.py [--max-bytes 1073741824] [--out sweep.json]
    python -m torch.distributed.run ... benchmarks/collectives_sweep.py --impl reference \
        --max-bytes 16777216 --out sweep_reference.json          # N = 2 only (its validated surface)

"bytes" is the size of the full buffer (allreduce / broadcast: the tensor; allgather: the
gathered output; reduce_scatter / scatter: the input).  Device time (CUDA events around
`iters` back-to-back calls, max over ranks, median of three batches); bus GB/s uses the usual factors (allreduce
2(n-1)/n, allgather / reduce_scatter / scatter (n-1)/n, broadcast 1).  Every row of this
library is checked once against NCCL's result on the same inputs before it is timed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def timed(fn, iters, dev, batches=3):
    """Per-call device time: `batches` batches of `iters` back-to-back calls, each between two
    CUDA events; per batch the max over ranks, then the median over batches (one stalled
    iteration on a shared host otherwise decides a whole row, for either library)."""
    for _ in range(3):
        fn()
    per_batch = []
    for _ in range(batches):
        torch.cuda.synchronize()
        dist.barrier()
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        per_batch.append(s.elapsed_time(e) / iters)
    t = torch.tensor(per_batch, dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.median().item())


def sizes(lo, hi, step):
    n = lo
    while n <= hi:
        yield n
        n *= step


def rel_err(got, ref):
    return float((got.float() - ref.float()).abs().max() / (ref.float().abs().max() + 1e-9))


def sweep_ours(args, rank, ws, dev):
    sys.path.insert(0, ROOT)
    import tileccl_b200 as tccl
    from tileccl_b200 import ops
    from tileccl_b200.primitives import collectives as coll

    ctx = tccl.init(heap_size=int(2.5 * args.max_bytes) + (64 << 20))
    rows = []
    for nbytes in sizes(args.min_bytes, args.max_bytes, args.step):
        for dtype in args.dtype_list:
            es = torch.empty((), dtype=dtype).element_size()
            n = max(ws, nbytes // es // ws * ws)
            ctx.barrier()
            ctx.heap.reset_allocator()           # drops the library's own workspaces as well
            full = ctx.empty(n, dtype=dtype)
            part = ctx.zeros(n // ws, dtype=dtype)
            ref_full = torch.empty(n, dtype=dtype, device=dev)
            ref_part = torch.empty(n // ws, dtype=dtype, device=dev)

            def fill():
                gen = torch.Generator(device=dev).manual_seed(7 + rank)
                full.copy_(torch.rand(n, device=dev, generator=gen) * 2 - 1)
                part.copy_(full[:n // ws] * 0.5)
                ref_full.copy_(full)
                ref_part.copy_(part)

            ctx.barrier()
            iters = 20 if nbytes <= (16 << 20) else (5 if nbytes <= (256 << 20) else 3)
            tol = 2e-2 if dtype is torch.float16 else 1e-5
            cases = {
                "allreduce": (lambda: ops.allreduce(full, ctx=ctx), lambda: dist.all_reduce(ref_full),
                              2 * (ws - 1) / ws, lambda: rel_err(full, ref_full)),
                "allgather": (lambda: ops.allgather(part, full, ctx=ctx),
                              lambda: dist.all_gather_into_tensor(ref_full, ref_part), (ws - 1) / ws,
                              lambda: rel_err(full, ref_full)),
                "reduce_scatter": (lambda: ops.reduce_scatter(full, part, ctx=ctx),
                                   lambda: dist.reduce_scatter_tensor(ref_part, ref_full),
                                   (ws - 1) / ws, lambda: rel_err(part, ref_part)),
                "broadcast": (lambda: ops.broadcast(full, ctx=ctx, root=0),
                              lambda: dist.broadcast(ref_full, src=0), 1.0,
                              lambda: rel_err(full, ref_full)),
                "scatter": (lambda: ops.scatter(full, part, ctx=ctx, root=0), None, (ws - 1) / ws,
                            None),
            }
            for name, (ours, nccl, factor, check) in cases.items():
                if name not in args.op_list:
                    continue
                fill()
                ctx.barrier()
                ours()
                err = None
                if nccl is not None:
                    nccl()
                    torch.cuda.synchronize()
                    err = check()
                else:                              # scatter: compare with the root's slice
                    root_full = ref_full.clone()
                    dist.broadcast(root_full, src=0)
                    err = rel_err(part, root_full[rank * (n // ws):(rank + 1) * (n // ws)])
                # a device wait that gave up (status words) fails the row on every rank
                # instead of being timed 20 more times
                status = ctx.heap._state.get("status")
                gave_up = 0.0 if status is None or int(status[0]) == 0 else 1.0
                e = torch.tensor([err, gave_up], dtype=torch.float64, device=dev)
                dist.all_reduce(e, op=dist.ReduceOp.MAX)
                err, gave_up = float(e[0].item()), float(e[1].item())
                row = {"collective": name, "bytes": n * es, "dtype": str(dtype).split(".")[-1],
                       "world_size": ws, "max_rel_err_vs_nccl": err, "correct": bool(err <= tol)}
                if gave_up:
                    if status is not None:
                        row["error"] = f"device wait timed out, status words {status.tolist()}"
                        status.zero_()
                    else:
                        row["error"] = "device wait timed out on a peer"
                    row["correct"] = False
                    rows.append(row)
                    ctx.barrier()
                    continue
                ms = timed(ours, iters, dev)
                row.update(ms=ms, bus_gbps=n * es * factor / ms / 1e6)
                if nccl is not None:
                    ms_n = timed(nccl, iters, dev)
                    row.update(nccl_ms=ms_n, nccl_bus_gbps=n * es * factor / ms_n / 1e6)
                rows.append(row)
            coll.check_status(ctx.heap)
    from tileccl_b200.utils.config import current

    cfg = current()
    payload = {"suite": "collectives_sweep", "impl": "ours", "world_size": ws,
               "nvls": ctx.heap.has_multicast and not cfg.disable_nvls,
               "switches": {"disable_nvls": cfg.disable_nvls, "ll_max_bytes": cfg.ll_max_bytes,
                            "bcast_relay_min_bytes": cfg.bcast_relay_min_bytes},
               "rows": rows}
    ctx.barrier()
    ctx.heap.cleanup()
    return payload


def sweep_reference(args, rank, ws, dev):
    """The reference's Triton tile collectives through its own API (multi-process, which it
    validates for two ranks).  A row that raises, or a sweep that runs out of its time budget,
    is recorded as such instead of stopping the run."""
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    import tileccl
    from tileccl.primitives import collectives as rcoll

    # its allocator never frees: room for every size's buffers
    ctx = tileccl.init(backend="cuda", heap_size=8 * args.max_bytes + (64 << 20))
    rows, t_start = [], time.time()
    for nbytes in sizes(args.min_bytes, args.max_bytes, args.step):
        for dtype in args.dtype_list:
            es = torch.empty((), dtype=dtype).element_size()
            n = max(ws, nbytes // es // ws * ws)
            full = ctx.zeros(n, dtype=dtype)
            part = ctx.zeros(n // ws, dtype=dtype)
            gen = torch.Generator(device=dev).manual_seed(7 + rank)
            full.copy_(torch.rand(n, device=dev, generator=gen) * 2 - 1)
            cases = {
                "allreduce": (lambda: tileccl.ops.allreduce(full, ctx=ctx), 2 * (ws - 1) / ws),
                "allgather": (lambda: tileccl.ops.allgather(part, full, ctx=ctx), (ws - 1) / ws),
                "reduce_scatter": (lambda: tileccl.ops.reduce_scatter(full, part, ctx=ctx),
                                   (ws - 1) / ws),
                "broadcast": (lambda: rcoll.broadcast(full, ctx.heap, root=0), 1.0),
                "scatter": (lambda: rcoll.scatter(full, part, ctx.heap, root=0), (ws - 1) / ws),
            }
            for name, (fn, factor) in cases.items():
                if name not in args.op_list:
                    continue
                row = {"collective": name, "bytes": n * es, "dtype": str(dtype).split(".")[-1],
                       "world_size": ws}
                flag = torch.tensor([1.0 if time.time() - t_start > args.time_budget_s else 0.0],
                                    device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)
                if flag.item() > 0:
                    row["skipped"] = "time budget of the reference sweep used up"
                    rows.append(row)
                    continue
                try:
                    ms = timed(fn, 5 if nbytes > (1 << 20) else 10, dev)
                    row.update(ms=ms, bus_gbps=n * es * factor / ms / 1e6)
                except Exception as exc:        # every rank runs the same code, so all of them raise
                    row["error"] = f"{type(exc).__name__}: {exc}"[:200]
                rows.append(row)
    return {"suite": "collectives_sweep", "impl": "reference", "world_size": ws, "rows": rows}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=4096)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--step", type=int, default=2, help="ratio between consecutive sizes")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--time-budget-s", type=float, default=240.0, help="reference sweep only")
    ap.add_argument("--ops", default="allreduce,allgather,reduce_scatter,broadcast,scatter",
                    help="comma-separated subset of the five collectives")
    ap.add_argument("--dtypes", default="float16,float32")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    args.op_list = [o.strip() for o in args.ops.split(",") if o.strip()]
    args.dtype_list = [getattr(torch, d.strip()) for d in args.dtypes.split(",") if d.strip()]
    rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    payload = (sweep_ours if args.impl == "ours" else sweep_reference)(args, rank, ws, dev)
    if rank == 0:
        for r in payload["rows"]:
            if "ms" not in r:
                print(f"{r['collective']:<15s} {r['dtype']:<8s} {r['bytes']:>11d} B  "
                      f"{r.get('error') or r.get('skipped')}")
                continue
            print(f"{r['collective']:<15s} {r['dtype']:<8s} {r['bytes']:>11d} B  {args.impl} "
                  f"{r['ms'] * 1e3:9.1f} us {r['bus_gbps']:7.1f} GB/s"
                  + (f"   nccl {r['nccl_ms'] * 1e3:9.1f} us {r['nccl_bus_gbps']:7.1f} GB/s"
                     if "nccl_ms" in r else "")
                  + ("" if r.get("correct", True) else "   MISMATCH"))
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            with open(args.out, "w") as f:
                json.dump(payload, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
