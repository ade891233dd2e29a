#!/usr/bin/env python
"""Tile-collective sweep: allreduce(sum), allgather, reduce_scatter, broadcast(root 0),
scatter on symmetric-heap buffers, 4 KiB .. 1 GiB, fp16 and fp32, values U(-1, 1) seeded per
rank, against NCCL on the same buffers.  One process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/collectives_sweep.py [--max-bytes 1073741824] [--out sweep.json]

Device time (CUDA events), max over ranks; bus GB/s uses the usual factors
(allreduce 2(n-1)/n, allgather / reduce_scatter / scatter (n-1)/n, broadcast 1).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn, iters, dev):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s = torch.cuda.Event(enable_timing=True)
    e = torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=4096)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import tileccl_b200 as tccl
    from tileccl_b200 import ops
    from tileccl_b200.primitives import collectives as coll

    ctx = tccl.init(heap_size=int(2.5 * args.max_bytes) + (64 << 20))
    rows = []
    nbytes = args.min_bytes
    while nbytes <= args.max_bytes:
        for dtype in (torch.float16, torch.float32):
            es = torch.empty((), dtype=dtype).element_size()
            n = max(ws, nbytes // es // ws * ws)
            ctx.barrier()
            ctx.heap.reset_allocator()
            ctx._workspace_cache.clear()
            ctx._state.clear()
            ctx.heap._state.clear()
            gen = torch.Generator(device=dev).manual_seed(7 + rank)
            full = ctx.empty(n, dtype=dtype)
            full.copy_(torch.rand(n, device=dev, generator=gen) * 2 - 1)
            part = ctx.zeros(n // ws, dtype=dtype)
            ctx.barrier()
            iters = 20 if nbytes <= (16 << 20) else 5
            cases = {
                "allreduce": (lambda: ops.allreduce(full, ctx=ctx), lambda: dist.all_reduce(full),
                              2 * (ws - 1) / ws),
                "allgather": (lambda: ops.allgather(part, full, ctx=ctx),
                              lambda: dist.all_gather_into_tensor(full, part), (ws - 1) / ws),
                "reduce_scatter": (lambda: ops.reduce_scatter(full, part, ctx=ctx),
                                   lambda: dist.reduce_scatter_tensor(part, full), (ws - 1) / ws),
                "broadcast": (lambda: ops.broadcast(full, ctx=ctx, root=0),
                              lambda: dist.broadcast(full, src=0), 1.0),
                "scatter": (lambda: ops.scatter(full, part, ctx=ctx, root=0), None, (ws - 1) / ws),
            }
            for name, (ours, nccl, factor) in cases.items():
                ms = timed(ours, iters, dev)
                row = {"collective": name, "bytes": n * es, "dtype": str(dtype).split(".")[-1],
                       "world_size": ws, "ms": ms, "bus_gbps": n * es * factor / ms / 1e6}
                if nccl is not None:
                    ms_n = timed(nccl, iters, dev)
                    row.update(nccl_ms=ms_n, nccl_bus_gbps=n * es * factor / ms_n / 1e6)
                rows.append(row)
            coll.check_status(ctx.heap)
        nbytes *= 4
    if rank == 0:
        payload = {"suite": "collectives_sweep", "world_size": ws, "nvls": ctx.heap.has_multicast,
                   "rows": rows}
        for r in rows:
            print(f"{r['collective']:<15s} {r['dtype']:<8s} {r['bytes']:>11d} B  ours {r['ms'] * 1e3:9.1f} us "
                  f"{r['bus_gbps']:7.1f} GB/s" + (f"   nccl {r['nccl_ms'] * 1e3:9.1f} us {r['nccl_bus_gbps']:7.1f} GB/s"
                                                    if "nccl_ms" in r else ""))
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            with open(args.out, "w") as f:
                json.dump(payload, f, indent=1)
    ctx.barrier()
    ctx.heap.cleanup()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
