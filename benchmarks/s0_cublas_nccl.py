#!/usr/bin/env python
"""S0 baseline: library GEMM followed by a library collective (no fusion, no overlap).

For every gate shape, row-sharded like the fused operators:

* GEMM + all-gather:      ``C_local = A_local @ B`` (cuBLAS), then
  ``all_gather_into_tensor`` of the row blocks (NCCL);
* GEMM -> reduce-scatter: ``P = A @ B`` with the K-shard operands (cuBLAS), then
  ``reduce_scatter_tensor`` of the row blocks (NCCL).

Timed like ``bench.py``: CUDA events per problem, a 256 MiB write between
problems to flush L2, max over ranks, mean over steps.  Prints one JSON line.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/s0_cublas_nccl.py --steps 20 --warmup 5
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

AG_SHAPES = [(16384, 4096, 1024), (8192, 4096, 2048), (8192, 4096, 1024)]
RS_SHAPES = [(16384, 4096, 2048), (8192, 4096, 4096), (8192, 4096, 2048)]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    args = ap.parse_args()
    rank, ws = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if ws > 1:
        dist.init_process_group("nccl", device_id=dev)
    dt = torch.float16 if args.dtype == "fp16" else torch.bfloat16

    probs = []
    for (M, N, K) in AG_SHAPES:
        a = (torch.randn(M // ws, K, device=dev) / K ** 0.5).to(dt)
        b = torch.randn(K, N, device=dev).to(dt)
        c_loc = torch.empty(M // ws, N, device=dev, dtype=dt)
        c = torch.empty(M, N, device=dev, dtype=dt)
        probs.append(("ag", (M, N, K), a, b, c_loc, c))
    for (M, N, K) in RS_SHAPES:
        a = (torch.randn(M, K // ws, device=dev) / K ** 0.5).to(dt)
        b = torch.randn(K // ws, N, device=dev).to(dt)
        part = torch.empty(M, N, device=dev, dtype=dt)
        c = torch.empty(M // ws, N, device=dev, dtype=dt)
        probs.append(("rs", (M, N, K), a, b, part, c))

    def run(p):
        kind, _, a, b, tmp, out = p
        torch.matmul(a, b, out=tmp)
        if ws == 1:
            out.copy_(tmp)
        elif kind == "ag":
            dist.all_gather_into_tensor(out, tmp)
        else:
            dist.reduce_scatter_tensor(out, tmp)

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(max(args.warmup, 3)):
        for p in probs:
            flush.zero_()
            run(p)
    torch.cuda.synchronize()
    if ws > 1:
        dist.barrier()
    totals = [0.0] * len(probs)
    events = []
    for _ in range(args.steps):
        row = []
        for p in probs:
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            run(p)
            e.record()
            row.append((s, e))
        events.append(row)
    torch.cuda.synchronize()
    for row in events:
        for i, (s, e) in enumerate(row):
            totals[i] += s.elapsed_time(e)
    t = torch.tensor([x / args.steps for x in totals], dtype=torch.float64, device=dev)
    if ws > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    per = t.tolist()
    if rank == 0:
        shapes = {f"{p[0]}_{p[1][0]}x{p[1][1]}x{p[1][2]}": round(ms, 5) for p, ms in zip(probs, per)}
        print(json.dumps({"impl": "s0_cublas_nccl", "n_gpus": ws, "dtype": args.dtype,
                          "value": round(sum(per) / len(per), 5), "unit": "ms",
                          "steps": args.steps, "shapes_ms": shapes}), flush=True)
    if ws > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
