#!/usr/bin/env python
"""TP-MLP block forward: 8192 tokens, hidden 4096, FFN 14336, bf16, sharded over N ranks.

Ours: ``tileccl_b200.models.TPMLP`` (two fused launches: all-gather + gate/up GEMM with
SiLU-gate epilogue, then down GEMM with reduce-scatter epilogue).
S0:   NCCL ``all_gather_into_tensor`` -> ``torch.matmul`` (gate|up) -> SiLU * up
      (torch elementwise) -> ``torch.matmul`` (down) -> NCCL ``reduce_scatter_tensor``.

Timing: CUDA events around one forward, 256 MiB L2 flush before each, max over ranks,
mean over steps.  One JSON line on rank 0.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/tp_mlp.py --steps 20 --warmup 5
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    rank, ws = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if ws > 1:
        dist.init_process_group("nccl", device_id=dev)
    import tileccl_b200 as tccl
    from tileccl_b200.models.tp_mlp import TPMLP
    from tileccl_b200.ops import check_status

    ctx = tccl.init(heap_size=2 << 30)
    T, H, F = args.tokens, args.hidden, args.ffn
    mlp = TPMLP(ctx, tokens=T, hidden=H, ffn=F, dtype=torch.bfloat16, seed=1)
    mlp.x_local.copy_(torch.randn(T // ws, H, device=dev).bfloat16())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    # S0 operands of the same shard shapes
    fl = F // ws
    w_gu = (torch.randn(H, 2 * fl, device=dev) * 0.02).bfloat16()
    w_dn = (torch.randn(fl, H, device=dev) * 0.02).bfloat16()
    x_shard = mlp.x_local.clone()
    x_full = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    h_gu = torch.empty(T, 2 * fl, device=dev, dtype=torch.bfloat16)
    part = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    y = torch.empty(T // ws, H, device=dev, dtype=torch.bfloat16)

    def s0():
        if ws > 1:
            dist.all_gather_into_tensor(x_full, x_shard)
        else:
            x_full.copy_(x_shard)
        torch.matmul(x_full, w_gu, out=h_gu)
        h1 = torch.nn.functional.silu(h_gu[:, :fl]) * h_gu[:, fl:]
        torch.matmul(h1, w_dn, out=part)
        if ws > 1:
            dist.reduce_scatter_tensor(y, part)
        else:
            y.copy_(part)

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            flush.zero_()
            fn()
        torch.cuda.synchronize()
        if ws > 1:
            dist.barrier()
        evs = []
        for _ in range(args.steps):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            evs.append((s, e))
        torch.cuda.synchronize()
        t = torch.tensor([sum(s.elapsed_time(e) for s, e in evs) / args.steps],
                         dtype=torch.float64, device=dev)
        if ws > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ours = timed(lambda: mlp.forward())
    check_status(ctx)
    lib = timed(s0)
    if rank == 0:
        flops = 2.0 * T * H * (2 * F) / ws + 2.0 * T * F * H / ws
        print(json.dumps({"bench": "tp_mlp_forward", "n_gpus": ws, "dtype": "bf16",
                          "tokens": T, "hidden": H, "ffn": F, "ours_ms": round(ours, 5),
                          "s0_cublas_nccl_ms": round(lib, 5),
                          "ours_tflops_per_gpu": round(flops / ours / 1e9, 1),
                          "speedup_vs_s0": round(lib / ours, 3), "steps": args.steps}), flush=True)
    if ws > 1:
        dist.barrier()
    ctx.heap.cleanup()
    if ws > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
