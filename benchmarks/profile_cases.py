#!/usr/bin/env python
"""Small, self-terminating cases for kernel profiling on ONE GPU.

    python benchmarks/profile_cases.py gemm [--m 16384 --n 4096 --k 1024] [--launches 3]
    python benchmarks/profile_cases.py collective [--op allreduce --bytes 16777216 --ranks 4]
    python benchmarks/profile_cases.py fused [--mode ag|rs --ranks 2]

``gemm``: the CTA-pair tcgen05 GEMM kernel on one problem (operands + output well above the
L2 size together with the flush buffer, a few hundred MB on the device).
``collective``: the collective kernel with `ranks` ranks emulated on this GPU; the phases of a
call are separate launches there, so no launch waits for another.
``fused``: the fused GEMM + all-gather / reduce-scatter operator with emulated ranks (tile-range
launches of the one-CTA form).

Meant to be run plainly first and then under
``ncu --set full --clock-control none -k regex:<kernel> -c <n>``; each case launches only a
handful of kernels.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def case_gemm(args) -> None:
    from tileccl_b200.kernels.fused_gemm import gemm

    a = (torch.randn(args.m, args.k, device="cuda") / args.k ** 0.5).half()
    b = torch.randn(args.k, args.n, device="cuda").half()
    c = torch.empty(args.m, args.n, device="cuda", dtype=torch.float16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    times = []
    for _ in range(args.launches):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        gemm(a, b, c)
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    ref = a[:256].float() @ b.float()
    err = (c[:256].float() - ref).abs().max().item() / ref.abs().max().item()
    flops = 2.0 * args.m * args.n * args.k
    print(f"gemm {args.m}x{args.n}x{args.k} fp16: best {min(times) * 1e3:.1f} us "
          f"({flops / min(times) / 1e9:.0f} TFLOP/s), rel err {err:.2e}")
    assert err < 5e-3


def case_collective(args) -> None:
    import tileccl_b200 as tccl
    from tileccl_b200 import ops

    ws = args.ranks
    ctxs = tccl.init_local(ws, 4 * args.bytes + (64 << 20), devices=[0] * ws)
    n = args.bytes // 2 // ws * ws
    full = [c.randn(n, dtype=torch.float16) for c in ctxs]
    part = [c.zeros(n // ws, dtype=torch.float16) for c in ctxs]
    want = sum(f.float() for f in full)
    for _ in range(args.launches):
        for r, c in enumerate(ctxs):
            if args.op == "allreduce":
                ops.allreduce(full[r], ctx=c)
            elif args.op == "allgather":
                ops.allgather(part[r], full[r], ctx=c)
            elif args.op == "reduce_scatter":
                ops.reduce_scatter(full[r], part[r], ctx=c)
            else:
                ops.broadcast(full[r], ctx=c, root=0)
        torch.cuda.synchronize()
        if args.op == "allreduce":
            err = (full[0].float() - want).abs().max().item() / want.abs().max().item()
            assert err < 2e-2, err
            want = want * ws
    print(f"{args.op} {n * 2} bytes, {ws} emulated ranks: ok")
    for c in ctxs:
        c.heap.cleanup()


def case_fused(args) -> None:
    import tileccl_b200 as tccl
    from tileccl_b200 import ops

    ws = args.ranks
    ctxs = tccl.init_local(ws, 1 << 30, devices=[0] * ws)
    M, N, K = args.m, args.n, args.k
    if args.mode == "ag":
        A = [(torch.randn(M // ws, K, device="cuda") / K ** 0.5).half() for _ in ctxs]
        B = [torch.randn(K, N, device="cuda").half() for _ in ctxs]
        C = [c.zeros(M, N, dtype=torch.float16) for c in ctxs]
        for _ in range(args.launches):
            for r, c in enumerate(ctxs):
                ops.gemm_allgather_rows(A[r], B[r], C[r], ctx=c)
        torch.cuda.synchronize()
        ref = torch.cat([A[r][:128].float() @ B[r].float() for r in range(ws)])
        got = torch.cat([C[0][r * (M // ws):r * (M // ws) + 128] for r in range(ws)])
    else:
        A = [(torch.randn(M, K // ws, device="cuda") / K ** 0.5).half() for _ in ctxs]
        B = [torch.randn(K // ws, N, device="cuda").half() for _ in ctxs]
        C = [torch.zeros(M // ws, N, device="cuda", dtype=torch.float16) for _ in ctxs]
        for _ in range(args.launches):
            for r, c in enumerate(ctxs):
                ops.gemm_reducescatter_rows(A[r], B[r], C[r], ctx=c)
        torch.cuda.synchronize()
        ref = sum(A[r][:128].float() @ B[r].float() for r in range(ws))
        got = C[0][:128]
    for c in ctxs:
        ops.check_status(c)
    err = (got.float() - ref).abs().max().item() / ref.abs().max().item()
    print(f"fused {args.mode} {M}x{N}x{K}, {ws} emulated ranks: rel err {err:.2e}")
    assert err < 1e-2
    for c in ctxs:
        c.heap.cleanup()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "collective", "fused"])
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--op", default="allreduce",
                    choices=["allreduce", "allgather", "reduce_scatter", "broadcast"])
    ap.add_argument("--bytes", type=int, default=16 << 20)
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--mode", default="ag", choices=["ag", "rs"])
    args = ap.parse_args()
    torch.cuda.set_device(0)
    {"gemm": case_gemm, "collective": case_collective, "fused": case_fused}[args.case](args)


if __name__ == "__main__":
    main()
