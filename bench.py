#!/usr/bin/env python
"""Headline benchmark: fused GEMM + all-gather and GEMM -> reduce-scatter latency.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...            # the unmodified reference

For N > 1 launch with ``python -m torch.distributed.run --nnodes=1
--nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...``
(one rank per GPU, NCCL only for the rendezvous).

One *step* runs the six gate problems once (fp16, synthetic seeded inputs):

  all-gather of the GEMM output   A[M/ws, K] @ B[K, N] -> C[M, N] on every rank
      16384x4096x1024, 8192x4096x2048, 8192x4096x1024
  GEMM -> reduce-scatter          A[M, K/ws] @ B[K/ws, N] partials -> C[M/ws, N]
      16384x4096x2048, 8192x4096x4096, 8192x4096x2048   (K is the total K)

Every problem is timed on the device with CUDA events around its own launch;
L2 is flushed (a 256 MiB write) before each problem, outside the timed events.
The reported value is the mean latency per problem in milliseconds (max over
ranks), total work is fixed as N grows (strong scaling).  Rank 0 prints ONE
JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

AG_SHAPES = [(16384, 4096, 1024), (8192, 4096, 2048), (8192, 4096, 1024)]
RS_SHAPES = [(16384, 4096, 2048), (8192, 4096, 4096), (8192, 4096, 2048)]
# Published S2 latencies of the reference (2 x H100 NVLink, its README), same order.
PUBLISHED_S2_MS = [0.801, 0.639, 0.482, 0.965, 0.769, 0.609]
METRIC = "fused GEMM+AG / GEMM->RS latency (mean over the 3+3 gate shapes)"
FLUSH_BYTES = 256 << 20


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--push-mode", default=None, choices=[None, "stores", "tma", "multimem"])
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


# ------------------------------------------------------------------ clocks
def ClockSampler(gpu_index: int):
    """NVML sampler thread (SM clock, power, throttle reasons) for the timed region."""
    sys.path.insert(0, ROOT) if ROOT not in sys.path else None
    import importlib.util

    spec = importlib.util.spec_from_file_location(
        "_tccl_clocks", os.path.join(ROOT, "tileccl_b200", "utils", "clocks.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.ClockSampler(gpu_index)


# ------------------------------------------------------------------ helpers
def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def max_over_ranks(values, world, device):
    import torch

    if world == 1:
        return list(values)
    import torch.distributed as dist

    t = torch.tensor(values, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def make_problems(torch, alloc_sym, device, rank, world):
    """Seeded synthetic operands: A, B ~ N(0,1)/sqrt(K_total), per-rank seeds."""
    gen = torch.Generator(device=device)
    gen.manual_seed(1234 + rank)
    probs = []

    def rnd(rows, cols, scale):
        return (torch.randn(rows, cols, device=device, generator=gen) * scale).to(torch.float16)

    for (M, N, K) in AG_SHAPES:
        a = rnd(M // world, K, K ** -0.5)
        b = rnd(K, N, 1.0)
        c = alloc_sym(M, N)
        probs.append(("ag", (M, N, K), a, b, c))
    for (M, N, K) in RS_SHAPES:
        a = rnd(M, K // world, K ** -0.5)
        b = rnd(K // world, N, 1.0)
        c = torch.zeros(M // world, N, dtype=torch.float16, device=device)
        probs.append(("rs", (M, N, K), a, b, c))
    return probs


def roofline_ms(kind, shape, world, peaks):
    M, N, K = shape
    flops = 2.0 * M * N * K / world
    gemm_ms = flops / (peaks["bf16_tflops"] * 1e12) * 1e3
    nv_bytes = (world - 1) / world * M * N * 2
    comm_ms = nv_bytes / 770e9 * 1e3
    return max(gemm_ms, comm_ms)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"bf16_tflops": float(d["bf16_tflops"]), "hbm_gbs": float(d["hbm_gbs"]),
                "source": "measured"}
    except Exception:
        return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


# ------------------------------------------------------------------ our arm
def run_ours(args):
    import torch

    rank, world, local = dist_env()
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks "
                             f"(WORLD_SIZE is {world})")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    if args.push_mode:
        os.environ["TILECCL_PUSH_MODE"] = args.push_mode

    sys.path.insert(0, ROOT)
    import tileccl_b200 as tccl
    from tileccl_b200 import ops
    from tileccl_b200.kernels import fused_gemm

    ctx = tccl.init(heap_size=3 << 30)
    probs = make_problems(torch, lambda m, n: ctx.zeros(m, n, dtype=torch.float16), device, rank,
                          world)

    def run_one(p):
        kind, _, a, b, c = p
        if kind == "ag":
            ops.gemm_allgather_rows(a, b, c, ctx=ctx)
        else:
            ops.gemm_reducescatter_rows(a, b, c, ctx=ctx)

    flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=device)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        for p in probs:
            flush.zero_()
            run_one(p)
    sync_all()
    ops.check_status(ctx)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = fused_gemm.LAUNCH_COUNT
    events = []
    sync_all()
    t_wall0 = time.perf_counter()
    host_s = 0.0
    for _ in range(args.steps):
        row = []
        for p in probs:
            flush.zero_()
            s = torch.cuda.Event(enable_timing=True)
            e = torch.cuda.Event(enable_timing=True)
            s.record()
            h0 = time.perf_counter()
            run_one(p)
            host_s += time.perf_counter() - h0
            e.record()
            row.append((s, e))
        events.append(row)
    sync_all()
    t_wall = time.perf_counter() - t_wall0
    launches = fused_gemm.LAUNCH_COUNT - launches0
    clocks = sampler.stop() if rank == 0 else None
    ops.check_status(ctx)

    per_prob = [0.0] * len(probs)
    for row in events:
        for i, (s, e) in enumerate(row):
            per_prob[i] += s.elapsed_time(e)
    per_prob = [x / args.steps for x in per_prob]
    per_prob = max_over_ranks(per_prob, world, device)
    ms_per_step = sum(per_prob)
    value = ms_per_step / len(probs)

    # ---- end to end through the public API: H2D of A from pinned memory, op, D2H of a result slice
    e2e = None
    if not args.no_e2e:
        pinned = [torch.empty_like(p[2], device="cpu").pin_memory() for p in probs]
        for pin, p in zip(pinned, probs):
            pin.copy_(p[2])
        out_host = torch.empty(4096, dtype=torch.float16).pin_memory()
        h2d = sum(pin.numel() * 2 for pin in pinned)
        d2h = out_host.numel() * 2 * len(probs)
        e2e_steps = max(3, min(args.steps, 10))

        def e2e_step():
            for pin, p in zip(pinned, probs):
                kind, _, a, b, c = p
                # The op itself brings A over from the pinned host tensor (a_host=...).
                # (every problem has its own A buffer and nothing else touches it, so the
                # copy only has to follow the operator's previous call on that buffer)
                if kind == "ag":
                    ops.gemm_allgather_rows(a, b, c, ctx=ctx, a_host=pin, a_host_order="plan")
                else:
                    ops.gemm_reducescatter_rows(a, b, c, ctx=ctx, a_host=pin, a_host_order="plan")
                out_host.copy_(c.view(-1)[:4096], non_blocking=True)
            torch.cuda.synchronize()

        for _ in range(2):
            e2e_step()
        sync_all()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        sync_all()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps / len(probs)
        e2e_ms = max_over_ranks([e2e_ms], world, device)[0]
        e2e = {"value": round(e2e_ms, 5), "unit": "ms", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": e2e_steps,
               "what": "per problem: pinned-host A -> device (streamed by the op, a_host=), "
                       "fused op, 8 KiB of C -> host"}

    peaks = load_peaks()
    shapes = {}
    for p, ms in zip(probs, per_prob):
        kind, shape, *_ = p
        roof = roofline_ms(kind, shape, world, peaks)
        shapes[f"{kind}_{shape[0]}x{shape[1]}x{shape[2]}"] = {
            "ms": round(ms, 5), "roofline_ms": round(roof, 5),
            "frac_of_roofline": round(roof / ms, 4)}
    if rank == 0:
        out = {
            "metric": METRIC, "value": round(value, 5), "unit": "ms", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 5), "higher_is_better": False, "scaling": "strong",
            "vs_baseline": round(value / (sum(PUBLISHED_S2_MS) / len(PUBLISHED_S2_MS)), 4),
            "dtype": "fp16", "data": "synthetic (seeded N(0,1)/sqrt(K) operands, random-init)",
            "impl": "ours",
            "config": {"model": "gate shapes: AG 16384x4096x1024, 8192x4096x2048, 8192x4096x1024; "
                                "RS 16384x4096x2048, 8192x4096x4096, 8192x4096x2048",
                       "global_batch": None, "seq_len": None,
                       "parallelism": f"tp{world} row-sharded",
                       "l2": "256 MiB flush write before every problem, outside the timed events",
                       "timing": "CUDA events per problem, max over ranks, mean over steps",
                       "push_mode": os.environ.get("TILECCL_PUSH_MODE", "tma"),
                       "nvls_bound": bool(ctx.heap.has_multicast),
                       "roofline_peaks": peaks},
            "shapes": shapes, "clocks": clocks, "gpu_launches": launches,
            "host_us_per_op": round(host_s / (args.steps * len(probs)) * 1e6, 1),
            "wall_ms_per_step_incl_flush": round(t_wall * 1e3 / args.steps, 4),
            "baseline_published": {"what": "reference S2, 2x H100 NVLink", "ms": PUBLISHED_S2_MS},
        }
        if e2e is not None:
            out["e2e"] = e2e
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        ctx.heap.cleanup()
        dist.destroy_process_group()


# ------------------------------------------------------------ reference arm
def run_reference(args):
    """The unmodified reference (baseline/_ref) through its own public API.

    The reference has no row-sharded GEMM+collective operator: its
    ``ops.gemm_allgather(A, B_shard, C)`` and ``ops.gemm_reducescatter(A, B, C)``
    shard along N.  The same global problem sizes are run through that
    contract (equal FLOPs per rank and equal bytes on the wire).  Its validated
    multi-process surface is world_size 2; larger N reports `unavailable`.
    """
    rank, world, local = dist_env()

    def unavailable(why):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0

    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "tileccl")):
        return unavailable("baseline/_ref is not installed")
    if world > 2:
        return unavailable("reference multi-process device collectives are validated for "
                           "world_size 2 only (tileccl/utils/feature_gates.py:17-24)")
    sys.path.insert(0, ref_dir)
    try:
        import torch

        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        if world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=device)
        import tileccl  # the reference package from baseline/_ref

        if os.path.realpath(os.path.dirname(tileccl.__file__)).startswith(
                os.path.realpath(os.path.join(ROOT, "tileccl"))):
            return unavailable("import resolved to this repository's package, not the reference")
        ctx = tileccl.init(backend="cuda", heap_size=3 << 30)
        gen = torch.Generator(device=device)
        gen.manual_seed(1234 + rank)

        def rnd(rows, cols, scale):
            return (torch.randn(rows, cols, device=device, generator=gen) * scale).to(torch.float16)

        probs = []
        for (M, N, K) in AG_SHAPES:
            a = ctx.zeros(M, K, dtype=torch.float16)
            a.copy_(rnd(M, K, K ** -0.5))
            b = ctx.zeros(K, N // world, dtype=torch.float16)
            b.copy_(rnd(K, N // world, 1.0))
            c = ctx.zeros(M, N, dtype=torch.float16)
            probs.append(("ag", (M, N, K), a, b, c))
        for (M, N, K) in RS_SHAPES:
            a = ctx.zeros(M, K // world, dtype=torch.float16)
            a.copy_(rnd(M, K // world, K ** -0.5))
            b = ctx.zeros(K // world, N, dtype=torch.float16)
            b.copy_(rnd(K // world, N, 1.0))
            c = ctx.zeros(M, N // world, dtype=torch.float16)
            probs.append(("rs", (M, N, K), a, b, c))

        def run_one(p):
            kind, _, a, b, c = p
            if kind == "ag":
                tileccl.ops.gemm_allgather(a, b, c, ctx=ctx)
            else:
                tileccl.ops.gemm_reducescatter(a, b, c, ctx=ctx)

        flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=device)

        def sync_all():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
                torch.cuda.synchronize()

        for _ in range(max(args.warmup, 3)):
            for p in probs:
                flush.zero_()
                run_one(p)
        sync_all()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        events = []
        sync_all()
        for _ in range(args.steps):
            row = []
            for p in probs:
                flush.zero_()
                s = torch.cuda.Event(enable_timing=True)
                e = torch.cuda.Event(enable_timing=True)
                s.record()
                run_one(p)
                e.record()
                row.append((s, e))
            events.append(row)
        sync_all()
        clocks = sampler.stop() if rank == 0 else None
        per_prob = [0.0] * len(probs)
        for row in events:
            for i, (s, e) in enumerate(row):
                per_prob[i] += s.elapsed_time(e)
        per_prob = max_over_ranks([x / args.steps for x in per_prob], world, device)

        e2e = None
        if not args.no_e2e:
            pinned = [torch.empty_like(p[2], device="cpu").pin_memory() for p in probs]
            for pin, p in zip(pinned, probs):
                pin.copy_(p[2])
            out_host = torch.empty(4096, dtype=torch.float16).pin_memory()
            e2e_steps = max(3, min(args.steps, 10))

            def e2e_step():
                for pin, p in zip(pinned, probs):
                    p[2].copy_(pin, non_blocking=True)
                    run_one(p)
                    out_host.copy_(p[4].view(-1)[:4096], non_blocking=True)
                torch.cuda.synchronize()

            for _ in range(2):
                e2e_step()
            sync_all()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                e2e_step()
            sync_all()
            e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps / len(probs)
            e2e_ms = max_over_ranks([e2e_ms], world, device)[0]
            e2e = {"value": round(e2e_ms, 5), "unit": "ms",
                   "h2d_bytes_per_step": sum(pin.numel() * 2 for pin in pinned),
                   "d2h_bytes_per_step": out_host.numel() * 2 * len(probs), "steps": e2e_steps}
        ms_per_step = sum(per_prob)
        value = ms_per_step / len(probs)
        if rank == 0:
            out = {
                "metric": METRIC, "value": round(value, 5), "unit": "ms", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": round(ms_per_step, 5), "higher_is_better": False,
                "scaling": "strong",
                "vs_baseline": round(value / (sum(PUBLISHED_S2_MS) / len(PUBLISHED_S2_MS)), 4),
                "dtype": "fp16", "data": "synthetic (seeded N(0,1)/sqrt(K) operands, random-init)",
                "impl": "reference",
                "config": {"model": "gate shapes (same global sizes as the other arm)",
                           "parallelism": f"tp{world} column-sharded (the reference's only "
                                          "GEMM+collective contract)",
                           "api": "tileccl.ops.gemm_allgather / gemm_reducescatter",
                           "l2": "256 MiB flush write before every problem, outside the timed events"},
                "shapes": {f"{p[0]}_{p[1][0]}x{p[1][1]}x{p[1][2]}": {"ms": round(ms, 5)}
                           for p, ms in zip(probs, per_prob)},
                "clocks": clocks,
            }
            if e2e is not None:
                out["e2e"] = e2e
            print(json.dumps(out), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0
    except BaseException as exc:  # the reference arm must never take the bench down
        msg = f"{type(exc).__name__}: {exc}".replace("\n", " ")[:300]
        return unavailable(f"reference failed on this box: {msg}")


def main():
    args = parse_args()
    if args.impl == "reference":
        sys.exit(run_reference(args))
    run_ours(args)


if __name__ == "__main__":
    main()
