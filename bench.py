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
JSON line.  Besides the headline it carries, measured in the same process:

  "shapes"    per-shape latency and fraction of the roofline
              max(FLOPs / measured cuBLAS peak, NVLink bytes per rank / 900 GB/s),
              plus the same fraction against the 770 GB/s copy-engine figure
  "verified"  every problem checked once against an fp32 torch product
              (operands gathered over NCCL); a mismatch exits non-zero
  "s0"        torch.matmul + NCCL all_gather_into_tensor / reduce_scatter_tensor
              on the same shapes, timed the same way
  "e2e"       the same metric through the public API with the host -> device copy
              of A and a device -> host read inside the timed region, next to
              the time of the copies alone ("h2d_floor_ms")
  "tp_mlp"    the bf16 tensor-parallel MLP block (8192 tokens, 4096, 14336)
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
    ap.add_argument("--no-align", action="store_true",
                    help="do not align the ranks on the device before each timed problem")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the S0 (cuBLAS + NCCL) and TP-MLP sections")
    ap.add_argument("--reference-mode", default="auto", choices=["auto", "single-process"],
                    help="reference arm: 'single-process' drives every rank from rank 0 through "
                         "tileccl.init_local (what 'auto' does for more than two ranks)")
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


NVLINK_NOMINAL_GBS = 900.0     # per direction per GPU: the roofline's link term
NVLINK_COPY_GBS = 770.0        # measured peer copy (copy engine) on this pool
NVLINK_SM_STORE_GBS = 690.0    # measured ceiling of SM-issued stores / bulk stores to a peer


def roofline_ms(kind, shape, world, peaks, link_gbs=NVLINK_NOMINAL_GBS):
    M, N, K = shape
    flops = 2.0 * M * N * K / world
    gemm_ms = flops / (peaks["bf16_tflops"] * 1e12) * 1e3
    nv_bytes = (world - 1) / world * M * N * 2
    comm_ms = nv_bytes / (link_gbs * 1e9) * 1e3
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


class RankAligner:
    """Brings the ranks' streams to the same point before a timed problem: a tiny NCCL
    all-reduce on the launching stream, after the L2 flush and before the start event.  The
    256 MiB flush does not take the same time on every GPU; without this its jitter (the
    maximum over N ranks) is billed to the operator, because every fused call ends only when
    the slowest peer's data has arrived.  It is the barrier-before-timing of the usual
    collective benchmarks, used for every arm alike, outside the timed events; the host never
    blocks on it."""

    def __init__(self, torch, world, device, enabled=True):
        self.world, self.enabled = world, enabled and world > 1
        self.token = torch.zeros(1, device=device) if self.enabled else None

    def __call__(self):
        if self.enabled:
            import torch.distributed as dist

            dist.all_reduce(self.token)


def verify_problems(torch, probs, world, rank, device):
    """fp32 torch product of every problem (operands gathered over NCCL) against the fused
    result of the last call.  Returns the largest max-abs error relative to max |reference|."""
    if world > 1:
        import torch.distributed as dist

    def gather(t):
        if world == 1:
            return [t]
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        return parts

    worst = 0.0
    for kind, (M, N, K), a, b, c in probs:
        As, Bs = gather(a), gather(b)
        if kind == "ag":
            ref = torch.cat([As[r].float() @ Bs[r].float() for r in range(world)], 0)
        else:
            rows = M // world
            ref = sum(As[r][rank * rows:(rank + 1) * rows].float() @ Bs[r].float()
                      for r in range(world))
        err = (c.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-9)
        worst = max(worst, err)
        del ref, As, Bs
    return max_over_ranks([worst], world, device)[0]


def run_s0(torch, probs, world, device, flush, steps, warmup, align=lambda: None):
    """S0 of the reference's README: library GEMM, then the bulk library collective
    (torch.matmul + NCCL), on the same operands and with the same timing as the fused arm."""
    if world > 1:
        import torch.distributed as dist
    items = []
    for kind, (M, N, K), a, b, _ in probs:
        if kind == "ag":
            tmp = torch.empty(M // world, N, device=device, dtype=a.dtype)
            out = torch.empty(M, N, device=device, dtype=a.dtype)
        else:
            tmp = torch.empty(M, N, device=device, dtype=a.dtype)
            out = torch.empty(M // world, N, device=device, dtype=a.dtype)
        items.append((kind, a, b, tmp, out))

    def run(it):
        kind, a, b, tmp, out = it
        torch.matmul(a, b, out=tmp)
        if world == 1:
            out.copy_(tmp)
        elif kind == "ag":
            dist.all_gather_into_tensor(out, tmp)
        else:
            dist.reduce_scatter_tensor(out, tmp)

    for _ in range(max(warmup, 3)):
        for it in items:
            flush.zero_()
            align()
            run(it)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    events = []
    for _ in range(steps):
        row = []
        for it in items:
            flush.zero_()
            align()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            run(it)
            e.record()
            row.append((s, e))
        events.append(row)
    torch.cuda.synchronize()
    per = [sum(row[i][0].elapsed_time(row[i][1]) for row in events) / steps
           for i in range(len(items))]
    per = max_over_ranks(per, world, device)
    return {"what": "torch.matmul (cuBLAS) + NCCL all_gather_into_tensor / reduce_scatter_tensor, "
                    "same shapes, CUDA events per problem, max over ranks",
            "value": round(sum(per) / len(per), 5), "unit": "ms",
            "shapes_ms": {f"{p[0]}_{p[1][0]}x{p[1][1]}x{p[1][2]}": round(ms, 5)
                          for p, ms in zip(probs, per)}}


def run_tp_mlp(torch, ctx, world, rank, device, flush, steps, warmup, align=lambda: None):
    """Tensor-parallel SwiGLU MLP block, bf16, 8192 tokens, hidden 4096, FFN 14336 sharded:
    all-gather -> gate/up GEMM + SiLU-gate -> down GEMM -> reduce-scatter (two fused launches)."""
    from tileccl_b200.models.tp_mlp import TPMLP
    from tileccl_b200.ops import check_status

    T, H, F = 8192, 4096, 14336
    mlp = TPMLP(ctx, tokens=T, hidden=H, ffn=F, dtype=torch.bfloat16, seed=1)
    gen = torch.Generator(device=device)
    gen.manual_seed(99 + rank)
    mlp.x_local.copy_(torch.randn(T // world, H, device=device, generator=gen).bfloat16())
    ctx.barrier()
    for _ in range(max(warmup, 3)):
        flush.zero_()
        align()
        mlp.forward()
    check_status(ctx)
    ctx.barrier()
    evs = []
    for _ in range(steps):
        flush.zero_()
        align()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        mlp.forward()
        e.record()
        evs.append((s, e))
    torch.cuda.synchronize()
    check_status(ctx)
    ms = max_over_ranks([sum(s.elapsed_time(e) for s, e in evs) / steps], world, device)[0]
    flops = 2.0 * T * H * (F // world) * 3
    roof_ms = max(flops / (load_peaks()["bf16_tflops"] * 1e12) * 1e3,
                  (world - 1) / world * T * H * 2 / (NVLINK_NOMINAL_GBS * 1e9) * 1e3)
    return {"what": "TP-MLP forward bf16, tokens 8192, hidden 4096, ffn 14336 / N, weights N(0,0.02)",
            "ms": round(ms, 5), "tflops_per_gpu": round(flops / ms / 1e9, 1),
            "roofline_ms": round(roof_ms, 5), "frac_of_roofline": round(roof_ms / ms, 4)}


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

    ctx = tccl.init(heap_size=4 << 30)
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

    align = RankAligner(torch, world, device, not args.no_align)
    for _ in range(max(args.warmup, 3)):
        for p in probs:
            flush.zero_()
            align()
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
            align()
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

    # ---- outside the timed region: every problem's result against an fp32 torch product
    verify_err = verify_problems(torch, probs, world, rank, device)
    verified = verify_err < 1e-2

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

        # The copies alone (same pinned buffers, same destination, no kernel): the floor
        # that PCIe sets for any implementation of this step.
        def floor_step():
            for pin, p in zip(pinned, probs):
                p[2].copy_(pin, non_blocking=True)
                out_host.copy_(p[4].view(-1)[:4096], non_blocking=True)
            torch.cuda.synchronize()

        floor_step()
        sync_all()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            floor_step()
        sync_all()
        floor_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps / len(probs)
        floor_ms = max_over_ranks([floor_ms], world, device)[0]
        e2e = {"value": round(e2e_ms, 5), "unit": "ms", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": e2e_steps,
               "h2d_floor_ms": round(floor_ms, 5),
               "over_floor": round(e2e_ms / floor_ms, 4),
               "what": "per problem: pinned-host A -> device (streamed by the op, a_host=), "
                       "fused op, 8 KiB of C -> host; h2d_floor_ms = the same copies with no kernel"}

    extras = {}
    if not args.no_extras:
        extras["s0"] = run_s0(torch, probs, world, device, flush, args.steps, args.warmup, align)
        extras["tp_mlp"] = run_tp_mlp(torch, ctx, world, rank, device, flush, args.steps,
                                      args.warmup, align)

    peaks = load_peaks()
    shapes = {}
    for p, ms in zip(probs, per_prob):
        kind, shape, *_ = p
        roof = roofline_ms(kind, shape, world, peaks)
        shapes[f"{kind}_{shape[0]}x{shape[1]}x{shape[2]}"] = {
            "ms": round(ms, 5), "roofline_ms": round(roof, 5),
            "frac_of_roofline": round(roof / ms, 4),
            "frac_of_roofline_770": round(
                roofline_ms(kind, shape, world, peaks, NVLINK_COPY_GBS) / ms, 4),
            "frac_of_sm_store_ceiling_690": round(
                roofline_ms(kind, shape, world, peaks, NVLINK_SM_STORE_GBS) / ms, 4)}
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
                       "rank_alignment": ("none" if args.no_align or world == 1 else
                                          "tiny NCCL all-reduce on the stream after the flush, "
                                          "before the start event (every arm)"),
                       "push_mode": os.environ.get("TILECCL_PUSH_MODE", "tma"),
                       "nvls_bound": bool(ctx.heap.has_multicast),
                       "roofline_peaks": peaks,
                       "roofline": "max(FLOPs / measured cuBLAS bf16 burst, NVLink bytes per rank / "
                                   "900 GB/s per direction); frac_of_roofline_770 uses the measured "
                                   "peer-copy rate, frac_of_sm_store_ceiling_690 the measured "
                                   "ceiling of SM-issued stores to a peer"},
            "shapes": shapes, "clocks": clocks, "gpu_launches": launches,
            "verified": verified, "verify_max_rel_err": round(verify_err, 6),
            "host_us_per_op": round(host_s / (args.steps * len(probs)) * 1e6, 1),
            "wall_ms_per_step_incl_flush": round(t_wall * 1e3 / args.steps, 4),
            "baseline_published": {"what": "reference S2, 2x H100 NVLink", "ms": PUBLISHED_S2_MS},
        }
        if e2e is not None:
            out["e2e"] = e2e
        out.update(extras)
        if "s0" in extras:
            out["speedup_vs_s0"] = round(extras["s0"]["value"] / value, 4)
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        ctx.heap.cleanup()
        dist.destroy_process_group()
    if not verified:
        if rank == 0:
            print(f"bench: result check failed, max relative error {verify_err:.3e}",
                  file=sys.stderr, flush=True)
        sys.exit(4)


# ------------------------------------------------------------ reference arm
def run_reference(args):
    """The unmodified reference (baseline/_ref) through its own public API.

    The reference has no row-sharded GEMM+collective operator: its
    ``ops.gemm_allgather(A, B_shard, C)`` and ``ops.gemm_reducescatter(A, B, C)``
    shard along N.  The same global problem sizes are run through that
    contract (equal FLOPs per rank and equal bytes on the wire).  Its validated
    multi-process surface is world_size 2; larger N runs in its single-process
    mode (see ``run_reference_single_process``).
    """
    rank, world, local = dist_env()

    def unavailable(why):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0

    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "tileccl")):
        return unavailable("baseline/_ref is not installed")
    if world > 2 or (world > 1 and args.reference_mode == "single-process"):
        # The reference's multi-process device collectives are gated to two ranks
        # (tileccl/utils/feature_gates.py:17-24); more ranks run in its single-process
        # mode, one Python process driving every GPU (tileccl/__init__.py:321-356).
        return run_reference_single_process(args, rank, world, local, ref_dir, unavailable)
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

        align = RankAligner(torch, world, device, not args.no_align)
        for _ in range(max(args.warmup, 3)):
            for p in probs:
                flush.zero_()
                align()
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
                align()
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



def run_reference_single_process(args, rank, world, local, ref_dir, unavailable):
    """Reference arm for more than two ranks: launcher rank 0 alone drives all `world` GPUs
    through the reference's single-process mode (``tileccl.init_local``), calling its
    ``ops.gemm_allgather`` / ``ops.gemm_reducescatter`` once per rank context as its own
    example does; the other launcher ranks wait at a host-side (gloo) barrier and touch no GPU.
    Device time = CUDA events on every GPU around one problem, max over GPUs."""
    import datetime

    import torch
    import torch.distributed as dist

    dist.init_process_group("gloo", timeout=datetime.timedelta(minutes=30))
    line = None
    if rank == 0:
        try:
            sys.path.insert(0, ref_dir)
            import tileccl  # the reference package from baseline/_ref

            if os.path.realpath(os.path.dirname(tileccl.__file__)).startswith(
                    os.path.realpath(os.path.join(ROOT, "tileccl"))):
                raise RuntimeError("import resolved to this repository's package, not the reference")
            if torch.cuda.device_count() < world:
                raise RuntimeError(f"launcher rank 0 sees {torch.cuda.device_count()} GPUs, "
                                   f"needs {world}")
            ctxs = tileccl.init_local(world, 3 << 30)
            devs = [torch.device("cuda", r) for r in range(world)]

            def rnd(gen, dev, rows, cols, scale):
                return (torch.randn(rows, cols, device=dev, generator=gen) * scale).to(torch.float16)

            probs = []          # (kind, shape, [a_r], [b_r], [c_r])
            gens = []
            for r in range(world):
                g = torch.Generator(device=devs[r])
                g.manual_seed(1234 + r)
                gens.append(g)
            for kind, shapes in (("ag", AG_SHAPES), ("rs", RS_SHAPES)):
                for (M, N, K) in shapes:
                    a_l, b_l, c_l = [], [], []
                    for r in range(world):
                        with torch.cuda.device(r):
                            if kind == "ag":
                                a = ctxs[r].zeros(M, K, dtype=torch.float16)
                                a.copy_(rnd(gens[r], devs[r], M, K, K ** -0.5))
                                b = ctxs[r].zeros(K, N // world, dtype=torch.float16)
                                b.copy_(rnd(gens[r], devs[r], K, N // world, 1.0))
                                c = ctxs[r].zeros(M, N, dtype=torch.float16)
                            else:
                                a = ctxs[r].zeros(M, K // world, dtype=torch.float16)
                                a.copy_(rnd(gens[r], devs[r], M, K // world, K ** -0.5))
                                b = ctxs[r].zeros(K // world, N, dtype=torch.float16)
                                b.copy_(rnd(gens[r], devs[r], K // world, N, 1.0))
                                c = ctxs[r].zeros(M, N // world, dtype=torch.float16)
                        a_l.append(a), b_l.append(b), c_l.append(c)
                    probs.append((kind, (M, N, K), a_l, b_l, c_l))
            flush = [torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=d) for d in devs]

            def run_one(p):
                kind, _, a_l, b_l, c_l = p
                for r in range(world):
                    with torch.cuda.device(r):
                        if kind == "ag":
                            tileccl.ops.gemm_allgather(a_l[r], b_l[r], c_l[r], ctx=ctxs[r])
                        else:
                            tileccl.ops.gemm_reducescatter(a_l[r], b_l[r], c_l[r], ctx=ctxs[r])

            def sync_all():
                for r in range(world):
                    torch.cuda.synchronize(r)

            def flush_all():
                for r in range(world):
                    with torch.cuda.device(r):
                        flush[r].zero_()

            def record_all():
                evs = []
                for r in range(world):
                    with torch.cuda.device(r):
                        e = torch.cuda.Event(enable_timing=True)
                        e.record()
                        evs.append(e)
                return evs

            t_first = time.perf_counter()
            for p in probs:
                flush_all()
                run_one(p)
            sync_all()
            first_s = time.perf_counter() - t_first
            budget_s = 600.0
            total_iters = max(args.warmup, 3) + args.steps + 12
            if first_s * total_iters > budget_s:
                raise RuntimeError(f"one step of the reference takes {first_s:.1f} s in its "
                                   f"single-process mode; {total_iters} steps do not fit in "
                                   f"{budget_s:.0f} s")
            for _ in range(max(args.warmup, 3) - 1):
                for p in probs:
                    flush_all()
                    run_one(p)
            sync_all()
            sampler = ClockSampler(0)
            sampler.start()
            per_prob = [0.0] * len(probs)
            for _ in range(args.steps):
                for i, p in enumerate(probs):
                    flush_all()
                    sync_all()
                    s_ev = record_all()
                    run_one(p)
                    e_ev = record_all()
                    sync_all()
                    per_prob[i] += max(s.elapsed_time(e) for s, e in zip(s_ev, e_ev))
            clocks = sampler.stop()
            per_prob = [x / args.steps for x in per_prob]

            e2e = None
            if not args.no_e2e:
                pinned = [[torch.empty_like(a, device="cpu").pin_memory() for a in p[2]]
                          for p in probs]
                for pins, p in zip(pinned, probs):
                    for pin, a in zip(pins, p[2]):
                        pin.copy_(a)
                out_host = [torch.empty(4096, dtype=torch.float16).pin_memory()
                            for _ in range(world)]
                e2e_steps = max(3, min(args.steps, 10))

                def e2e_step():
                    for pins, p in zip(pinned, probs):
                        for r in range(world):
                            with torch.cuda.device(r):
                                p[2][r].copy_(pins[r], non_blocking=True)
                        run_one(p)
                        for r in range(world):
                            with torch.cuda.device(r):
                                out_host[r].copy_(p[4][r].view(-1)[:4096], non_blocking=True)
                    sync_all()

                for _ in range(2):
                    e2e_step()
                t0 = time.perf_counter()
                for _ in range(e2e_steps):
                    e2e_step()
                e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps / len(probs)
                e2e = {"value": round(e2e_ms, 5), "unit": "ms",
                       "h2d_bytes_per_step": sum(pins[0].numel() * 2 for pins in pinned),
                       "d2h_bytes_per_step": 4096 * 2 * len(probs), "steps": e2e_steps,
                       "note": "bytes per rank; every rank's copies are inside the timed region"}
            ms_per_step = sum(per_prob)
            value = ms_per_step / len(probs)
            line = {
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
                           "api": "tileccl.init_local + tileccl.ops.gemm_allgather / "
                                  "gemm_reducescatter, one call per rank context",
                           "process_model": "single process: launcher rank 0 drives all GPUs (the "
                                            "reference gates its multi-process device collectives to "
                                            "two ranks); the other launcher ranks wait at a host barrier",
                           "timing": "CUDA events on every GPU around one problem, max over GPUs",
                           "l2": "256 MiB flush write on every GPU before every problem, outside "
                                 "the timed events"},
                "shapes": {f"{p[0]}_{p[1][0]}x{p[1][1]}x{p[1][2]}": {"ms": round(ms, 5)}
                           for p, ms in zip(probs, per_prob)},
                "clocks": clocks,
            }
            if e2e is not None:
                line["e2e"] = e2e
        except BaseException as exc:  # the reference arm must never take the bench down
            msg = f"{type(exc).__name__}: {exc}".replace("\n", " ")[:300]
            line = {"impl": "reference",
                    "unavailable": f"reference failed in its single-process mode: {msg}"}
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


def main():
    args = parse_args()
    if args.impl == "reference":
        sys.exit(run_reference(args))
    run_ours(args)


if __name__ == "__main__":
    main()
