#!/usr/bin/env python
"""Phase-0 calibration of the alpha-beta link model on this machine.

Measures peer pushes (the broadcast collective from rank 0: one direct NVLink hop
per peer) over a range of sizes, fits ``time = alpha + beta * bytes`` (plus the
small-message floor) with ``CostModelCalibrator`` and writes the result, together
with the derived P2P saturation size tau_min, to a JSON file that
``HardwareProfile.b200_measured`` / ``TILECCL_CALIBRATION`` pick up.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/phase0_calibrate.py --out calibration/b200.json

The launch-level fit above includes kernel-launch latency and the collectives' three-phase
handshake, so it says little about a TileGroup inside the fused kernel.  The second mode
fits the push phase *inside* the kernel from its %globaltimer trace and needs no GPU:

    python benchmarks/phase0_calibrate.py --from-trace trace_n2.log \
        --out calibration/b200.json

reads the JSON lines that ``benchmarks/trace_fused_gemm.py`` prints, regresses "first
accumulator ready -> last bulk store issued" on the bytes each rank pushed (alpha = fixed
in-kernel overhead, 1 / beta = achieved link rate), derives tau_min = link rate x (signal
cost + visibility latency of a remote counter), and stores all of it under ``in_kernel`` in
the calibration file.  ``ops`` sizes TileGroups with that tau_min.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def fit_in_kernel(trace_files, visibility_us: float = 1.0) -> dict:
    """alpha / beta / tau_min of the in-kernel push phase from trace_fused_gemm.py output."""
    import re

    from tileccl_b200.planning import CalibrationPoint, CostModelCalibrator

    points, signals, rows = [], [], []
    for path in trace_files:
        with open(path) as f:
            for line in f:
                line = line.strip()
                if not line.startswith("{"):
                    continue
                d = json.loads(line)
                m = re.match(r"GEMM\+AG (\d+)x(\d+)x(\d+) ws=(\d+)", d.get("label", ""))
                if not m:                      # reduce-scatter rows also wait for peers: not a pure push
                    continue
                M, N, _, ws = (int(x) for x in m.groups())
                sent = (ws - 1) * (M // ws) * N * 2
                us = d["last_stores_issued_us"] - d["first_acc_ready_us"]
                points.append(CalibrationPoint(sent, 1, "int8", us))
                rows.append({"bytes": sent, "us": round(us, 2), "ws": ws})
                if d.get("median_signal_us") is not None:
                    signals.append(d["median_signal_us"])
    if len({p.tile_M for p in points}) < 2:
        raise SystemExit("need all-gather traces of at least two different sizes")
    alpha, beta = CostModelCalibrator.calibrate_comm(points)
    rate = 1.0 / beta                                     # bytes per microsecond
    signal_us = sorted(signals)[len(signals) // 2] if signals else 0.25
    return {"what": "push phase inside the fused kernel, from its %globaltimer trace "
                    "(benchmarks/trace_fused_gemm.py): first finished accumulator -> last bulk "
                    "store issued, against bytes pushed per rank",
            "alpha_us": round(alpha, 3), "beta_us_per_byte": beta, "link_gb_s": round(rate / 1e3, 1),
            "signal_us": round(signal_us, 3), "visibility_us": visibility_us,
            "tau_min_bytes": int(rate * (signal_us + visibility_us)), "points": rows}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="calibration/b200.json")
    ap.add_argument("--max-bytes", type=int, default=256 << 20)
    ap.add_argument("--from-trace", nargs="+", default=None,
                    help="fit the in-kernel model from trace_fused_gemm.py logs (no GPU needed)")
    args = ap.parse_args()
    if args.from_trace:
        fit = fit_in_kernel(args.from_trace)
        try:
            with open(args.out) as f:
                data = json.load(f)
        except (OSError, ValueError):
            data = {}
        data["in_kernel"] = fit
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            json.dump(data, f, indent=1)
        print(json.dumps({k: v for k, v in fit.items() if k != "points"}))
        return
    rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import tileccl_b200 as tccl
    from tileccl_b200 import ops
    from tileccl_b200.planning import (CalibrationPoint, CostModelCalibrator, HardwareProfile,
                                       Interconnect)

    ctx = tccl.init(heap_size=args.max_bytes + (64 << 20))
    buf = ctx.zeros(args.max_bytes, dtype=torch.uint8)
    points, rows = [], []
    nbytes = 4096
    while nbytes <= args.max_bytes:
        view = buf[:nbytes]
        for _ in range(3):
            ops.broadcast(view, ctx=ctx, root=0)
        torch.cuda.synchronize()
        dist.barrier()
        iters = 50 if nbytes <= (1 << 20) else 10
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            ops.broadcast(view, ctx=ctx, root=0)
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / iters * 1e3], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item())
        # bytes that leave the root per call
        sent = nbytes * (1 if ctx.heap.has_multicast else ws - 1)
        points.append(CalibrationPoint(sent, 1, "int8", us))
        rows.append({"bytes": nbytes, "bytes_on_wire": sent, "us": us, "gbps": sent / us / 1e3})
        nbytes *= 4
    if rank == 0:
        alpha, beta, floor = CostModelCalibrator.calibrate_two_regime(points)
        base = HardwareProfile.from_interconnect(Interconnect.NVLINK_5)
        prof = HardwareProfile(alpha, beta, base.gemm_tflops_fp16, base.gemm_efficiency, floor,
                               "NVLink 5 / NVSwitch (B200), calibrated")
        out = {"alpha_us": alpha, "beta_us_per_byte": beta, "min_comm_us": floor,
               "bandwidth_gb_s": prof.bandwidth_gb_s,
               "tau_min_bytes_90pct": CostModelCalibrator.saturation_bytes(prof, 0.9),
               "world_size": ws, "nvls": ctx.heap.has_multicast, "points": rows}
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            json.dump(out, f, indent=1)
        print(json.dumps({k: v for k, v in out.items() if k != "points"}))
    ctx.barrier()
    ctx.heap.cleanup()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
