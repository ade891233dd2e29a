#!/usr/bin/env python
"""Phase-0 calibration of the alpha-beta link model on this machine.

Measures peer pushes (the broadcast collective from rank 0: one direct NVLink hop
per peer) over a range of sizes, fits ``time = alpha + beta * bytes`` (plus the
small-message floor) with ``CostModelCalibrator`` and writes the result, together
with the derived P2P saturation size tau_min, to a JSON file that
``HardwareProfile.b200_measured`` / ``TILECCL_CALIBRATION`` pick up.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/phase0_calibrate.py --out calibration/b200.json
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
    ap.add_argument("--out", default="calibration/b200.json")
    ap.add_argument("--max-bytes", type=int, default=256 << 20)
    args = ap.parse_args()
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
