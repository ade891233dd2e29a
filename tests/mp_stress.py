"""Stress worker (one rank per GPU under torchrun): thousands of back-to-back fused calls
with inputs that change on every call and a device-side check of EVERY result.

What it is for: a TileGroup signal that overtook the data it announces, a staging slot
reused too early or a stale epoch would leave tiles of an earlier call in the output; with
inputs that differ from call to call that shows up as a mismatch.  Both signal forms run
(``TILECCL_TUNING=1``: relaxed add after a completed bulk store, ``=0``: release add).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        tests/mp_stress.py --calls 2000
"""

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--calls", type=int, default=2000)
    ap.add_argument("--full-check-every", type=int, default=50)
    args = ap.parse_args()
    rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import tileccl_b200 as tccl
    from tileccl_b200 import ops

    def gather(t):
        out = [torch.empty_like(t) for _ in range(ws)]
        dist.all_gather(out, t.contiguous())
        return out

    def value(call, r):
        return ((call * 7 + r * 3) % 13 + 1) / 16.0

    failures = []
    for tuning in ("1", "0"):
        os.environ["TILECCL_TUNING"] = tuning
        ctx = tccl.init(heap_size=1 << 30)
        gen = torch.Generator(device=dev)
        gen.manual_seed(4242 + rank)
        mloc, N, K = 1024, 2048, 512
        M = mloc * ws
        # all-gather problem: A_r [mloc, K] @ B_r [K, N] -> C [M, N]
        A = torch.empty(mloc, K, device=dev, dtype=torch.float16)
        B = (torch.randn(K, N, device=dev, generator=gen) * K ** -0.5).half()
        C = ctx.zeros(M, N, dtype=torch.float16)
        colsum = [b.float().sum(0) for b in gather(B)]                  # [N] per rank
        # reduce-scatter problem: A2_r [M, K/ws] @ B2_r [K/ws, N] summed -> C2 [mloc, N]
        kl = K // ws
        A2 = torch.empty(M, kl, device=dev, dtype=torch.float16)
        B2 = (torch.randn(kl, N, device=dev, generator=gen) * K ** -0.5).half()
        C2 = torch.zeros(mloc, N, device=dev, dtype=torch.float16)
        colsum2 = [b.float().sum(0) for b in gather(B2)]
        bad = torch.zeros(2, device=dev, dtype=torch.int32)             # mismatching calls (AG, RS)
        worst = torch.zeros(2, device=dev, dtype=torch.float32)
        tol = 6e-3
        for call in range(args.calls):
            full = args.full_check_every > 0 and call % args.full_check_every == args.full_check_every - 1
            if full:
                A.copy_(torch.randn(mloc, K, device=dev, generator=gen) * 0.5)
                A2.copy_(torch.randn(M, kl, device=dev, generator=gen) * 0.5)
            else:
                A.fill_(value(call, rank))
                A2.fill_(value(call, rank))
            ops.gemm_allgather_rows(A, B, C, ctx=ctx)
            ops.gemm_reducescatter_rows(A2, B2, C2, ctx=ctx)
            if full:
                ref = torch.cat([a.float() @ b.float() for a, b in zip(gather(A), gather(B))])
                ref2 = sum(a[rank * mloc:(rank + 1) * mloc].float() @ b.float()
                           for a, b in zip(gather(A2), gather(B2)))
            else:
                ref = torch.cat([(value(call, r) * colsum[r]).expand(mloc, N) for r in range(ws)])
                ref2 = sum(value(call, r) * colsum2[r] for r in range(ws)).expand(mloc, N)
            e1 = (C.float() - ref).abs().max() / ref.abs().max()
            e2 = (C2.float() - ref2).abs().max() / ref2.abs().max()
            err = torch.stack([e1, e2])
            bad += (err > tol).to(torch.int32)
            worst = torch.maximum(worst, err)
        ops.check_status(ctx)
        t = torch.cat([bad.float(), worst])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        nb_ag, nb_rs, w_ag, w_rs = t.tolist()
        if rank == 0:
            print(f"stress tuning={tuning} ws={ws} calls={args.calls}: mismatching calls AG {int(nb_ag)} "
                  f"RS {int(nb_rs)}; worst rel err AG {w_ag:.2e} RS {w_rs:.2e}", flush=True)
        if nb_ag or nb_rs:
            failures.append((tuning, nb_ag, nb_rs))
        dist.barrier()
        torch.cuda.synchronize()
        ctx.heap.cleanup()
    dist.barrier()
    dist.destroy_process_group()
    if failures:
        print(f"MP_STRESS_FAILED {failures}", flush=True)
        return 1
    if rank == 0:
        print("MP_STRESS_OK", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
