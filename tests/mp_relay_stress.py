"""One process per GPU (three or more): large relayed broadcasts, every call checked.

Each call the root's buffer holds a pattern that depends on the call number and the other
ranks hold a different one; after the broadcast every rank compares its whole buffer with the
root's pattern on the device.  Sizes are the ones where a piece flag that overtakes its data
shows up as stale pieces (hundreds of MiB keep the links saturated for most of a call).
Launched by tests/test_gpu_multiprocess.py through torchrun."""

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--calls", type=int, default=24)
    ap.add_argument("--mib", type=int, nargs="+", default=[512, 96])
    ap.add_argument("--bulk", type=int, default=0, help="1: the bulk-copy form of the relay")
    args = ap.parse_args()
    os.environ["TILECCL_BCAST_RELAY_BULK"] = str(args.bulk)
    rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import tileccl_b200 as tccl
    from tileccl_b200 import ops
    from tileccl_b200.primitives import collectives as coll

    os.environ.setdefault("TILECCL_BCAST_RELAY_MIN_BYTES", str(8 << 20))   # the relay is opt-in
    ctx = tccl.init(heap_size=(max(args.mib) << 20) + (64 << 20))
    bad = torch.zeros(1, dtype=torch.int64, device=dev)
    for mib in args.mib:
        n = (mib << 20) // 4
        ctx.barrier()
        ctx.heap.reset_allocator()
        buf = ctx.empty(n, dtype=torch.int32)
        assert coll._relay_ok(ctx.heap, n * 4, buf.data_ptr()), "expected the relay path"
        ramp = torch.arange(n, dtype=torch.int32, device=dev)
        for call in range(args.calls):
            root = call % ws
            # root: ramp + 7 * call; the others: something that differs everywhere
            buf.copy_(ramp + (7 * call if rank == root else -1 - call - 1000 * rank))
            ops.broadcast(buf, ctx=ctx, root=root)
            bad += (buf != ramp + 7 * call).sum()
        coll.check_status(ctx.heap)
    dist.all_reduce(bad)
    ok = int(bad.item()) == 0
    dist.barrier()
    torch.cuda.synchronize()
    ctx.heap.cleanup()
    dist.destroy_process_group()
    if rank == 0:
        print("MP_RELAY_OK" if ok else f"MP_RELAY_MISMATCH {int(bad.item())} elements", flush=True)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
