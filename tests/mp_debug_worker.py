"""One process per GPU with TILECCL_DEBUG=1: every collective call is followed by the
debug epilogue (status words, recorded bounds checks, epoch invariants of the counter block).
Launched by tests/test_gpu_multiprocess.py through torchrun."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import tileccl_b200 as tccl
    from tileccl_b200 import debug, ops

    assert debug.enabled()
    ctx = tccl.init(heap_size=256 << 20)
    assert debug.is_debug_build()

    def rel(got, ref):
        return (got.float() - ref.float()).abs().max().item() / (ref.float().abs().max().item() + 1e-9)

    for call in range(3):
        for n in (300_000 // ws * ws, 2_000_000 // ws * ws):
            x = ctx.randn(n, dtype=torch.float32)
            ref = x.clone()
            dist.all_reduce(ref)
            ops.allreduce(x, ctx=ctx)                      # two-shot: checked after the call
            assert rel(x, ref) < 1e-5
            part = ctx.randn(n // ws, dtype=torch.float32)
            out = ctx.zeros(n, dtype=torch.float32)
            want = torch.empty(n, dtype=torch.float32, device=dev)
            dist.all_gather_into_tensor(want, part)
            ops.allgather(part, out, ctx=ctx)
            assert torch.equal(out, want)
            rs = ctx.zeros(n // ws, dtype=torch.float32)
            ops.reduce_scatter(out, rs, ctx=ctx)
            assert rel(rs, want[rank * (n // ws):(rank + 1) * (n // ws)] * ws) < 1e-5
            root = call % ws
            b = ctx.randn(n, dtype=torch.float32)
            wantb = b.clone()
            dist.broadcast(wantb, src=root)
            ops.broadcast(b, ctx=ctx, root=root)
            assert torch.equal(b, wantb)
            sc = ctx.zeros(n // ws, dtype=torch.float32)
            ops.scatter(b, sc, ctx=ctx, root=root)
            assert torch.equal(sc, wantb[rank * (n // ws):(rank + 1) * (n // ws)])
        ctx.barrier()
        ctx.heap.reset_allocator()
    if ws >= 3:                                             # relay broadcast, debug epilogue too
        os.environ["TILECCL_BCAST_RELAY_MIN_BYTES"] = str(8 << 20)
        big = ctx.zeros((9 << 20) // 4, dtype=torch.float32)
        for root in (0, ws - 1):
            big.fill_(float(rank + 1))
            ops.broadcast(big, ctx=ctx, root=root)
            assert float(big.min()) == float(big.max()) == float(root + 1)
    assert debug.read_records(dev) == []
    dist.barrier()
    torch.cuda.synchronize()
    ctx.heap.cleanup()
    dist.destroy_process_group()
    if rank == 0:
        print("MP_DEBUG_OK", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
