"""One process per GPU.

    torchrun --nproc_per_node=<gpus> --master-addr 127.0.0.1 examples/multiprocess.py
"""

import os

import torch
import torch.distributed as dist

import tileccl


def main() -> None:
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local))
    ctx = tileccl.init(backend="auto", heap_size=512 * 1024 * 1024)

    M, K, N = 4096, 4096, 8192
    A = ctx.randn(M // ctx.world_size, K, dtype=torch.float16)
    A.mul_(K ** -0.5)
    B = ctx.randn(K, N, dtype=torch.float16)
    C = ctx.zeros(M, N, dtype=torch.float16)
    tileccl.ops.gemm_allgather_rows(A, B, C, ctx=ctx)      # C holds every rank's rows on return
    tileccl.ops.check_status(ctx)
    rows = M // ctx.world_size
    mine = C[ctx.rank * rows:(ctx.rank + 1) * rows]
    err = (mine.float() - A.float() @ B.float()).abs().max().item()
    print(f"[rank {ctx.rank}] nvls={ctx.heap.has_multicast} max error of own rows: {err:.3e}")
    ctx.barrier()
    ctx.heap.cleanup()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
