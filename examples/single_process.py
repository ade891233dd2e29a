"""One process drives every visible GPU (two emulated ranks if there is only one GPU).

    python examples/single_process.py
"""

import torch

import tileccl


def main() -> None:
    world = max(2, torch.cuda.device_count())
    ctxs = tileccl.init_local(world, 512 * 1024 * 1024)
    M, K, N = 2048, 1024, 2048
    torch.manual_seed(0)
    a = (torch.randn(M, K) / K ** 0.5).half()
    b = torch.randn(K, N).half()
    A = [a.to(c.device) for c in ctxs]
    B = [b.to(c.device) for c in ctxs]
    C = [c.zeros(M, N, dtype=torch.float16) for c in ctxs]
    for ctx, x, w, out in zip(ctxs, A, B, C):
        tileccl.ops.gemm_allscatter(x, w, out, ctx=ctx)
    ref = a.float() @ b.float()
    for ctx, out in zip(ctxs, C):
        tileccl.ops.check_status(ctx)
        err = (out.float().cpu() - ref).abs().max().item()
        print(f"[rank {ctx.rank} on {ctx.device}] max error vs fp32 matmul: {err:.3e}")
    for ctx in ctxs:
        ctx.heap.cleanup()


if __name__ == "__main__":
    main()
