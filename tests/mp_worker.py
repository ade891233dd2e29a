"""Worker of tests/test_gpu_multiprocess.py: one rank per GPU under torchrun.

Checks the multi-process heap (fd exchange, NVLS when available), the fused
operators in every push mode, the collectives with and without NVLS, and the
TP-MLP block, against references built with NCCL all-gathers of the inputs.
Exits non-zero on the first mismatch (so that torchrun tears all ranks down)."""

import os
import sys
import traceback

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
    from tileccl_b200 import ops
    from tileccl_b200.kernels import fused_gemm as fg
    from tileccl_b200.models.tp_mlp import TPMLP
    from tileccl_b200.ops import _fused
    from tileccl_b200.primitives import collectives as coll

    ctx = tccl.init(heap_size=1 << 30)
    assert ctx.heap.mode == "multiprocess" and ctx.heap.transport_strategy == "vmm_fd"

    def gather(t):
        out = [torch.empty_like(t) for _ in range(ws)]
        dist.all_gather(out, t.contiguous())
        return out

    def check(name, got, ref, tol):
        err = (got.float() - ref.float()).abs().max().item() / (ref.float().abs().max().item() + 1e-9)
        if not err < tol:
            raise AssertionError(f"[rank {rank}] {name}: rel err {err:.3e} >= {tol}")

    torch.manual_seed(100 + rank)
    modes = [fg.PUSH_STORES, fg.PUSH_TMA] + ([fg.PUSH_MULTIMEM] if ctx.heap.has_multicast else [])
    for dtype, tol in ((torch.float16, 5e-3), (torch.bfloat16, 2e-2)):
        for push in modes:
            M, N, K = 256 * ws, 1024, 512
            mloc = M // ws
            A = ctx.randn(mloc, K, dtype=dtype)
            A.mul_(K ** -0.5)
            B = ctx.randn(K, N, dtype=dtype)
            C = ctx.zeros(M, N, dtype=dtype)
            for _ in range(3):
                _fused.push_all(ctx, f"t_ag_{push}", A, B, C, region_row0=rank * mloc, region_col0=0,
                                push_mode=push)
            ops.check_status(ctx)
            As, Bs = gather(A), gather(B)
            check(f"gemm_allgather push{push} {dtype}", C,
                  torch.cat([As[r].float() @ Bs[r].float() for r in range(ws)]), tol)
            dist.barrier()
            if push == fg.PUSH_MULTIMEM:
                continue
            A2 = ctx.randn(M, K // ws, dtype=dtype)
            A2.mul_(K ** -0.5)
            B2 = ctx.randn(K // ws, N, dtype=dtype)
            C2 = torch.zeros(mloc, N, dtype=dtype, device=dev)
            for _ in range(4):
                _fused.reduce_scatter(ctx, f"t_rs_{push}", A2, B2, C2, split_axis=0, push_mode=push)
            ops.check_status(ctx)
            A2s, B2s = gather(A2), gather(B2)
            full = sum(A2s[r].float() @ B2s[r].float() for r in range(ws))
            check(f"gemm_reducescatter push{push} {dtype}", C2, full[rank * mloc:(rank + 1) * mloc], tol)
            dist.barrier()

    # Many more tiles than CTAs: every CTA goes from remote tiles to its own (reducing)
    # tiles while signals of its last remote tiles are still held back.
    M, N, K = 8192, 2048, 256 * ws
    mloc = M // ws
    A3 = ctx.randn(M, K // ws, dtype=torch.float16)
    A3.mul_(K ** -0.5)
    B3 = ctx.randn(K // ws, N, dtype=torch.float16)
    C3 = torch.zeros(mloc, N, dtype=torch.float16, device=dev)
    for _ in range(3):
        _fused.reduce_scatter(ctx, "t_rs_large", A3, B3, C3, split_axis=0)
    ops.check_status(ctx)
    A3s, B3s = gather(A3), gather(B3)
    full = sum(A3s[r].float() @ B3s[r].float() for r in range(ws))
    check("gemm_reducescatter large", C3, full[rank * mloc:(rank + 1) * mloc], 5e-3)
    C4 = ctx.zeros(M, N, dtype=torch.float16)
    A4 = ctx.randn(mloc, K, dtype=torch.float16)
    A4.mul_(K ** -0.5)
    B4 = ctx.randn(K, N, dtype=torch.float16)
    for _ in range(3):
        _fused.push_all(ctx, "t_ag_large", A4, B4, C4, region_row0=rank * mloc, region_col0=0)
    ops.check_status(ctx)
    A4s, B4s = gather(A4), gather(B4)
    check("gemm_allgather large", C4,
          torch.cat([A4s[r].float() @ B4s[r].float() for r in range(ws)]), 5e-3)
    dist.barrier()

    # Entry handshake: back-to-back all-gathers into the same C with a slow consumer on
    # rank 0 in between.  The peers' second call must not overwrite rank 0's C before rank 0
    # has entered that call itself, i.e. before its consumer (sleep + snapshot) has run.
    M, N, K = 512 * ws, 1024, 256
    mloc = M // ws
    Ae = ctx.randn(mloc, K, dtype=torch.float16)
    Ae.mul_(K ** -0.5)
    Be = ctx.randn(K, N, dtype=torch.float16)
    Ce = ctx.zeros(M, N, dtype=torch.float16)
    snap = torch.empty_like(Ce)
    for rep in range(3):
        Ae.copy_(torch.full_like(Ae, 0.01 * (rep + 1)))       # call 1 data
        _fused.push_all(ctx, "t_entry", Ae, Be, Ce, region_row0=rank * mloc, region_col0=0)
        want1 = torch.cat([t.float() @ b.float() for t, b in zip(gather(Ae), gather(Be))])
        if rank == 0:
            torch.cuda._sleep(20_000_000)                      # ~10 ms: the slow consumer
        snap.copy_(Ce)
        Ae.copy_(torch.full_like(Ae, -0.02 * (rep + 1)))       # call 2 data
        _fused.push_all(ctx, "t_entry", Ae, Be, Ce, region_row0=rank * mloc, region_col0=0)
        ops.check_status(ctx)
        check(f"entry handshake: consumer of call 1 (rep {rep})", snap, want1, 5e-3)
        want2 = torch.cat([t.float() @ b.float() for t, b in zip(gather(Ae), gather(Be))])
        check(f"entry handshake: call 2 (rep {rep})", Ce, want2, 5e-3)
        dist.barrier()

    # tile_barrier across processes, and the two NVLS verbs when a multicast mapping is bound
    from tileccl_b200.primitives import harness

    bar = ctx.heap.allocate_signal_buffer(8)
    dist.barrier()
    for epoch in (1, 2, 3):
        res = harness.run(ctx.heap, "barrier", a=bar.data_ptr(), value=epoch, budget_us=2e6)
        assert res[0] == 1 and int(bar[0]) == epoch * ws, (res, bar.tolist())
    if ctx.heap.has_multicast:
        src = ctx.zeros(2048, dtype=torch.float32)
        dst = ctx.zeros(2048, dtype=torch.float32)
        src.copy_(torch.arange(2048, dtype=torch.float32, device=dev) * (rank + 1))
        torch.cuda.synchronize()
        dist.barrier()
        if rank == ws - 1:       # one multicast store per 16 bytes lands the tile on every rank
            harness.run(ctx.heap, "put_mc", a=src.data_ptr(), b=dst.data_ptr(), nbytes=8192)
        torch.cuda.synchronize()
        dist.barrier()
        check("tile_put_mc", dst, torch.arange(2048, dtype=torch.float32, device=dev) * ws, 1e-7)
        dist.barrier()
        harness.run(ctx.heap, "get_reduce", a=src.data_ptr(), b=dst.data_ptr(), nbytes=8192, sub_op=2)
        check("tile_get_reduce", dst,
              torch.arange(2048, dtype=torch.float32, device=dev) * sum(range(1, ws + 1)), 1e-6)
        dist.barrier()

    for nvls_off in ("1", "0"):
        os.environ["TILECCL_DISABLE_NVLS"] = nvls_off
        os.environ["TILECCL_FORCE_NVLS"] = "1"       # also at two ranks
        for dtype, tol in ((torch.float16, 2e-2), (torch.float32, 1e-5)):
            for n in (1024, 8198, 1_000_000):
                n = n // ws * ws
                x = ctx.randn(n, dtype=dtype)
                orig = x.clone()
                ops.allreduce(x, ctx=ctx)
                ref = orig.float().clone()
                dist.all_reduce(ref)
                check(f"allreduce n{n} {dtype} nvls_off={nvls_off}", x, ref, tol)
                out = ctx.zeros(n * ws, dtype=dtype)
                x.copy_(orig)
                ops.allgather(x, out, ctx=ctx)
                check(f"allgather n{n}", out, torch.cat(gather(orig)), 1e-7)
                part = ctx.zeros(n // ws, dtype=dtype)
                ops.reduce_scatter(x, part, ctx=ctx)
                check(f"reduce_scatter n{n}", part, ref[rank * (n // ws):(rank + 1) * (n // ws)], tol)
                b = ctx.randn(n, dtype=dtype)
                bl = gather(b)
                ops.broadcast(b, ctx=ctx, root=ws - 1)
                check(f"broadcast n{n}", b, bl[ws - 1], 1e-7)
                sc = ctx.zeros(n // ws, dtype=dtype)
                ops.scatter(x, sc, ctx=ctx, root=0)
                check(f"scatter n{n}", sc, gather(x)[0][rank * (n // ws):(rank + 1) * (n // ws)], 1e-7)
                dist.barrier()
    # rooted collectives with the root changing from call to call
    rb = ctx.zeros(8192, dtype=torch.float32)
    for call, root in enumerate([0, 1, 0, ws - 1, 1]):
        rb.fill_(float(10 * call + rank))
        ops.broadcast(rb, ctx=ctx, root=root)
        check(f"broadcast alternating root call {call}", rb,
              torch.full_like(rb, float(10 * call + root)), 1e-7)
    dist.barrier()
    coll.check_status(ctx.heap)
    os.environ["TILECCL_DISABLE_NVLS"] = "0"
    os.environ["TILECCL_FORCE_NVLS"] = "0"
    # large broadcast: pipelined relay from three ranks on (root sends every piece once, the
    # others forward theirs); sizes repeat and roots alternate so several epochs are covered
    if ws >= 3:
        os.environ["TILECCL_BCAST_RELAY_MIN_BYTES"] = str(8 << 20)   # (default: from 64 MiB)
        big = ctx.zeros((12 << 20) // 4 + 4096, dtype=torch.float32)
        assert coll._relay_ok(ctx.heap, big.numel() * 4, big.data_ptr())
        for call, root in enumerate([0, ws - 1, 1, 0, 2]):
            gen = torch.Generator(device=dev).manual_seed(1000 + 10 * call + rank)
            big.copy_(torch.rand(big.numel(), device=dev, generator=gen))
            want = gather(big)[root]
            ops.broadcast(big, ctx=ctx, root=root)
            check(f"relay broadcast call {call} root {root}", big, want, 1e-7)
        dist.barrier()
        coll.check_status(ctx.heap)
        del os.environ["TILECCL_BCAST_RELAY_MIN_BYTES"]

    tokens, hidden, ffn = 128 * ws * 2, 512, 256 * ws
    mlp = TPMLP(ctx, tokens=tokens, hidden=hidden, ffn=ffn, dtype=torch.bfloat16, seed=3)
    gen = torch.Generator(device=dev).manual_seed(11)
    x_full = torch.randn(tokens, hidden, device=dev, generator=gen).bfloat16()   # same on every rank
    t = tokens // ws
    mlp.x_local.copy_(x_full[rank * t:(rank + 1) * t])
    dist.barrier()
    for _ in range(3):
        y = mlp.forward()
    ops.check_status(ctx)
    ref = torch.zeros(tokens, hidden, device=dev)
    for wg, wu, wd in zip(gather(mlp.w_gate), gather(mlp.w_up), gather(mlp.w_down)):
        h = torch.nn.functional.silu(x_full.float() @ wg.float()) * (x_full.float() @ wu.float())
        ref += h @ wd.float()
    check("tp_mlp", y, ref[rank * t:(rank + 1) * t], 3e-2)
    dist.barrier()
    torch.cuda.synchronize()
    ctx.heap.cleanup()
    dist.destroy_process_group()
    if rank == 0:
        print("MP_WORKER_OK", flush=True)
    return 0


if __name__ == "__main__":
    try:
        code = main()
    except BaseException:
        traceback.print_exc()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(3)
    sys.exit(code)
