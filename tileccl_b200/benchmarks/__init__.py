"""In-process benchmarks behind ``tileccl bench`` (single process driving the GPUs).

Every number is device time from CUDA events, after warm-up, with an L2 flush
between iterations; with several GPUs the slowest rank counts.  The multi-process
(one rank per GPU) benchmarks of the fused operators are ``bench.py`` at the
repository root and ``benchmarks/collectives_sweep.py``.
"""

from __future__ import annotations

import time
from typing import Callable, Optional

_FLUSH_BYTES = 256 << 20


def _torch():
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("benchmarks need a CUDA device")
    return torch


def _contexts(world_size: int, heap_bytes: int):
    import tileccl_b200 as tccl

    torch = _torch()
    ws = world_size or torch.cuda.device_count()
    return tccl.init_local(ws, heap_bytes)


def _time_group(ctxs, fn: Callable[[int], None], *, warmup: int, iters: int) -> float:
    """fn(r) issues rank r's work; returns mean ms per iteration, max over ranks."""
    torch = _torch()
    devs = sorted({c.torch_device for c in ctxs}, key=str)
    flush = {d: torch.empty(_FLUSH_BYTES, dtype=torch.uint8, device=d) for d in devs}

    def sync():
        for d in devs:
            torch.cuda.synchronize(d)

    for _ in range(warmup):
        for r in range(len(ctxs)):
            fn(r)
    sync()
    totals = [0.0] * len(ctxs)
    for _ in range(iters):
        for d in devs:
            flush[d].zero_()
        sync()
        evs = []
        for r, c in enumerate(ctxs):
            with torch.cuda.device(c.torch_device):
                s = torch.cuda.Event(enable_timing=True)
                s.record()
                evs.append([s, None])
        for r in range(len(ctxs)):
            fn(r)
        for r, c in enumerate(ctxs):
            with torch.cuda.device(c.torch_device):
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                evs[r][1] = e
        sync()
        for r, (s, e) in enumerate(evs):
            totals[r] += s.elapsed_time(e)
    return max(totals) / iters


def _cleanup(ctxs) -> None:
    torch = _torch()
    for d in range(torch.cuda.device_count()):
        torch.cuda.synchronize(d)
    for c in ctxs:
        c.heap.cleanup()


def bench_gemm(quick: bool = False) -> dict:
    """tcgen05 GEMM against torch.matmul (cuBLAS) on one GPU."""
    torch = _torch()
    from tileccl_b200.kernels.fused_gemm import gemm
    from tileccl_b200.utils.profiling import device_time_ms

    shapes = [(8192, 4096, 1024), (16384, 4096, 1024)] if quick else \
        [(8192, 4096, 1024), (8192, 4096, 2048), (16384, 4096, 1024), (8192, 8192, 8192)]
    rows = []
    for (M, N, K) in shapes:
        a = (torch.randn(M, K, device="cuda") / K ** 0.5).half()
        b = torch.randn(K, N, device="cuda").half()
        c = torch.empty(M, N, device="cuda", dtype=torch.float16)
        ours = device_time_ms(lambda: gemm(a, b, c), flush_l2_bytes=_FLUSH_BYTES)
        lib = device_time_ms(lambda: torch.matmul(a, b, out=c), flush_l2_bytes=_FLUSH_BYTES)
        rows.append({"name": f"gemm_{M}x{N}x{K}_fp16", "ms": ours, "tflops": 2 * M * N * K / ours / 1e9,
                     "cublas_ms": lib, "cublas_tflops": 2 * M * N * K / lib / 1e9})
    return {"suite": "gemm", "rows": rows, "timestamp": time.time()}


def bench_p2p(world_size: int = 0, quick: bool = False) -> dict:
    """Point-to-point primitives between rank 0 and rank 1 through the symmetric heap:
    ``translate_ptr`` (one launch of pointer arithmetic), small ``tile_put`` / ``tile_get``
    latency (one CTA, device time of one launch) and grid-wide put / get bandwidth.
    Counterpart of the reference's translate / put / get benchmark behind ``tileccl bench p2p``
    (tileccl/cli.py:212)."""
    torch = _torch()
    from tileccl_b200 import _native
    from tileccl_b200.primitives import harness
    from tileccl_b200.utils.profiling import device_time_ms

    ctxs = _contexts(world_size or min(2, max(2, torch.cuda.device_count())), 1 << 30)
    try:
        rows = []
        h0 = ctxs[0].heap
        dev0 = ctxs[0].torch_device
        shared_gpu = len({str(c.torch_device) for c in ctxs[:2]}) < 2
        small = [c.zeros(2048, dtype=torch.float32) for c in ctxs]
        result = torch.zeros(4, dtype=torch.int32, device=dev0)

        def prim(op, nbytes):
            _native.call("tccl_prim_test", harness.OPS[op], 0, 0, h0.world_size, 1, h0.window_base,
                         h0.stride, 0, small[0].data_ptr(), small[0].data_ptr(), nbytes, 0, 0,
                         result.data_ptr(), 10 ** 9, torch.cuda.current_stream().cuda_stream)

        with torch.cuda.device(dev0):
            for op, nbytes in (("translate", 0), ("put", 16), ("put", 8192), ("get", 16),
                               ("get", 8192)):
                ms = device_time_ms(lambda: prim(op, nbytes), warmup=5, iters=50)
                rows.append({"name": f"{op}_{nbytes}B_one_cta", "us": ms * 1e3})
            sizes = [16 << 20] if quick else [1 << 20, 16 << 20, 256 << 20]
            sms = torch.cuda.get_device_properties(dev0).multi_processor_count
            for nbytes in sizes:
                src = ctxs[0].zeros(nbytes // 4, dtype=torch.float32)
                for c in ctxs[1:]:
                    c.zeros(nbytes // 4, dtype=torch.float32)        # same offset on every rank
                for direction, name in ((0, "put"), (1, "get")):
                    grid = max(1, min(2 * sms, nbytes // 16 // 512 // 8))
                    ms = device_time_ms(
                        lambda: _native.call("tccl_p2p_copy", direction, 0, h0.world_size, 1,
                                             h0.window_base, h0.stride, src.data_ptr(),
                                             src.data_ptr(), nbytes, grid,
                                             torch.cuda.current_stream().cuda_stream),
                        warmup=3, iters=10, flush_l2_bytes=_FLUSH_BYTES)
                    rows.append({"name": f"{name}_{nbytes}B_grid{grid}", "ms": ms,
                                 "gbps": nbytes / ms / 1e6})
        return {"suite": "p2p", "world_size": len(ctxs), "rows": rows, "timestamp": time.time(),
                "note": ("both ranks share one GPU: the numbers are local-memory figures"
                         if shared_gpu else "rank 0 and rank 1 on different GPUs")}
    finally:
        _cleanup(ctxs)


def bench_collectives(world_size: int = 0, quick: bool = False) -> dict:
    """Bus bandwidth of the five tile collectives (fp16)."""
    torch = _torch()
    ctxs = _contexts(world_size, 3 << 30)
    ws = len(ctxs)
    try:
        from tileccl_b200.primitives import collectives as coll

        sizes = [1 << 20, 64 << 20] if quick else [4 << 10, 64 << 10, 1 << 20, 16 << 20, 256 << 20]
        rows = []
        for nbytes in sizes:
            n = max(ws, nbytes // 2 // ws * ws)
            full = [c.zeros(n, dtype=torch.float16) for c in ctxs]
            part = [c.zeros(n // ws, dtype=torch.float16) for c in ctxs]
            cases = {
                "allreduce": (lambda r: coll.allreduce(full[r], ctxs[r].heap), 2 * (ws - 1) / ws),
                "allgather": (lambda r: coll.allgather(part[r], full[r], ctxs[r].heap), (ws - 1) / ws),
                "reduce_scatter": (lambda r: coll.reduce_scatter(full[r], part[r], ctxs[r].heap),
                                   (ws - 1) / ws),
                "broadcast": (lambda r: coll.broadcast(full[r], ctxs[r].heap, root=0), 1.0),
                "scatter": (lambda r: coll.scatter(full[r], part[r], ctxs[r].heap, root=0),
                            (ws - 1) / ws),
            }
            for name, (fn, factor) in cases.items():
                ms = _time_group(ctxs, fn, warmup=3, iters=10)
                rows.append({"name": f"{name}_{n * 2}B_ws{ws}", "ms": ms,
                             "bus_gbps": n * 2 * factor / ms / 1e6})
            for c in ctxs:
                coll.check_status(c.heap)
        return {"suite": "collective", "world_size": ws, "rows": rows, "timestamp": time.time()}
    finally:
        _cleanup(ctxs)


def bench_patterns(M: int = 8192, N: int = 4096, K: int = 2048, pattern: Optional[str] = None,
                   world_size: int = 0, quick: bool = False) -> dict:
    """The four GEMM + all-scatter overlap patterns on one shape."""
    torch = _torch()
    ctxs = _contexts(world_size, 3 << 30)
    try:
        from tileccl_b200 import ops
        from tileccl_b200.patterns import PATTERN_ALIASES, PATTERN_CLASSES

        names = [PATTERN_ALIASES.get(pattern, pattern)] if pattern else list(PATTERN_CLASSES)
        A = [(torch.randn(M, K, device=c.torch_device) / K ** 0.5).half() for c in ctxs]
        B = [torch.randn(K, N, device=c.torch_device).half() for c in ctxs]
        C = [c.zeros(M, N, dtype=torch.float16) for c in ctxs]
        rows = []
        for name in names:
            ms = _time_group(ctxs, lambda r: ops.gemm_allscatter(A[r], B[r], C[r], ctx=ctxs[r],
                                                                 pattern=name),
                             warmup=2 if quick else 3, iters=5 if quick else 10)
            rows.append({"name": f"{name}_{M}x{N}x{K}_ws{len(ctxs)}", "ms": ms,
                         "tflops_per_gpu": 2 * M * N * K / ms / 1e9})
        for c in ctxs:
            ops.check_status(c)
        return {"suite": "pattern", "world_size": len(ctxs), "rows": rows, "timestamp": time.time()}
    finally:
        _cleanup(ctxs)


def render(payload: dict) -> str:
    from tileccl_b200.utils.profiling import format_benchmark_table

    head = f"== {payload.get('suite')} (world_size {payload.get('world_size', 1)}) =="
    return head + "\n" + format_benchmark_table(payload.get("rows", []))
