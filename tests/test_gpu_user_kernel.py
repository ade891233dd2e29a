"""A kernel written outside the library, built against csrc/device/*.cuh and run on the heap."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _example():
    sys.path.insert(0, os.path.join(ROOT, "examples"))
    import custom_kernel

    return custom_kernel


@pytest.mark.parametrize("world_size", [2, 4, 8])
def test_custom_kernel_emulated_ranks(world_size):
    """One cooperative grid, CTA r plays rank r: device tile_allreduce, tile_put,
    tile_signal / tile_wait and tile_barrier inside a user kernel."""
    _example().run(world_size, n=4096 + 3, real=False, calls=3)


def test_custom_kernel_one_launch_per_gpu():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    _example().run(min(n, 4), real=True, calls=3)


def test_barrier_put_mc_get_reduce_on_real_gpus():
    """tile_barrier across GPUs, and the two NVLS verbs where a multicast mapping is bound."""
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs two GPUs")
    import tileccl_b200 as tccl
    from tileccl_b200.primitives import harness

    ctxs = tccl.init_local(n, 64 << 20)
    try:
        heaps = [c.heap for c in ctxs]
        ctr = [h.allocate_signal_buffer(8) for h in heaps]
        for epoch in (1, 2, 3):
            res = harness.run_concurrent([(h, "barrier", {"a": c.data_ptr(), "value": epoch})
                                          for h, c in zip(heaps, ctr)])
            assert all(r[0] == 1 for r in res), res
            assert all(int(c[0]) == epoch * n for c in ctr)
        # a barrier that one rank never joins gives up and says so (bounded wait)
        res = harness.run_concurrent([(h, "barrier", {"a": c.data_ptr() + 4, "value": 1,
                                                      "budget_us": 3000})
                                      for h, c in list(zip(heaps, ctr))[:-1]])
        assert all(r[0] == 0 for r in res), res
        if not heaps[0].has_multicast:
            pytest.skip("no NVLS multicast mapping bound on this machine")
        src = [h.allocate_tensor((2048,), torch.float32) for h in heaps]
        dst = [h.allocate_tensor((2048,), torch.float32) for h in heaps]
        for r in range(n):
            src[r].copy_(torch.arange(2048, dtype=torch.float32) * (r + 1))
            dst[r].zero_()
        for c in ctxs:
            torch.cuda.synchronize(c.torch_device)
        # rank 1's tile lands in every rank's dst through one multicast store per 16 bytes
        harness.run(heaps[1], "put_mc", a=src[1].data_ptr(), b=dst[1].data_ptr(), nbytes=8192)
        for r in range(n):
            assert torch.equal(dst[r].cpu(), src[1].cpu()), r
        # rank 0 reads the switch-reduced sum of every rank's src
        harness.run(heaps[0], "get_reduce", a=src[0].data_ptr(), b=dst[0].data_ptr(), nbytes=8192,
                    sub_op=2)
        want = torch.arange(2048, dtype=torch.float32) * sum(r + 1 for r in range(n))
        assert torch.equal(dst[0].cpu(), want)
    finally:
        for c in ctxs:
            torch.cuda.synchronize(c.torch_device)
        for c in ctxs:
            c.heap.cleanup()
