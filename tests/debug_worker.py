"""Child process of tests/test_gpu_debug_build.py: runs with TILECCL_DEBUG=1, i.e. on the
native library compiled with recorded bounds checks.  Two ranks driven by one process
(emulated on one GPU, or two real GPUs when present).  Every call here is one that a
release build would also complete without a fault: the out-of-heap "symmetric" addresses
used below are valid device memory (the other rank's copy of the buffer) and the target
rank of the translation is the caller itself, so the only difference the checks make is
that the access is recorded and skipped."""

import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "examples"))

import tileccl_b200 as tccl  # noqa: E402
from tileccl_b200 import debug, ops  # noqa: E402
from tileccl_b200.primitives import harness  # noqa: E402


def main() -> None:
    assert debug.enabled(), "run with TILECCL_DEBUG=1"
    ctxs = tccl.init_local(2, 64 << 20)
    try:
        assert debug.is_debug_build()
        h0, h1 = ctxs[0].heap, ctxs[1].heap
        a0 = ctxs[0].zeros(1024, dtype=torch.float32)
        a1 = ctxs[1].zeros(1024, dtype=torch.float32)
        ramp = torch.arange(1024, dtype=torch.float32, device=h0.device)

        # 1. in-bounds traffic records nothing
        a0.copy_(ramp)
        harness.run(h0, "put", peer=1, a=a0.data_ptr(), b=a0.data_ptr(), nbytes=4096)
        assert torch.equal(a1.cpu(), ramp.cpu())
        harness.run(h0, "get", peer=1, a=a0.data_ptr(), b=a0.data_ptr(), nbytes=4096)
        assert debug.read_records(h0.device) == []

        # 2. a "symmetric" destination outside the caller's heap: recorded, nothing moves
        a1.zero_()
        harness.run(h0, "put", peer=0, a=a0.data_ptr(), b=a1.data_ptr(), nbytes=4096)
        recs = debug.read_records(h0.device)
        assert len(recs) == 1, recs
        r = recs[0]
        assert (r["source"], r["code"], r["rank"], r["count"]) == ("primitives", 3, 0, 128), r
        assert r["addr"] == a1.data_ptr() and r["bytes"] == 4096, r
        assert float(a1.abs().sum()) == 0.0, "the out-of-heap put must have been skipped"
        assert debug.read_records(h0.device) == []          # reading cleared the record

        # 3. the same through check(): raises with the facts, context stays usable
        harness.run(h0, "remote_store", peer=0, a=a0.data_ptr(), b=a1.data_ptr(), nbytes=4096)
        try:
            debug.check(h0.device)
        except debug.TileCCLDebugError as exc:
            assert "span leaves the owner's heap" in str(exc), exc
        else:
            raise AssertionError("debug.check() did not raise")
        assert float(a1.abs().sum()) == 0.0

        # 4. collectives of the debug library: right answers, no record
        xs = [c.randn(300_000, dtype=torch.float16) for c in ctxs]
        want = xs[0].float().cpu() + xs[1].float().cpu()
        for c, x in zip(ctxs, xs):
            ops.allreduce(x, ctx=c)
        for c in ctxs:
            torch.cuda.synchronize(c.torch_device)
        for x in xs:
            err = (x.float().cpu() - want).abs().max().item() / want.abs().max().item()
            assert err < 2e-2, err
        outs = [c.zeros(2 * 4096, dtype=torch.float32) for c in ctxs]
        parts = [c.randn(4096, dtype=torch.float32) for c in ctxs]
        for c, p, o in zip(ctxs, parts, outs):
            ops.allgather(p, o, ctx=c)
        for c in ctxs:
            torch.cuda.synchronize(c.torch_device)
        gathered = torch.cat([p.cpu() for p in parts])
        for o in outs:
            assert torch.equal(o.cpu(), gathered)
        for c in ctxs:
            assert debug.read_records(c.torch_device) == []
    finally:
        for c in ctxs:
            torch.cuda.synchronize(c.torch_device)
        for c in ctxs:
            c.heap.cleanup()

    # 5. a user kernel compiled with the checks: runs clean
    import custom_kernel

    custom_kernel.run(2, n=4096 + 3, real=False, calls=2, debug=True)
    print("debug worker ok")


if __name__ == "__main__":
    main()
