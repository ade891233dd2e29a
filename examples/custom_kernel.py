"""Compile and run ``custom_kernel.cu``: a user kernel built on the device primitives.

    python examples/custom_kernel.py              # one GPU: CTA r of one cooperative grid plays rank r
    python examples/custom_kernel.py --real 2     # one launch per GPU on 2 GPUs (single process)

Checks the all-reduced vector and the token each rank received from its left neighbour.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import tileccl_b200 as tccl  # noqa: E402
from tileccl_b200 import userkernel  # noqa: E402

SOURCE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "custom_kernel.cu")


def run(world_size: int = 4, n: int = 4096, real: bool = False, calls: int = 3,
        debug: bool = False) -> None:
    """``debug=True`` compiles the kernel with the recorded bounds checks and verifies at the
    end that none of them fired."""
    mod = userkernel.compile(SOURCE, debug=debug)
    devices = list(range(world_size)) if real else [0] * world_size
    ctxs = tccl.init_local(world_size, 64 << 20, devices=devices)
    try:
        data = [c.zeros(n, dtype=torch.float32) for c in ctxs]
        sync = [c.zeros(64, dtype=torch.int32) for c in ctxs]
        token = [c.zeros(4, dtype=torch.int32) for c in ctxs]
        status = [torch.zeros(8, dtype=torch.int32, device=c.torch_device) for c in ctxs]
        for epoch in range(1, calls + 1):
            if real:
                for r, c in enumerate(ctxs):      # one CTA per GPU; the GPUs run side by side
                    mod.launch(c, [data[r].data_ptr(), n, sync[r].data_ptr(), epoch, 0,
                                   token[r].data_ptr(), status[r].data_ptr()], grid=1, block=256)
            else:                                  # rank 0's addresses, CTA r translates to rank r
                mod.launch(ctxs[0], [data[0].data_ptr(), n, sync[0].data_ptr(), epoch, 1,
                                     token[0].data_ptr(), status[0].data_ptr()],
                           grid=world_size, block=256)
            for c in ctxs:
                torch.cuda.synchronize(c.torch_device)
            scale = sum(r + 1 for r in range(world_size))
            want = torch.arange(n, dtype=torch.float32).remainder(7).add(1).mul(scale)
            for r in range(world_size):
                assert int(status[r if real else 0][0]) == 0, f"device wait gave up: {status[r].tolist()}"
                assert torch.equal(data[r].cpu(), want), f"rank {r}: wrong all-reduce result"
                left = (r - 1) % world_size
                assert int(token[r][0]) == 1000 * epoch + left, f"rank {r}: wrong token"
        if debug:
            for c in ctxs:
                with torch.cuda.device(c.torch_device):
                    rec = mod.debug_record()
                    assert rec.enabled == 1 and rec.count == 0, rec.to_dict("custom_kernel")
        print(f"custom kernel ok: world_size={world_size} real_gpus={real} calls={calls}"
              + (" (bounds checks on)" if debug else ""))
    finally:
        for c in ctxs:
            torch.cuda.synchronize(c.torch_device)
        for c in ctxs:
            c.heap.cleanup()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--real", type=int, default=0, help="run on this many real GPUs")
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--debug", action="store_true", help="compile with recorded bounds checks")
    args = ap.parse_args()
    run(args.real or args.ranks, real=bool(args.real), debug=args.debug)
