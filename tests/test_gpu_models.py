"""TP-MLP block (all-gather -> gated GEMM -> GEMM -> reduce-scatter) and the AG -> GEMM chain."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("ws", [1, 2, 4])
def test_tp_mlp_matches_fp32_reference(ws):
    import tileccl_b200 as tccl
    from tileccl_b200.models.tp_mlp import smoke_forward

    ctxs = tccl.init_local(ws, 256 << 20)
    try:
        smoke_forward(ctxs, tokens=512, hidden=256, ffn=1024)
    finally:
        for d in range(torch.cuda.device_count()):
            torch.cuda.synchronize(d)
        for c in ctxs:
            c.heap.cleanup()


def test_allgather_gemm_column_shards():
    import tileccl_b200 as tccl
    from tileccl_b200 import ops

    ws = 2
    ctxs = tccl.init_local(ws, 256 << 20)
    try:
        M, K, N = 256, 128, 256
        torch.manual_seed(0)
        x = (torch.randn(M, K) / K ** 0.5).half()
        w = torch.randn(K, N).half()
        shards = [c.zeros(M, K // ws, dtype=torch.float16) for c in ctxs]
        for r, s in enumerate(shards):
            s.copy_(x[:, r * K // ws:(r + 1) * K // ws])
        W = [w.to(c.torch_device) for c in ctxs]
        out = [c.zeros(M, N, dtype=torch.float16) for c in ctxs]
        for r, c in enumerate(ctxs):
            ops.allgather_gemm_reducescatter(shards[r], W[r], out[r], ctx=c)
        for c in ctxs:
            ops.check_status(c)
        ref = x.float() @ w.float()
        for r in range(ws):
            err = (out[r].float().cpu() - ref).abs().max().item() / ref.abs().max().item()
            assert err < 1e-2
    finally:
        for d in range(torch.cuda.device_count()):
            torch.cuda.synchronize(d)
        for c in ctxs:
            c.heap.cleanup()
