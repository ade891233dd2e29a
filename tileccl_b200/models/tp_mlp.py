"""Tensor-parallel, sequence-parallel SwiGLU MLP block.

``y = (silu(x @ W_gate) * (x @ W_up)) @ W_down`` with the FFN dimension sharded
over ranks and activations sharded over tokens:

    x_shard [T/ws, H] --all-gather--> X [T, H]
    H1 = silu(X @ W_gate_r) * (X @ W_up_r)          [T, F/ws]   (one fused GEMM)
    y_shard = reduce-scatter_rows(H1 @ W_down_r)    [T/ws, H]   (one fused GEMM)

Two kernel launches per forward: the first GEMM gathers ``x`` itself while it
computes (``parallel.chain.rows_allgather_gemm``) and applies the SiLU-gate in
its epilogue; the second reduce-scatters its partial sums from its epilogue
(``ops._fused.reduce_scatter``).  The reference has no model layer; this is the
"TP MLP" benchmark configuration built from its operator set.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import fused_gemm as fg
from ..ops import _fused
from ..parallel.chain import rows_allgather_gemm

GATE_BLOCK = fg.BLOCK_N // 2  # 128 gate columns followed by 128 up columns per 256-column tile


def pack_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """Interleave ``[H, F]`` gate and up projections in 128-column blocks: ``[H, 2F]``."""
    H, F = w_gate.shape
    if w_up.shape != w_gate.shape:
        raise ValueError("w_gate and w_up must have the same shape")
    if F % GATE_BLOCK:
        raise ValueError(f"FFN shard width {F} must be a multiple of {GATE_BLOCK}")
    g = w_gate.reshape(H, F // GATE_BLOCK, 1, GATE_BLOCK)
    u = w_up.reshape(H, F // GATE_BLOCK, 1, GATE_BLOCK)
    return torch.cat([g, u], dim=2).reshape(H, 2 * F).contiguous()


class TPMLP:
    """One rank's shard of the block.  Weights: N(0, 0.02), seeded per (seed, rank)."""

    def __init__(self, ctx, *, tokens: int, hidden: int = 4096, ffn: int = 14336,
                 dtype: torch.dtype = torch.bfloat16, seed: int = 0, name: str = "tp_mlp",
                 weights: Optional[tuple] = None):
        ws, rank = ctx.world_size, ctx.rank
        if ffn % ws or tokens % ws:
            raise ValueError("ffn and tokens must be divisible by world_size")
        self.ctx, self.name = ctx, name
        self.tokens, self.hidden, self.ffn, self.dtype = tokens, hidden, ffn, dtype
        self.f_local = ffn // ws
        self.t_local = tokens // ws
        dev = ctx.torch_device
        if weights is None:
            gen = torch.Generator(device=dev)
            gen.manual_seed(seed * 1000 + rank)
            mk = lambda r, c: (torch.randn(r, c, device=dev, generator=gen) * 0.02).to(dtype)
            w_gate, w_up, w_down = mk(hidden, self.f_local), mk(hidden, self.f_local), mk(self.f_local, hidden)
        else:
            w_gate, w_up, w_down = (w.to(device=dev, dtype=dtype) for w in weights)
        self.w_gate, self.w_up, self.w_down = w_gate, w_up, w_down.contiguous()
        self.w_gu = pack_gate_up(w_gate, w_up)
        # Gathered activations live on the heap; the rank's own rows are the input buffer.
        self.x_full = ctx.zeros(tokens, hidden, dtype=dtype)
        self.h1 = torch.empty(tokens, self.f_local, dtype=dtype, device=dev)
        self.y = torch.empty(self.t_local, hidden, dtype=dtype, device=dev)

    @property
    def x_local(self) -> torch.Tensor:
        """Rows of ``x_full`` owned by this rank: write the input shard here (zero-copy)."""
        r = self.ctx.rank
        return self.x_full[r * self.t_local:(r + 1) * self.t_local]

    def forward(self, x_shard: Optional[torch.Tensor] = None) -> torch.Tensor:
        if x_shard is not None and x_shard.data_ptr() != self.x_local.data_ptr():
            self.x_local.copy_(x_shard)
        rows_allgather_gemm(self.ctx, f"{self.name}:up", self.x_full, self.w_gu, self.h1,
                            epilogue="silu_gate")
        _fused.reduce_scatter(self.ctx, f"{self.name}:down", self.h1, self.w_down, self.y,
                              split_axis=0)
        return self.y

    __call__ = forward

    def flops(self) -> float:
        """FLOPs this rank performs per forward."""
        return 2.0 * self.tokens * self.hidden * self.f_local * 3


def reference_forward(x_full: torch.Tensor, shards: list) -> torch.Tensor:
    """fp32 PyTorch reference of the unsharded block from the per-rank weight shards."""
    x = x_full.float()
    y = torch.zeros(x.shape[0], shards[0].w_down.shape[1], dtype=torch.float32, device=x.device)
    for m in shards:
        h = torch.nn.functional.silu(x @ m.w_gate.float().to(x.device)) * (x @ m.w_up.float().to(x.device))
        y += h @ m.w_down.float().to(x.device)
    return y


def smoke_forward(ctxs, tokens: int = 512, hidden: int = 256, ffn: int = 1024) -> None:
    """Tiny forward on the given single-process contexts, checked against fp32 PyTorch."""
    ws = len(ctxs)
    mlps = [TPMLP(ctx, tokens=tokens, hidden=hidden, ffn=ffn, dtype=torch.bfloat16, seed=0)
            for ctx in ctxs]
    gen = torch.Generator(device=ctxs[0].torch_device)
    gen.manual_seed(7)
    x = torch.randn(tokens, hidden, device=ctxs[0].torch_device, generator=gen).to(torch.bfloat16)
    t = tokens // ws
    for r, m in enumerate(mlps):
        m.x_local.copy_(x[r * t:(r + 1) * t].to(m.x_local.device))
    for it in range(2):
        outs = [m.forward() for m in mlps]
    for ctx in ctxs:
        _fused.check_status(ctx)
    ref = reference_forward(x, mlps)
    for r, y in enumerate(outs):
        want = ref[r * t:(r + 1) * t].to(y.device)
        err = (y.float() - want).abs().max().item() / (want.abs().max().item() + 1e-9)
        if err > 3e-2:
            raise AssertionError(f"TP-MLP mismatch on rank {r}: rel err {err:.3e}")
