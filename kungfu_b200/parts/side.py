"""A per-layer input looked up by token id, gated by the residual stream.

For a token with id v and residual row x (after the block's feed-forward), with a table row e = table[v, col0:col0 + dim]:
  g = gelu_tanh(W_gate x) * e;   y = W_proj g;   x <- x + rms_norm(y) * w
`forward` returns y; the block adds its norm to the residual (`norm.add_into`), together with the next block's first norm.
Layers share one table and read their own columns of it.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Norm, Part


class TokenSide(Part):
    def __init__(self, table: torch.Tensor, col0: int, dim: int, w_gate: torch.Tensor, w_proj: torch.Tensor, norm: Norm):
        self.table, self.col0, self.dim = table, int(col0), int(dim)
        self.w_gate, self.w_proj, self.norm = w_gate, w_proj, norm
        self.width = w_proj.shape[0]

    def forward(self, x, ctx) -> torch.Tensor:
        """x: the residual rows in the element type products take; returns 32-bit [rows, width]."""
        T = x.shape[0]
        gate = ctx.buf("side_gate", (T, self.dim), torch.float32)
        ops.linear(x, self.w_gate, gate)
        g = ctx.buf("side_g", (T, self.dim), ctx.act_dtype)
        ops.side_gate(gate, ctx.tokens, self.table, self.col0, g)
        y = ctx.buf("side_out", (T, self.width), torch.float32)
        ops.linear(g, self.w_proj, y)
        return y
