"""A state-space mixer in the manner of Mamba-2 (a scalar decay per head, the state an outer-product memory).

With inner = heads * head_dim, N = state_dim and G groups, for the normed input x of a token:
  [z | xs | B | C | dt] = x W_in^T                          widths inner, inner, G N, G N, heads
  [xs | B | C] <- silu(short causal convolution + bias)     (`conv`; state: its last taps - 1 inputs)
  dt_h = softplus(dt_h + dt_bias_h)
  S_h <- exp(-exp(A_log_h) dt_h) S_h + dt_h B_g xs_h^T      S_h is N x head_dim, zero at admission, g = h / (heads / G)
  y_h = S_h^T C_g + D_h xs_h
  y <- y * silu(z); every one of `norm_groups` equal parts of y divided by its own root mean square; times `norm`
  out = y W_o^T
The recurrent state, dt, the decay and the norm are 32-bit; the state is carried per request in the cache manager's
state slots, so a request may be fed in portions of any size.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FixedState, Mixer, StateBundle, pad_rows, register_mixer
from .conv import ShortConv


class Mamba2Mixer(Mixer):
    def __init__(self, w_in: torch.Tensor, wo: torch.Tensor, conv: ShortConv, dt_bias: torch.Tensor, a_log: torch.Tensor,
                 d_skip: torch.Tensor, norm_weight: torch.Tensor, *, heads: int, head_dim: int, state_dim: int,
                 groups: int, norm_groups: int, norm_eps: float):
        self.w_in, self.wo, self.conv = w_in, wo, conv
        self.dt_bias, self.a_log, self.d_skip, self.norm_weight = dt_bias, a_log, d_skip, norm_weight
        self.heads, self.head_dim, self.state_dim = int(heads), int(head_dim), int(state_dim)
        self.groups, self.norm_groups, self.norm_eps = int(groups), int(norm_groups), float(norm_eps)
        self.inner = self.heads * self.head_dim
        self.conv_width = self.inner + 2 * self.groups * self.state_dim
        self.proj_width = self.inner + self.conv_width + self.heads
        self.width = wo.shape[0]
        if w_in.numel() and w_in.shape[0] != self.proj_width:
            raise ValueError(f"the input projection has {w_in.shape[0]} rows, expected {self.proj_width}")
        self.w_in = pad_rows(w_in)                          # result rows start on 16-byte boundaries
        self.proj_width = max(self.proj_width, self.w_in.shape[0])
        if self.heads % self.groups:
            raise ValueError(f"heads {self.heads} is not a multiple of groups {self.groups}")
        if self.inner % self.norm_groups:
            raise ValueError(f"inner width {self.inner} is not a multiple of norm_groups {self.norm_groups}")
        if self.state_dim > 256:
            raise ValueError(f"state size {self.state_dim} is above 256, the most the scan kernel keeps in registers")
        if conv.channels != self.conv_width:
            raise ValueError(f"the convolution has {conv.channels} channels, x|B|C have {self.conv_width}")

    def state_need(self):
        return StateBundle((FixedState((self.heads, self.head_dim, self.state_dim), torch.float32), self.conv.state_need()))

    def forward(self, x, ctx, cache):
        memory, tail = cache
        T = x.shape[0]
        proj = ctx.buf("ssm_proj", (T, self.proj_width), torch.float32)
        ops.linear(x, self.w_in, proj)
        xbc = self.conv.forward(proj, self.inner, None, ctx, tail, tag="ssm_xbc")        # also moves the tail on
        y = ctx.buf("ssm_y", (T, self.inner), torch.float32)
        ops.ssm_scan(xbc, proj, self.inner + self.conv_width, self.dt_bias, self.a_log, self.d_skip, memory.state, y,
                     self.heads, self.groups, self.head_dim, self.state_dim, ctx, writes=memory.writes)
        normed = ctx.buf("ssm_normed", (T, self.inner), ctx.act_dtype)
        ops.gated_group_norm(y, proj, 0, self.norm_weight, self.norm_eps, self.norm_groups, normed, ctx)
        out = ctx.buf("branch_out", (T, self.width), torch.float32)
        ops.linear(normed, self.wo, out)
        return out


register_mixer("mamba2", Mamba2Mixer)
