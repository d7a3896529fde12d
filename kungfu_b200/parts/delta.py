"""A gated delta-rule mixer: a recurrent memory per head that is decayed, corrected towards each token's value and read.

With H heads, KH query/key heads of size d and values of size dv, for the normed input x of a token:
  [q | k | v | b | a | g] = x W_in^T            widths KH d, KH d, H dv, H, and a, g as below (one product)
  [q | k | v] <- silu(short causal convolution over time, per channel)   (`conv`; state: its last taps - 1 inputs)
  q, k <- unit vectors per head (x / sqrt(sum x^2 + 1e-6)); q also times d^-1/2; head h reads q/k head h // (H / KH)
  beta_h = sigmoid(b_h)
  decay:  per head      g_h  = exp(-exp(A_log_h) softplus(a_h + dt_bias_h))               a: H columns
          per channel   g_hi = exp(-exp(A_log_h) softplus((W_a2 a)_hi + dt_bias_hi))      a: a low-rank row, W_a2 [H d, rank]
  S_h <- diag(g_h) S_h;  u = beta_h (v_h - S_h^T k_h);  S_h <- S_h + k_h u^T;  o_h = S_h^T q_h          S_h: d x dv
  o_h <- o_h / rms(o_h) * w (one weight vector for all heads), times a gate:
          silu(g) with g H dv columns of the product, or sigmoid(W_g2 g) with g a low-rank row (W_g2 [H dv, rank])
  y = o W_o^T
The state, the decays, beta, the unit norms and the output norm are 32-bit; the state starts at zero and is carried per
request in the cache manager's state slots, so a request may be fed in portions of any size.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FixedState, Mixer, StateBundle, pad_rows, register_mixer
from .conv import ShortConv


class GatedDeltaMixer(Mixer):
    def __init__(self, w_in: torch.Tensor, wo: torch.Tensor, conv: ShortConv, dt_bias: torch.Tensor, a_log: torch.Tensor,
                 norm_weight: torch.Tensor, *, heads: int, kv_heads: int, dim: int, vdim: int, norm_eps: float,
                 w_a2: torch.Tensor | None = None, w_g2: torch.Tensor | None = None, gate: str = "silu"):
        """`w_a2` given: one decay per head and key channel, from a low-rank row of the product; `w_g2` given: the gate
        comes from a low-rank row likewise.  `gate`: silu or sigmoid."""
        if heads % kv_heads:
            raise ValueError(f"heads {heads} is not a multiple of kv_heads {kv_heads}")
        if dim > 256:
            raise ValueError(f"key size {dim} is above 256, the most the recurrence kernel keeps in registers")
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"gate {gate!r} is not one of silu, sigmoid")
        self.wo, self.conv = wo, conv
        self.dt_bias, self.a_log, self.norm_weight = dt_bias, a_log, norm_weight
        self.w_a2, self.w_g2, self.gate = w_a2, w_g2, gate
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.norm_eps = float(norm_eps)
        self.per_channel = w_a2 is not None
        self.width = wo.shape[0]
        self.qkv_width = 2 * self.kv_heads * self.dim + self.heads * self.vdim
        self.a_width = int(w_a2.shape[1]) if (w_a2 is not None and w_a2.numel()) else self.heads
        self.g_width = int(w_g2.shape[1]) if (w_g2 is not None and w_g2.numel()) else self.heads * self.vdim
        self.b_col = self.qkv_width
        self.a_col = self.b_col + self.heads
        self.g_col = self.a_col + self.a_width
        want = self.g_col + self.g_width
        if w_in.numel() and w_in.shape[0] != want:
            raise ValueError(f"the input projection has {w_in.shape[0]} rows, expected {want}")
        self.w_in = pad_rows(w_in)                          # result rows start on 16-byte boundaries
        self.proj_width = max(want, self.w_in.shape[0])
        if conv.channels != self.qkv_width:
            raise ValueError(f"the convolution has {conv.channels} channels, q|k|v have {self.qkv_width}")

    def state_need(self):
        return StateBundle((FixedState((self.heads, self.dim, self.vdim), torch.float32), self.conv.state_need()))

    def forward(self, x, ctx, cache):
        memory, tail = cache
        T = x.shape[0]
        H, KH, d, dv = self.heads, self.kv_heads, self.dim, self.vdim
        proj = ctx.buf("delta_proj", (T, self.proj_width), torch.float32)
        ops.linear(x, self.w_in, proj)
        qkv = self.conv.forward(proj, 0, None, ctx, tail, tag="delta_qkv")              # also moves the tail on
        if self.per_channel:
            decay, decay0 = ctx.buf("delta_decay", (T, H * d), torch.float32), 0
            ops.linear_cols(proj, self.a_col, self.w_a2, decay)
        else:
            decay, decay0 = proj, self.a_col
        if self.w_g2 is not None:
            gate, gate0 = ctx.buf("delta_gate", (T, H * dv), torch.float32), 0
            ops.linear_cols(proj, self.g_col, self.w_g2, gate)
        else:
            gate, gate0 = proj, self.g_col
        o = ctx.buf("delta_o", (T, H * dv), torch.float32)
        ops.delta_rule(qkv, 0, KH * d, 2 * KH * d, proj, self.b_col, decay, decay0, self.per_channel, self.dt_bias, self.a_log,
                       memory.state, o, H, KH, d, dv, ctx, writes=memory.writes)
        normed = ctx.buf("delta_normed", (T, H * dv), ctx.act_dtype)
        ops.head_norm_gate(o, self.norm_weight, self.norm_eps, gate, gate0, self.gate, normed, H, dv)
        y = ctx.buf("branch_out", (T, self.width), torch.float32)
        ops.linear(normed, self.wo, y)
        return y


register_mixer("gated_delta", GatedDeltaMixer)
