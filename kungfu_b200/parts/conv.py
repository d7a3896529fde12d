"""A short causal convolution over time, one filter per channel.

y_t[c] = sum_j w[c, j] u_(t - taps + 1 + j)[c] for j = 0..taps-1 (the last column of w multiplies the current token),
zeros before the first token of a sequence; optionally a bias after the sum and an activation (silu).
A step brings only some of a request's tokens, so the last taps - 1 inputs of every live request are kept as a
fixed-size state [taps - 1, channels] in 32-bit, zeroed at admission.

The input is a column range of a 32-bit projection result (with an optional bias of the projection added as the values
are read); a mixer that fuses the convolution into a kernel of its own (`ops.qkv_prepare`) uses only `state_need`
and `commit` of this part.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FixedState, Part


class ShortConv(Part):
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None, activation: str | None = None):
        if activation not in (None, "none", "silu"):
            raise ValueError(f"activation {activation!r} of a short convolution is not one of none, silu")
        self.weight, self.bias = weight, bias           # [channels, taps], [channels]
        self.channels, self.taps = int(weight.shape[0]), int(weight.shape[1])
        self.activation = activation
        if not (1 <= self.taps <= 8):
            raise ValueError(f"a short convolution has 1 to 8 taps, found {self.taps}")

    def state_need(self):
        return FixedState((max(self.taps - 1, 1), self.channels), torch.float32)

    def forward(self, proj, col0: int, in_bias, ctx, state_view, tag: str = "conv_out") -> torch.Tensor:
        """32-bit [rows, channels]: the convolution of columns col0.. of `proj` (+ in_bias) over each request's rows; the
        state is moved on to the end of the step's rows (in the same kernel when no request has more than one row)."""
        out = ctx.buf(tag, (proj.shape[0], self.channels), torch.float32)
        inline = state_view.writes and bool(getattr(ctx, "decode_only", False))
        done = ops.short_conv(proj, col0, in_bias, self.weight, self.bias, self.activation, state_view.state, out, ctx,
                              commit_inline=inline)
        if not done:
            self.commit(proj, col0, in_bias, ctx, state_view)
        return out

    def commit(self, proj, col0: int, in_bias, ctx, state_view) -> None:
        """Move the state on to the end of this step's rows; call after everything that reads the old state."""
        if state_view.writes:
            ops.short_conv_commit(proj, col0, in_bias, self.channels, self.taps, state_view.state, ctx,
                                  w_dtype=self.weight.dtype)
