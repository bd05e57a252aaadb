"""A short causal convolution over time on every channel, added to its input.

``TimeConv`` sits between a sublayer's norm and the sublayer: what the sublayer
reads is h + conv(h), conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j), with zeros
before the sequence's start.  The last taps - 1 inputs h of a request are its
state (float32, in the request's slot), so a prompt may be cut anywhere.  The
norm before it and the convolution run as one kernel: the part takes the
residual stream and the norm part, not the normed rows."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, StateNeed, TensorDecl, register_part


class TimeConv(Part):
    KIND = "time_conv"

    def __init__(self, width: int, taps: int, dtype=torch.float32, device="cuda"):
        if not 1 <= taps <= 16:
            raise ValueError(f"a time convolution of {taps} taps: the kernels hold 1 to 16")
        self.width, self.taps, self.dtype = width, taps, dtype
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.width, self.taps), "vector")}

    def bind(self, tensors):
        """The kernel reads a tap of neighbouring channels at a time: the weight is kept tap-major."""
        super().bind(tensors)
        self.weight_taps = self.weight.t().contiguous()           # [taps, width]

    def cache_need(self):
        return StateNeed((max(self.taps - 1, 1), self.width), torch.float32)

    def forward(self, x, norm, ctx, cache):
        """x: residual stream [T, width] float32; norm: the RMS norm part in front.  Returns
        h + conv(h), h = norm(x), in the compute dtype, and brings the state up to date."""
        state = ctx.cache.state_layer(cache.group, cache.layer)
        if self.taps == 1:
            state = state[:, :0]
        return ops.rmsnorm_conv(x, norm.weight, self.weight_taps, state, ctx, norm.eps, self.dtype)


register_part(TimeConv.KIND, TimeConv)
