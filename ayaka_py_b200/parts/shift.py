"""Token shift: every channel of a sublayer's input is blended with the previous token's.

h_t = x_t + (x_(t-1) - x_t) * mu, one coefficient per channel, with x_(-1) = 0 for a
sequence's first token.  The previous token's x (before the blend) is the request's state
(float32, in its slot), so a prompt may be cut anywhere."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, StateNeed, TensorDecl, register_part


class TokenShift(Part):
    KIND = "token_shift"

    def __init__(self, width: int, dtype=torch.float32, device="cuda"):
        self.width, self.dtype = width, dtype
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.width,), "vector")}

    def cache_need(self):
        return StateNeed((self.width,), torch.float32)

    def forward(self, x, ctx, cache):
        """x: residual stream [T, width] float32.  Returns the blended rows in the compute dtype
        and leaves each request's last row in its state."""
        state = ctx.cache.state_layer(cache.group, cache.layer)
        return ops.token_shift(x, self.weight, state, ctx, self.dtype)

    def convert(self, x):
        """The stream as it is, in the compute dtype (float32: the stream itself)."""
        return x if self.dtype == torch.float32 else ops.token_shift(x, None, None, None, self.dtype)


register_part(TokenShift.KIND, TokenShift)
