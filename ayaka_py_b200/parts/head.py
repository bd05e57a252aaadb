"""Logits of the wanted rows: h @ W[:V]^T (times a constant), no bias, float32 out
(``models/_common.py:248-253``, ``layers/embedding.py:741-747``)."""

from __future__ import annotations

import torch

from .. import ops
from .base import Head, TensorDecl, register_part


class LMHead(Head):
    KIND = "lm_head"

    def __init__(self, vocab: int, width: int, scale: float = 1.0, dtype=torch.float32, device="cuda"):
        self.vocab, self.width, self.scale = vocab, width, float(scale)
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.vocab, self.width), "matrix")}

    def forward(self, h, ctx):
        logits = ops.linear(h, self.weight, None, out_dtype=torch.float32)
        return logits if self.scale == 1.0 else ops.scale_(logits, self.scale)

    def lower(self, builder, h):
        from ..engine.program import LOGITS
        if self.scale != 1.0:
            from .base import NotLowered
            raise NotLowered("the step program has no scaled head")
        return builder.linear(h, self.weight, None, out_dtype=torch.float32, out=LOGITS, wanted=True)


register_part(LMHead.KIND, LMHead)
