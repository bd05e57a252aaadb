"""Token embedding, fused with a learned position table when the position
encoding offers one (``models/gpt2.py:516-517``), or multiplied by a constant."""

from __future__ import annotations

import torch

from .. import ops
from .base import Embedding, TensorDecl, register_part


class TokenEmbedding(Embedding):
    KIND = "token_embedding"

    def __init__(self, vocab: int, width: int, scale: float = 1.0, dtype=torch.float32, device="cuda"):
        self.vocab, self.width, self.scale = vocab, width, float(scale)
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.vocab, self.width), "matrix")}

    def forward(self, ctx, position):
        table = position.embedding_table()
        if self.scale != 1.0:
            if table is not None:
                raise ValueError("a scaled embedding takes no position table")
            return ops.embed_scaled(ctx.tokens, self.weight, self.scale)
        return ops.embed(ctx.tokens, ctx.positions, self.weight, table)

    def lower(self, builder, position):
        if self.scale != 1.0:
            from .base import NotLowered
            raise NotLowered("the step program has no scaled embedding")
        return builder.embed(self.weight, position.embedding_table())


register_part(TokenEmbedding.KIND, TokenEmbedding)
