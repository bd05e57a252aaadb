"""HGRN2: linear attention in which the forget gate also decides what is written.

Per head, with q = silu(W_q h) (``dim`` channels), v = W_v h (``vdim``) and the
forget gate f = l + (1 - l) sigmoid(W_f h + b) bounded below by l per channel,

    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,      o_t = S_t^T q_t.

There is no key and no other scale.  Each head's o is RMS-normed over ``vdim``
with one weight shared by the heads, the heads are concatenated and projected
out.  The state S (dim x vdim per head, float32) starts at zero and lives in the
request's state slot; gates, state and sums are 32-bit (``csrc/hgrn2.cu``)."""

from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorDecl, register_part


class HGRN2(Mixer):
    KIND = "hgrn2"

    def __init__(self, width: int, heads: int, dim: int, vdim: int, eps: float, dtype=torch.float32, device="cuda"):
        self.width, self.heads, self.dim, self.vdim = width, heads, dim, vdim
        self.eps, self.dtype = float(eps), dtype
        self.in_weight = None

    def tensors(self):
        H = self.heads
        return {"q_weight": TensorDecl((H * self.dim, self.width), "matrix"),
                "f_weight": TensorDecl((H * self.dim, self.width), "matrix"),
                "f_bias": TensorDecl((H * self.dim,), "vector"),
                "lower": TensorDecl((H * self.dim,), "vector"),
                "v_weight": TensorDecl((H * self.vdim, self.width), "matrix"),
                "norm": TensorDecl((self.vdim,), "vector"),
                "out_weight": TensorDecl((self.width, H * self.vdim), "matrix")}

    def bind(self, tensors):
        """The three projections of the input become one product (q | f | v, rows padded to a multiple of 8)."""
        super().bind(tensors)
        nq, nv = self.heads * self.dim, self.heads * self.vdim
        fused = torch.zeros((-(-(2 * nq + nv) // 8) * 8, self.width), dtype=self.q_weight.dtype, device=self.q_weight.device)
        fused[:nq], fused[nq:2 * nq], fused[2 * nq:2 * nq + nv] = self.q_weight, self.f_weight, self.v_weight
        self.in_weight = fused
        self.q_weight, self.f_weight, self.v_weight = fused[:nq], fused[nq:2 * nq], fused[2 * nq:2 * nq + nv]

    def cache_need(self):
        return StateNeed((self.heads, self.dim, self.vdim), torch.float32)

    def forward(self, h, residual, ctx, cache):
        """residual + mix(h); with ``residual`` None the mixer's output alone, float32 [T, width]."""
        state = ctx.cache.state_layer(cache.group, cache.layer)
        T, H = h.shape[0], self.heads
        proj = ops.linear(h, self.in_weight, None, out_dtype=torch.float32)
        o = ops.hgrn2(proj, state, self.f_bias, self.lower, ctx, H, self.dim, self.vdim)
        normed = ops.rmsnorm(o.view(T * H, self.vdim), self.norm, self.eps, self.dtype)
        return ops.linear(normed.view(T, H * self.vdim), self.out_weight, None, residual=residual,
                          out_dtype=torch.float32, out=residual)


register_part(HGRN2.KIND, HGRN2)
