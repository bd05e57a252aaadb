"""Sigmoid attention: causal attention whose weights are not normalized over the keys.

q = W_q h + b_q, k = W_k h + b_k, v = W_v h + b_v, with ``heads`` query heads sharing
``kv_heads`` key/value heads, query/key size ``dim`` and value size ``vdim`` per head.  The
whole query row (all heads at once) is RMS-normed with a weight of its size, and so is the
whole key row; then the first ``rot.dims`` dimensions of every head are rotated by the position
(dimension i paired with i + dims/2).  With s = (q . k) scale, the weight of a visible key
(every position up to the query's) is sigmoid(cap tanh(s / cap) + b_head): there is no softmax,
and the output is the plain weighted sum of the values, projected out.

Rotated keys and the values are cached in pages (separate head sizes); norms, angles, scores
and weights are 32-bit (``csrc/attention_gated.cu``)."""

from __future__ import annotations

import torch

from .. import ops
from .base import KVNeed, Mixer, PartSpec, TensorDecl, make_part, register_part


def _padded(n: int) -> int:
    return -(-n // 8) * 8


class SigmoidAttention(Mixer):
    KIND = "sigmoid_attention"

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, softcap: float,
                 eps: float, rot: dict, dtype=torch.float32, device="cuda"):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads cannot share {kv_heads} key/value heads")
        if rot["dims"] > dim:
            raise ValueError(f"{rot['dims']} rotated dimensions do not fit a head of {dim}")
        if not (1 <= dim <= 256 and 1 <= vdim <= 256):
            raise ValueError(f"head sizes {dim} / {vdim}: the attention kernels take 1 to 256")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.scale, self.softcap, self.eps, self.dtype = float(scale), float(softcap), float(eps), dtype
        self.rotary = make_part(PartSpec("rotary", {"dims": rot["dims"], "base": rot["base"], "layout": "halves"}),
                                dtype, device)
        self.q_width, self.k_width, self.v_width = heads * dim, kv_heads * dim, kv_heads * vdim
        self.in_weight = self.in_bias = None

    def tensors(self):
        d = self.width
        return {"q_weight": TensorDecl((self.q_width, d), "matrix"), "q_bias": TensorDecl((self.q_width,), "vector"),
                "k_weight": TensorDecl((self.k_width, d), "matrix"), "k_bias": TensorDecl((self.k_width,), "vector"),
                "v_weight": TensorDecl((self.v_width, d), "matrix"), "v_bias": TensorDecl((self.v_width,), "vector"),
                "q_norm": TensorDecl((self.q_width,), "vector"), "k_norm": TensorDecl((self.k_width,), "vector"),
                "head_bias": TensorDecl((self.heads,), "vector"),
                "out_weight": TensorDecl((d, self.heads * self.vdim), "matrix")}

    def bind(self, tensors):
        """The three projections of the input become one product (q | k | v, rows padded to a multiple of 8)."""
        super().bind(tensors)
        a, b, c = self.q_width, self.q_width + self.k_width, self.q_width + self.k_width + self.v_width
        fused = torch.zeros((_padded(c), self.width), dtype=self.q_weight.dtype, device=self.q_weight.device)
        fused[:a], fused[a:b], fused[b:c] = self.q_weight, self.k_weight, self.v_weight
        bias = torch.zeros((fused.shape[0],), dtype=torch.float32, device=fused.device)
        bias[:a], bias[a:b], bias[b:c] = self.q_bias, self.k_bias, self.v_bias
        self.in_weight, self.in_bias = fused, bias
        self.q_weight, self.k_weight, self.v_weight = fused[:a], fused[a:b], fused[b:c]

    def cache_need(self):
        return KVNeed(kv_heads=self.kv_heads, head_dim=self.dim, window=None, value_heads=self.kv_heads, value_dim=self.vdim)

    def forward(self, h, residual, ctx, cache):
        """residual + mix(h); with ``residual`` None the mixer's output alone, float32 [T, width]."""
        kpages, vpages = ctx.cache.kv_layer(cache.group, cache.layer)
        table = ctx.tables[cache.group]
        proj = ops.linear(h, self.in_weight, self.in_bias, out_dtype=torch.float32)
        q = ops.qk_norm_rotary(proj, kpages, vpages, self.q_norm, self.k_norm, self.rotary.freq, self.rotary.dims, ctx,
                               table, self.heads, self.eps, cache.writes, self.dtype)
        o = ops.sigmoid_attention(q, kpages, vpages, table, ctx, self.heads, self.scale, self.softcap, self.head_bias)
        return ops.linear(o, self.out_weight, None, residual=residual, out_dtype=torch.float32, out=residual)


register_part(SigmoidAttention.KIND, SigmoidAttention)
