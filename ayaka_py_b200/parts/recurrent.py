"""Gated linear recurrences over channels: S_t = a_t S_(t-1) + b_t element by element, with
gates that are functions of the current token only.  The state S (float32) starts at zero and
lives in the request's state slot; gates, decays, state and sums are 32-bit
(``csrc/recurrent.cu``).

``MinGRU``: z = sigmoid(W_z h + b_z), u = W_x h + b_x, candidate c = u + 1/2 where u >= 0 and
sigmoid(u) below; a = 1 - z, b = z c; the output is W_o (S silu(W_g h)).

``RGLRU`` (the recurrent block of Griffin): two branches of ``inner`` channels,
y = gelu_tanh(W_y h + b_y) and u = conv(W_x h + b_x), a causal convolution per channel with a
bias.  u is cut into ``blocks`` equal parts; in each, r = sigmoid(A_r u + b_r) and
i = sigmoid(A_i u + b_i) with square matrices.  a = exp(-c r softplus(lam)) with c = 8,
b = sqrt(1 - a^2) i u; the output is W_o (S y).  The convolution's last taps - 1 inputs are
state too: the slot holds [taps, inner], row 0 the recurrence, the rest the inputs, oldest first."""

from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorDecl, register_part


def _padded(n: int) -> int:
    return -(-n // 8) * 8


class MinGRU(Mixer):
    KIND = "mingru"

    def __init__(self, width: int, inner: int, dtype=torch.float32, device="cuda"):
        self.width, self.inner, self.dtype = width, inner, dtype
        self.in_weight = self.in_bias = None

    def tensors(self):
        W, d = self.inner, self.width
        return {"z_weight": TensorDecl((W, d), "matrix"), "z_bias": TensorDecl((W,), "vector"),
                "x_weight": TensorDecl((W, d), "matrix"), "x_bias": TensorDecl((W,), "vector"),
                "g_weight": TensorDecl((W, d), "matrix"), "out_weight": TensorDecl((d, W), "matrix")}

    def bind(self, tensors):
        """The three projections of the input become one product (z | x | g, rows padded to a multiple of 8)."""
        super().bind(tensors)
        W = self.inner
        fused = torch.zeros((_padded(3 * W), self.width), dtype=self.z_weight.dtype, device=self.z_weight.device)
        fused[:W], fused[W:2 * W], fused[2 * W:3 * W] = self.z_weight, self.x_weight, self.g_weight
        bias = torch.zeros((fused.shape[0],), dtype=torch.float32, device=fused.device)
        bias[:W], bias[W:2 * W] = self.z_bias, self.x_bias
        self.in_weight, self.in_bias = fused, bias
        self.z_weight, self.x_weight, self.g_weight = fused[:W], fused[W:2 * W], fused[2 * W:3 * W]

    def cache_need(self):
        return StateNeed((self.inner,), torch.float32)

    def forward(self, h, residual, ctx, cache):
        """residual + mix(h); with ``residual`` None the mixer's output alone, float32 [T, width]."""
        state = ctx.cache.state_layer(cache.group, cache.layer)
        proj = ops.linear(h, self.in_weight, self.in_bias, out_dtype=torch.float32)
        o = ops.mingru_scan(proj, state, ctx, self.inner, self.dtype)
        return ops.linear(o, self.out_weight, None, residual=residual, out_dtype=torch.float32, out=residual)


class RGLRU(Mixer):
    KIND = "rglru"
    DECAY = 8.0

    def __init__(self, width: int, inner: int, blocks: int, taps: int, dtype=torch.float32, device="cuda"):
        if inner % blocks:
            raise ValueError(f"{inner} channels are not {blocks} equal blocks")
        if not 1 <= taps <= 16:
            raise ValueError(f"a convolution of {taps} taps: the kernels hold 1 to 16")
        self.width, self.inner, self.blocks, self.taps, self.dtype = width, inner, blocks, taps, dtype
        self.in_weight = self.in_bias = None

    def tensors(self):
        W, d, B = self.inner, self.width, self.blocks
        return {"y_weight": TensorDecl((W, d), "matrix"), "y_bias": TensorDecl((W,), "vector"),
                "x_weight": TensorDecl((W, d), "matrix"), "x_bias": TensorDecl((W,), "vector"),
                "conv_weight": TensorDecl((W, self.taps), "vector"), "conv_bias": TensorDecl((W,), "vector"),
                "ra_weight": TensorDecl((B, W // B, W // B), "matrix"), "ra_bias": TensorDecl((B, W // B), "vector"),
                "ri_weight": TensorDecl((B, W // B, W // B), "matrix"), "ri_bias": TensorDecl((B, W // B), "vector"),
                "lam": TensorDecl((W,), "vector"), "out_weight": TensorDecl((d, W), "matrix")}

    def bind(self, tensors):
        """The two projections of the input become one product (y | x); the two gate matrices of a
        block lie one after the other (r | i), for one per-block product; the taps are kept tap-major."""
        super().bind(tensors)
        W, B = self.inner, self.blocks
        fused = torch.zeros((_padded(2 * W), self.width), dtype=self.y_weight.dtype, device=self.y_weight.device)
        fused[:W], fused[W:2 * W] = self.y_weight, self.x_weight
        bias = torch.zeros((fused.shape[0],), dtype=torch.float32, device=fused.device)
        bias[:W], bias[W:2 * W] = self.y_bias, self.x_bias
        self.in_weight, self.in_bias = fused, bias
        self.y_weight, self.x_weight = fused[:W], fused[W:2 * W]
        self.gate_weight = torch.cat([self.ra_weight, self.ri_weight], dim=1).contiguous()        # [B, 2 bs, bs]
        self.gate_bias = torch.cat([self.ra_bias, self.ri_bias], dim=1).contiguous()              # [B, 2 bs]
        self.conv_taps = self.conv_weight.t().contiguous()                                        # [taps, W]

    def cache_need(self):
        return StateNeed((self.taps, self.inner), torch.float32)

    def forward(self, h, residual, ctx, cache):
        """residual + mix(h); with ``residual`` None the mixer's output alone, float32 [T, width]."""
        state = ctx.cache.state_layer(cache.group, cache.layer)            # [slots, taps, W]
        T, W, B = h.shape[0], self.inner, self.blocks
        proj = ops.linear(h, self.in_weight, self.in_bias, out_dtype=torch.float32)          # [T, y | x]
        u = ops.causal_conv(proj[:, W:2 * W], self.conv_taps, self.conv_bias, state, ctx)
        gates = torch.empty((T, B, 2 * (W // B)), dtype=torch.float32, device=h.device)
        ops.head_matmul(u.view(T, B, W // B), self.gate_weight, gates)
        o = ops.rglru_scan(proj, u, gates, self.gate_bias, self.lam, state, ctx, W, B, self.DECAY, self.dtype)
        return ops.linear(o, self.out_weight, None, residual=residual, out_dtype=torch.float32, out=residual)


register_part(MinGRU.KIND, MinGRU)
register_part(RGLRU.KIND, RGLRU)
