"""Position encodings.  GPT-2 uses a learned table of absolute positions that
is added to the token embedding; ``NoPositions`` adds nothing; ``Rotary`` turns
pairs of query and key dimensions by an angle that grows with the position."""

from __future__ import annotations

import math

import torch

from .. import ops

from .base import PositionEncoding, TensorDecl, register_part


class LearnedPositions(PositionEncoding):
    KIND = "learned_positions"

    def __init__(self, positions: int, width: int, dtype=torch.float32, device="cuda"):
        self.positions, self.width = positions, width
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.positions, self.width), "matrix")}

    def embedding_table(self):
        return self.weight

    def max_positions(self):
        return self.positions


class NoPositions(PositionEncoding):
    KIND = "no_positions"

    def __init__(self, dtype=torch.float32, device="cuda"):
        pass


class Rotary(PositionEncoding):
    """Rotary positions in the interleaved layout: dimension 2i is paired with 2i + 1, and the pair
    at position p turns by p * f_i, f_i = base^(-2i / dims), on the first ``dims`` dimensions of a
    head (the rest pass).  ``scaling`` = {factor, original, fast, slow} stretches the slow
    frequencies for contexts beyond ``original`` positions: with where(t) = dims ln(original /
    (2 pi t)) / (2 ln base), lo = max(floor(where(fast)), 0), hi = min(ceil(where(slow)), dims - 1)
    and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency becomes
    f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and sin are multiplied by 0.1 ln(factor) + 1.
    Frequencies are computed once on the host in double precision and kept as float32; angles,
    cos and sin are 32-bit on the device.  ``layout`` "halves" pairs dimension i with i + dims/2
    instead (the same frequencies).  No tensors of its own."""

    KIND = "rotary"

    def __init__(self, dims: int, base: float, scaling: dict | None = None, layout: str = "interleaved",
                 dtype=torch.float32, device="cuda"):
        if dims < 2 or dims % 2:
            raise ValueError(f"rotary positions pair dimensions: dims must be even and positive, got {dims}")
        if layout not in ("interleaved", "halves"):
            raise ValueError(f"rotary layout {layout!r}: 'interleaved' or 'halves'")
        self.dims, self.base, self.scaling = dims, float(base), dict(scaling) if scaling else None
        self.halves = layout == "halves"
        freq, self.gain = rotary_frequencies(dims, self.base, self.scaling)
        self.freq = torch.tensor(freq, dtype=torch.float64).to(torch.float32)
        if device != "meta":
            self.freq = self.freq.to(device)

    def rotate(self, x, positions, heads: int, head_stride: int, offset: int = 0) -> None:
        """Turns x[t, head * head_stride + offset + (0 .. dims)) in place."""
        ops.rotary(x, positions, self.freq, self.gain, heads, head_stride, offset, self.dims, self.halves)

    def rotate_qk(self, q, k, heads, kv_heads, head_dim, ctx) -> None:
        self.rotate(q, ctx.positions, heads, head_dim)
        self.rotate(k, ctx.positions, kv_heads, head_dim)


def rotary_frequencies(dims: int, base: float, scaling: dict | None) -> tuple[list[float], float]:
    """(frequency of every pair, factor on cos and sin); see ``Rotary``."""
    half = dims // 2
    freq = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def where(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freq):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


register_part(LearnedPositions.KIND, LearnedPositions)
register_part(Rotary.KIND, Rotary)
register_part(NoPositions.KIND, NoPositions)
