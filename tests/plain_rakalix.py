"""A plain, slow Rakalix for tests: whole sequences, no cache, NumPy only.

Rakalix is a decoder-only model whose layers carry either a latent attention
(keys and values are up-projections of one small normed latent per token, plus
one rotated key part that all heads share) or an HGRN2 recurrence (a gated
linear attention whose forget gate also says what is written), each followed by
an optional feed-forward with the PolyNorm activation.  Every sublayer reads
RMS-normed input that first passes a short causal convolution over time, and
its output is RMS-normed again before a scaled residual sum.

One function per mechanism; nothing here is shared with the engine.  Pass
float64 tensors for the strict oracle.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np


# ------------------------------------------------------------------ small ops --

def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def time_conv(h, w):
    """h + conv(h): w is [channels, taps]; tap j multiplies the input that lies
    taps - 1 - j steps back; inputs before the sequence's start are zero."""
    T, taps = h.shape[0], w.shape[1]
    out = h.copy()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def poly_norm(z, coeff, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e, N = division by the row's root mean square."""
    a, b, c, e = (float(v) for v in coeff)
    return a * rms_unit(z, eps) + b * rms_unit(z * z, eps) + c * rms_unit(z * z * z, eps) + e


# ------------------------------------------------------------------ rotation --

def rotary_frequencies(dims, base, scaling=None):
    """(frequency per pair, factor on cos and sin).  With ``scaling`` (factor,
    original, fast, slow) the low frequencies are divided by the factor, blended
    by a ramp over the pair index, and cos and sin grow by 0.1 ln(factor) + 1."""
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)], dtype=np.float64)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, dims, base, scaling=None):
    """x: [T, ..., D]; the first ``dims`` entries of the last axis are turned in
    neighbouring pairs (2i, 2i+1) by the angle position * frequency_i."""
    f, gain = rotary_frequencies(dims, base, scaling)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]          # [T, dims/2]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (dims // 2,)
    cos, sin = (np.cos(angle) * gain).reshape(shape), (np.sin(angle) * gain).reshape(shape)
    out = x.copy()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# -------------------------------------------------------------------- mixers --

def latent_attention(h, w, p, eps, positions=None):
    """w: the mixer's tensors by short name; p: its sizes and constants."""
    T = h.shape[0]
    H, dim, rot_dim, vdim, rank = p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]
    rot = p["rot"]
    positions = np.arange(T) if positions is None else positions
    q = (h @ w["q"].T).reshape(T, H, dim + rot_dim)
    q_plain, q_turn = q[..., :dim], rotate(q[..., dim:], positions, rot["dims"], rot["base"], rot.get("scaling"))
    down = h @ w["dkv"].T
    latent = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    k_turn = rotate(down[:, rank:], positions, rot["dims"], rot["base"], rot.get("scaling"))      # [T, rot_dim], all heads
    k_plain = (latent @ w["uk"].T).reshape(T, H, dim)
    value = (latent @ w["uv"].T).reshape(T, H, vdim)
    gate = sigmoid(h @ w["g"].T)                                                                # [T, H]
    out = np.zeros((T, H, vdim), dtype=h.dtype)
    for head in range(H):
        s = (q_plain[:, head] @ k_plain[:, head].T + q_turn[:, head] @ k_turn.T) * p["scale"]
        s = np.where(np.tril(np.ones((T, T), dtype=bool)), s, -np.inf)
        s = np.exp(s - s.max(axis=-1, keepdims=True))
        out[:, head] = (s / s.sum(axis=-1, keepdims=True)) @ value[:, head] * gate[:, head:head + 1]
    return out.reshape(T, H * vdim) @ w["o"].T


def hgrn2(h, w, p, eps, state=None):
    """Per head S <- diag(f) S + (1 - f) v^T, o = S^T q.  Returns (output, last state)."""
    T = h.shape[0]
    H, dim, vdim = p["heads"], p["dim"], p["vdim"]
    q = silu(h @ w["q"].T).reshape(T, H, dim)
    lower = w["lower"]
    f = (lower + (1.0 - lower) * sigmoid(h @ w["f"].T + w["f.b"])).reshape(T, H, dim)
    v = (h @ w["v"].T).reshape(T, H, vdim)
    S = np.zeros((H, dim, vdim), dtype=h.dtype) if state is None else state.copy()
    o = np.zeros((T, H, vdim), dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, w["norm"], eps)
    return o.reshape(T, H * vdim) @ w["o"].T, S


def feed_forward(h, w, eps):
    return poly_norm(h @ w["up"].T, w["act"], eps) @ w["down"].T


# --------------------------------------------------------------------- model --

def layer_tensors(tensors, i, part):
    prefix = f"l{i}.{part}."
    return {name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)}


def layer(x, tensors, config, i, positions=None):
    spec, eps, m = config["layers"][i], config["norm"]["eps"], config["residual_mult"]
    t = lambda name: tensors[f"l{i}.{name}"]
    h = time_conv(rms_norm(x, t("norm1"), eps), t("canon1"))
    if spec["type"] == "latent_attention":
        y = latent_attention(h, layer_tensors(tensors, i, "mix"), spec["mixer"], eps, positions)
    elif spec["type"] == "hgrn2":
        y, _ = hgrn2(h, layer_tensors(tensors, i, "mix"), spec["mixer"], eps)
    else:
        raise ValueError(spec["type"])
    x = x + m * rms_norm(y, t("norm1b"), eps)
    if spec.get("mlp") is not None:
        h = time_conv(rms_norm(x, t("norm2"), eps), t("canon2"))
        x = x + m * rms_norm(feed_forward(h, layer_tensors(tensors, i, "mlp"), eps), t("norm2b"), eps)
    return x


def forward(config, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer)."""
    x = tensors["embed"][np.asarray(tokens)] * config["embedding"]["scale"]
    after = []
    for i in range(len(config["layers"])):
        x = layer(x, tensors, config, i)
        after.append(x)
    logits = rms_norm(x, tensors["final.norm"], config["norm"]["eps"]) @ tensors["head"].T
    return (logits, np.stack(after)) if return_layers else logits


def greedy_generate(config, tensors, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward(config, tensors, tokens)[-1])))
    return tokens[len(prompt):]


# --------------------------------------------------- random models for tests --

def tensor_shapes(config):
    d, V, taps = config["width"], config["vocab"], config["canon"]["taps"]
    shapes = {"embed": (V, d), "final.norm": (d,), "head": (V, d)}
    for i, spec in enumerate(config["layers"]):
        p, mx = f"l{i}.", spec["mixer"]
        shapes.update({p + "norm1": (d,), p + "norm1b": (d,), p + "canon1": (d, taps)})
        H, dim, vdim = mx["heads"], mx["dim"], mx["vdim"]
        if spec["type"] == "hgrn2":
            shapes.update({p + "mix.q": (H * dim, d), p + "mix.f": (H * dim, d), p + "mix.f.b": (H * dim,),
                           p + "mix.lower": (H * dim,), p + "mix.v": (H * vdim, d), p + "mix.norm": (vdim,),
                           p + "mix.o": (d, H * vdim)})
        else:
            rank, rot_dim = mx["kv_rank"], mx["rot_dim"]
            shapes.update({p + "mix.q": (H * (dim + rot_dim), d), p + "mix.dkv": (rank + rot_dim, d),
                           p + "mix.dkv.norm": (rank,), p + "mix.uk": (H * dim, rank), p + "mix.uv": (H * vdim, rank),
                           p + "mix.g": (H, d), p + "mix.o": (d, H * vdim)})
        if spec.get("mlp") is not None:
            ff = spec["mlp"]["ff"]
            shapes.update({p + "norm2": (d,), p + "norm2b": (d,), p + "canon2": (d, taps),
                           p + "mlp.up": (ff, d), p + "mlp.down": (d, ff), p + "mlp.act": (4,)})
    return shapes


def bf16_round(a):
    """Round float32 values to the nearest bfloat16 (ties to even), kept as float32."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def random_tensors(config, seed):
    """Seeded tensors, bfloat16-exact, as float32: projections ~ N(0, 1/in), norm weights near
    one, gates' lower bounds in (0, 0.9), convolution taps and activation numbers of order one."""
    rs = np.random.RandomState(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith("mix.lower"):
            a = rs.uniform(0.0, 0.9, shape)
        elif name.endswith("mix.f.b"):
            a = rs.randn(*shape) * 0.5 + 1.0
        elif name.endswith("mlp.act"):
            a = np.array([0.6, 0.3, 0.2, 0.05]) + rs.randn(4) * 0.05
        elif last.startswith("canon"):
            a = rs.randn(*shape) * 0.3
        elif len(shape) == 1:
            a = 1.0 + rs.randn(*shape) * 0.1
        elif name == "embed":
            a = rs.randn(*shape) * 0.1
        else:
            a = rs.randn(*shape) / math.sqrt(shape[1])
        out[name] = bf16_round(a.astype(np.float32))
    return out


def write_folder(folder, config, tensors):
    """config.json and model.safetensors (bfloat16), with a writer of this file's own."""
    import struct
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    header, blobs, at = {}, [], 0
    for name, a in tensors.items():
        raw = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))
    return folder
