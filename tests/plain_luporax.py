"""Luporax in plain NumPy, one function per mechanism, a token at a time where the design has
a recurrence.  Slow and simple on purpose: it shares no code with the package and is what the
kernels are compared with.  Everything runs in the dtype of the tensors it is given (float64
in the tests).

Notation: x is the residual stream [T, d]; W are [out, in] and applied as W @ x."""

from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


# ----------------------------------------------------------- small functions --

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight lies around zero."""
    return unit_rms(x, eps) * (1.0 + w)


# -------------------------------------------------------------- token shift --

def token_shift(x, mu):
    """h_t = x_t + (x_(t-1) - x_t) * mu, with x_(-1) = 0."""
    prev = np.concatenate([np.zeros_like(x[:1]), x[:-1]], axis=0)
    return x + (prev - x) * mu


# -------------------------------------------------------------------- mixers --

def mingru(h, t, p, mx):
    z = sigmoid(h @ t[p + "z"].T + t[p + "z.b"])
    u = h @ t[p + "x"].T + t[p + "x.b"]
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    gate = h @ t[p + "g"].T
    gate = gate * sigmoid(gate)
    S = np.zeros(mx["width"], dtype=h.dtype)
    out = np.zeros((h.shape[0], mx["width"]), dtype=h.dtype)
    for i in range(h.shape[0]):
        S = (1.0 - z[i]) * S + z[i] * cand[i]
        out[i] = S * gate[i]
    return out @ t[p + "o"].T


def causal_conv(v, w, b):
    """v [T, C]; w [C, taps], the last column multiplies the current token; zeros before the start."""
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, v.shape[1]), dtype=v.dtype), v], axis=0)
    out = np.zeros_like(v)
    for j in range(taps):
        out += padded[j:j + v.shape[0]] * w[:, j]
    return out + b


def rglru(h, t, p, mx):
    W, B = mx["width"], mx["blocks"]
    y = gelu_tanh(h @ t[p + "y"].T + t[p + "y.b"])
    u = causal_conv(h @ t[p + "x"].T + t[p + "x.b"], t[p + "conv"], t[p + "conv.b"])
    ub = u.reshape(-1, B, W // B)
    r = sigmoid(np.einsum("boi,tbi->tbo", t[p + "ra"], ub) + t[p + "ra.b"]).reshape(-1, W)
    g = sigmoid(np.einsum("boi,tbi->tbo", t[p + "ri"], ub) + t[p + "ri.b"]).reshape(-1, W)
    a = np.exp(-8.0 * r * softplus(t[p + "lam"]))
    S = np.zeros(W, dtype=h.dtype)
    out = np.zeros((h.shape[0], W), dtype=h.dtype)
    for i in range(h.shape[0]):
        S = a[i] * S + np.sqrt(1.0 - a[i] ** 2) * g[i] * u[i]
        out[i] = S * y[i]
    return out @ t[p + "o"].T


def rotate_half(v, positions, dims, base):
    """v [T, heads, dim]: dimension i pairs with i + dims/2 on the first ``dims`` dimensions."""
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = positions[:, None].astype(np.float64) * freq[None, :]
    c, s = np.cos(ang)[:, None, :].astype(v.dtype), np.sin(ang)[:, None, :].astype(v.dtype)
    out = v.copy()
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def sigmoid_attention(h, t, p, mx, eps, pos0=0):
    T = h.shape[0]
    H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = h @ t[p + "q"].T + t[p + "q.b"]
    k = h @ t[p + "k"].T + t[p + "k.b"]
    v = (h @ t[p + "v"].T + t[p + "v.b"]).reshape(T, G, Dv)
    q = (unit_rms(q, eps) * t[p + "q.norm"]).reshape(T, H, D)
    k = (unit_rms(k, eps) * t[p + "k.norm"]).reshape(T, G, D)
    positions = pos0 + np.arange(T)
    q = rotate_half(q, positions, mx["rot"]["dims"], mx["rot"]["base"])
    k = rotate_half(k, positions, mx["rot"]["dims"], mx["rot"]["base"])
    cap = mx["softcap"]
    out = np.zeros((T, H, Dv), dtype=h.dtype)
    visible = np.tril(np.ones((T, T), dtype=bool))
    for head in range(H):
        g = head // (H // G)
        score = (q[:, head] @ k[:, g].T) * mx["scale"]
        score = cap * np.tanh(score / cap)
        weight = np.where(visible, sigmoid(score + t[p + "pb"][head]), 0.0)
        out[:, head] = weight @ v[:, g]
    return out.reshape(T, H * Dv) @ t[p + "o"].T


MIXERS = {"mingru": mingru, "rglru": rglru}


# -------------------------------------------------------------- feed-forward --

def expert(h, t, p, limit):
    g = np.minimum(h @ t[p + "gate"].T, limit)
    u = np.clip(h @ t[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ t[p + "down"].T


def moe(h, t, p, mlp, margins=None):
    """``margins``: a list that receives, per row, how far the last chosen logit lies above the first one
    left out, as a fraction of the row's largest logit (a small value: rounding may turn the choice)."""
    E, K = mlp["router"]["experts"], mlp["router"]["top"]
    logits = h @ t[p + "router"].T
    if margins is not None and K < E:
        ranked = -np.sort(-logits, axis=1)
        margins.append((ranked[:, K - 1] - ranked[:, K]) / np.abs(logits).max(axis=1))
    out = np.zeros_like(h)
    for i in range(h.shape[0]):
        order = np.argsort(-logits[i], kind="stable")[:K]
        w = np.exp(logits[i, order] - logits[i, order].max())
        w /= w.sum()
        for e, we in zip(order, w):
            out[i] += we * expert(h[i:i + 1], t, f"{p}e{int(e)}.", mlp["expert"]["limit"])[0]
    shared = expert(h, t, p + "shared.", mlp["shared"]["limit"])
    return out + shared * sigmoid(h @ t[p + "shared.sg"].T)


# --------------------------------------------------------------------- model --

def forward(cfg, t, tokens, layers_out=None, margins=None):
    """Logits [T, vocab] of one sequence from position 0.  ``layers_out``: a list that
    receives the residual stream after every layer run; ``margins``: see ``moe``."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = t["embed"][np.asarray(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        h = token_shift(x, t[p + "shift"])
        if layer["type"] == "attention":
            y = sigmoid_attention(h, t, p + "mix.", layer["mixer"], eps)
        else:
            y = MIXERS[layer["type"]](h, t, p + "mix.", layer["mixer"])
        x = x + m * norm_one_plus(y, t[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + m * norm_one_plus(moe(x, t, p + "mlp.", layer["mlp"], margins), t[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return (norm_one_plus(x, t["final.norm"], eps) @ t["embed"].T) * cfg["logit_scale"]


# ------------------------------------------------- tensors, files, configs --

def tensor_shapes(cfg):
    d, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "final.norm": (cfg["width"],)}
    for i, layer in enumerate(cfg["layers"]):
        if "weights_of" in layer:
            continue
        p, mx = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (d,)
        out[p + "shift"] = (d,)
        if layer["type"] == "mingru":
            W = mx["width"]
            out.update({p + "mix.z": (W, d), p + "mix.z.b": (W,), p + "mix.x": (W, d), p + "mix.x.b": (W,),
                        p + "mix.g": (W, d), p + "mix.o": (d, W)})
        elif layer["type"] == "rglru":
            W, B = mx["width"], mx["blocks"]
            out.update({p + "mix.y": (W, d), p + "mix.y.b": (W,), p + "mix.x": (W, d), p + "mix.x.b": (W,),
                        p + "mix.conv": (W, mx["conv"]), p + "mix.conv.b": (W,),
                        p + "mix.ra": (B, W // B, W // B), p + "mix.ra.b": (B, W // B),
                        p + "mix.ri": (B, W // B, W // B), p + "mix.ri.b": (B, W // B),
                        p + "mix.lam": (W,), p + "mix.o": (d, W)})
        else:
            H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            out.update({p + "mix.q": (H * D, d), p + "mix.q.b": (H * D,), p + "mix.k": (G * D, d), p + "mix.k.b": (G * D,),
                        p + "mix.v": (G * Dv, d), p + "mix.v.b": (G * Dv,), p + "mix.q.norm": (H * D,),
                        p + "mix.k.norm": (G * D,), p + "mix.pb": (H,), p + "mix.o": (d, H * Dv)})
        mlp = layer.get("mlp")
        if mlp is not None:
            out[p + "norm2"] = (d,)
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                out.update({f"{p}mlp.e{e}.gate": (ff, d), f"{p}mlp.e{e}.up": (ff, d), f"{p}mlp.e{e}.down": (d, ff)})
            out[p + "mlp.router"] = (mlp["router"]["experts"], d)
            sf = mlp["shared"]["ff"]
            out.update({p + "mlp.shared.gate": (sf, d), p + "mlp.shared.up": (sf, d), p + "mlp.shared.down": (d, sf),
                        p + "mlp.shared.sg": (1, d)})
    return out


def round_bf16(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return (u.astype(np.uint32) << 16).view(np.float32).reshape(a.shape)


def random_tensors(cfg, seed, gain=1.0):
    """Every tensor as float32 values that bfloat16 holds exactly."""
    rs = np.random.RandomState(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        g = rs.standard_normal(shape).astype(np.float32)
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            w = 0.5 * g
        elif last in ("norm1", "norm2") or name == "final.norm":
            w = 0.1 * g
        elif last == "shift":
            w = 0.5 + 0.25 * g
        elif name.endswith(".q.norm") or name.endswith(".k.norm"):
            w = 1.0 + 0.1 * g
        elif last == "lam":
            w = -2.0 + 1.0 * g
        elif last == "pb":
            w = -2.0 + 0.5 * g
        elif last == "b":
            w = 0.3 * g
        elif last == "conv":
            w = 0.4 * g
        elif last == "router":
            w = 2.0 * g / np.sqrt(shape[-1])
        else:
            w = gain * g / np.sqrt(shape[-1])
        out[name] = round_bf16(w.astype(np.float32))
    return out


def write_safetensors(path, tensors):
    """Floats as BF16 (the values are exact in it)."""
    header, chunks, off = {}, [], 0
    for name, arr in tensors.items():
        raw = (np.ascontiguousarray(arr, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        chunks.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for c in chunks:
            f.write(c)


def write_folder(folder, cfg, tensors):
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


def greedy_generate(cfg, t, prompt, n):
    """n tokens, each the arg max of the last position's logits (the whole sequence is run again every time)."""
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(np.argmax(forward(cfg, t, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
