"""Rakalix as data: which parts, with which constants, bound to which tensors.

A layer is a ``sandwich`` arrangement: RMS norm and a short convolution over time in
front of each sublayer, an RMS norm carrying the residual multiplier behind it.  The
mixer is a latent attention or an HGRN2 recurrence, as the layer's ``type`` says; the
feed-forward (PolyNorm activation) may be absent.  Layer i's tensors start with
``l<i>.``: ``norm1 norm1b norm2 norm2b canon1 canon2`` and ``mix.*`` / ``mlp.*``; the
model's own are ``embed``, ``final.norm`` and ``head``.  Linear weights are [out, in]."""

from __future__ import annotations

import math

from ..config.model import RakalixConfig
from ..parts.base import Init, LayerSpec, ModelSpec, PartSpec, RunStep, Source
from ..registry import Architecture, register_architecture

_GAMMA = Init(std=0.05, mean=1.0)


def rakalix_spec(config: RakalixConfig) -> ModelSpec:
    d, eps, taps, mult = config.width, float(config.norm["eps"]), int(config.canon["taps"]), float(config.residual_mult)

    def matrix(name: str, fan_in: int) -> Source:
        return Source(name, init=Init(std=1.0 / math.sqrt(fan_in)))

    def norm(name: str, out_scale: float = 1.0) -> PartSpec:
        return PartSpec("rmsnorm", {"width": d, "eps": eps, "out_scale": out_scale}, {"weight": Source(name, init=_GAMMA)})

    def conv(name: str) -> PartSpec:
        return PartSpec("time_conv", {"width": d, "taps": taps}, {"weight": Source(name, init=Init(std=0.3))})

    layers = []
    for i, layer in enumerate(config.layers):
        p, mx = f"l{i}.", layer["mixer"]
        H, dim, vdim = mx["heads"], mx["dim"], mx["vdim"]
        if layer["type"] == "hgrn2":
            mixer = PartSpec("hgrn2", {"width": d, "heads": H, "dim": dim, "vdim": vdim, "eps": eps},
                             {"q_weight": matrix(p + "mix.q", d), "f_weight": matrix(p + "mix.f", d),
                              "f_bias": Source(p + "mix.f.b", init=Init(std=0.5, mean=1.0)),
                              "lower": Source(p + "mix.lower", init=Init(std=0.1, mean=0.4)),
                              "v_weight": matrix(p + "mix.v", d), "norm": Source(p + "mix.norm", init=_GAMMA),
                              "out_weight": matrix(p + "mix.o", H * vdim)})
        else:
            rank = mx["kv_rank"]
            mixer = PartSpec("latent_attention",
                             {"width": d, "heads": H, "dim": dim, "rot_dim": mx["rot_dim"], "vdim": vdim, "kv_rank": rank,
                              "scale": float(mx["scale"]), "eps": eps, "rot": mx["rot"]},
                             {"q_weight": matrix(p + "mix.q", d), "down_weight": matrix(p + "mix.dkv", d),
                              "down_norm": Source(p + "mix.dkv.norm", init=_GAMMA),
                              "uk_weight": matrix(p + "mix.uk", rank), "uv_weight": matrix(p + "mix.uv", rank),
                              "gate_weight": matrix(p + "mix.g", d), "out_weight": matrix(p + "mix.o", H * vdim)})
        parts = [("norm1", norm(p + "norm1")), ("conv1", conv(p + "canon1")), ("mixer", mixer),
                 ("norm1b", norm(p + "norm1b", mult))]
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            ffn = PartSpec("polynorm_mlp", {"width": d, "inner": ff, "eps": eps},
                           {"up_weight": matrix(p + "mlp.up", d), "down_weight": matrix(p + "mlp.down", ff),
                            "coeff": Source(p + "mlp.act", init=Init(std=0.1, mean=0.3))})
            parts += [("norm2", norm(p + "norm2")), ("conv2", conv(p + "canon2")), ("ffn", ffn),
                      ("norm2b", norm(p + "norm2b", mult))]
            layers.append(LayerSpec(tuple(parts), "sandwich"))
        else:
            layers.append(LayerSpec(tuple(parts), "sandwich_mixer_only"))

    return ModelSpec(
        vocab_size=config.vocab, hidden_size=d, max_positions=None,
        embedding=PartSpec("token_embedding", {"vocab": config.vocab, "width": d, "scale": float(config.embedding["scale"])},
                           {"weight": Source("embed", init=Init(std=0.1))}),
        position=PartSpec("no_positions", {}, {}),
        layers=tuple(layers), order=tuple(RunStep(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab": config.vocab, "width": d}, {"weight": matrix("head", d)}))


def rakalix_normalize_name(name: str, config: RakalixConfig) -> str | None:
    """Tensors of the feed-forward sublayer of a layer that has none are passed over."""
    if name.startswith("l"):
        index, _, rest = name[1:].partition(".")
        if index.isdigit() and int(index) < len(config.layers) and config.layers[int(index)].get("mlp") is None:
            if rest in ("norm2", "norm2b", "canon2") or rest.startswith("mlp."):
                return None
    return name


register_architecture(Architecture(
    name="Rakalix", model_type="rakalix", config_class=RakalixConfig,
    build_spec=rakalix_spec, normalize_name=rakalix_normalize_name))
