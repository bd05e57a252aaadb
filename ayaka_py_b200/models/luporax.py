"""Luporax as data: which parts, with which constants, bound to which tensors.

A layer is a ``post_norm`` arrangement: the mixer reads the residual stream itself after a
token shift (each channel blended with the previous token's), the feed-forward reads the
stream as it is, and an RMS norm on each sublayer's output carries the residual multiplier:
x += m norm1(mixer(shift(x))); x += m norm2(ff(x)).  The mixer is a sigmoid attention, a
real-gated linear recurrent unit or a minGRU, as the layer's ``type`` says; the feed-forward
is a routed mixture of experts with a gated shared expert, or absent.  An entry of ``layers``
with ``weights_of`` is one more run of an earlier layer's parts with a cache of its own: the
run order names that layer twice.  Layer i's tensors start with ``l<i>.``: ``shift norm1
norm2`` and ``mix.*`` / ``mlp.*``; the model's own are ``embed`` (also the head, times
``logit_scale``) and ``final.norm``.  Norm weights are stored around zero.  Linear weights are
[out, in]."""

from __future__ import annotations

import math

from ..config.model import LuporaxConfig
from ..parts.base import Init, LayerSpec, ModelSpec, PartSpec, RunStep, Source
from ..registry import Architecture, register_architecture

_ZERO_GAMMA = Init(std=0.1)
_BIAS = Init(std=0.3)


def luporax_spec(config: LuporaxConfig) -> ModelSpec:
    d, eps, mult = config.width, float(config.norm["eps"]), float(config.residual_mult)

    def matrix(name: str, fan_in: int, gain: float = 1.0) -> Source:
        return Source(name, init=Init(std=gain / math.sqrt(fan_in)))

    def norm(name: str, out_scale: float = 1.0) -> PartSpec:
        return PartSpec("rmsnorm", {"width": d, "eps": eps, "out_scale": out_scale, "offset": 1.0},
                        {"weight": Source(name, init=_ZERO_GAMMA)})

    layers, index_of = [], {}
    for i, layer in enumerate(config.layers):
        if layer.get("weights_of") is not None:
            continue
        index_of[i] = len(layers)
        p, mx = f"l{i}.", layer["mixer"]
        if layer["type"] == "mingru":
            W = mx["width"]
            mixer = PartSpec("mingru", {"width": d, "inner": W},
                             {"z_weight": matrix(p + "mix.z", d), "z_bias": Source(p + "mix.z.b", init=_BIAS),
                              "x_weight": matrix(p + "mix.x", d), "x_bias": Source(p + "mix.x.b", init=_BIAS),
                              "g_weight": matrix(p + "mix.g", d), "out_weight": matrix(p + "mix.o", W)})
        elif layer["type"] == "rglru":
            W, B = mx["width"], mx["blocks"]
            mixer = PartSpec("rglru", {"width": d, "inner": W, "blocks": B, "taps": mx["conv"]},
                             {"y_weight": matrix(p + "mix.y", d), "y_bias": Source(p + "mix.y.b", init=_BIAS),
                              "x_weight": matrix(p + "mix.x", d), "x_bias": Source(p + "mix.x.b", init=_BIAS),
                              "conv_weight": Source(p + "mix.conv", init=Init(std=0.4)),
                              "conv_bias": Source(p + "mix.conv.b", init=_BIAS),
                              "ra_weight": matrix(p + "mix.ra", W // B), "ra_bias": Source(p + "mix.ra.b", init=_BIAS),
                              "ri_weight": matrix(p + "mix.ri", W // B), "ri_bias": Source(p + "mix.ri.b", init=_BIAS),
                              "lam": Source(p + "mix.lam", init=Init(std=1.0, mean=-2.0)),
                              "out_weight": matrix(p + "mix.o", W)})
        else:
            H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            mixer = PartSpec("sigmoid_attention",
                             {"width": d, "heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": float(mx["scale"]),
                              "softcap": float(mx["softcap"]), "eps": eps, "rot": dict(mx["rot"])},
                             {"q_weight": matrix(p + "mix.q", d), "q_bias": Source(p + "mix.q.b", init=_BIAS),
                              "k_weight": matrix(p + "mix.k", d), "k_bias": Source(p + "mix.k.b", init=_BIAS),
                              "v_weight": matrix(p + "mix.v", d), "v_bias": Source(p + "mix.v.b", init=_BIAS),
                              "q_norm": Source(p + "mix.q.norm", init=Init(std=0.1, mean=1.0)),
                              "k_norm": Source(p + "mix.k.norm", init=Init(std=0.1, mean=1.0)),
                              "head_bias": Source(p + "mix.pb", init=Init(std=0.5, mean=-2.0)),
                              "out_weight": matrix(p + "mix.o", H * Dv)})
        parts = [("shift", PartSpec("token_shift", {"width": d}, {"weight": Source(p + "shift", init=Init(std=0.25, mean=0.5))})),
                 ("mixer", mixer), ("norm1", norm(p + "norm1", mult))]
        mlp = layer.get("mlp")
        if mlp is None:
            layers.append(LayerSpec(tuple(parts), "post_norm_mixer_only"))
            continue
        E, ff, sf = mlp["router"]["experts"], mlp["expert"]["ff"], mlp["shared"]["ff"]
        sources = {"router_weight": matrix(p + "mlp.router", d, 2.0),
                   "shared_gate": matrix(p + "mlp.shared.gate", d), "shared_up": matrix(p + "mlp.shared.up", d),
                   "shared_down": matrix(p + "mlp.shared.down", sf), "shared_mix": matrix(p + "mlp.shared.sg", d)}
        for e in range(E):
            sources[f"gate_{e}"] = matrix(f"{p}mlp.e{e}.gate", d)
            sources[f"up_{e}"] = matrix(f"{p}mlp.e{e}.up", d)
            sources[f"down_{e}"] = matrix(f"{p}mlp.e{e}.down", ff)
        ffn = PartSpec("moe", {"width": d, "experts": E, "top": mlp["router"]["top"], "inner": ff,
                               "limit": float(mlp["expert"]["limit"]), "shared_inner": sf,
                               "shared_limit": float(mlp["shared"]["limit"])}, sources)
        parts += [("ffn", ffn), ("norm2", norm(p + "norm2", mult))]
        layers.append(LayerSpec(tuple(parts), "post_norm"))

    order = tuple(RunStep(index_of[layer.get("weights_of", i) if layer.get("weights_of") is not None else i])
                  for i, layer in enumerate(config.layers))
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=d, max_positions=None,
        embedding=PartSpec("token_embedding", {"vocab": config.vocab, "width": d}, {"weight": Source("embed", init=Init(std=0.5))}),
        position=PartSpec("no_positions", {}, {}),
        layers=tuple(layers), order=order,
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab": config.vocab, "width": d, "scale": float(config.logit_scale)},
                      {"weight": Source("embed", init=Init(std=0.5))}))


register_architecture(Architecture(
    name="Luporax", model_type="luporax", config_class=LuporaxConfig, build_spec=luporax_spec))
