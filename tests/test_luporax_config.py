"""Luporax on the host: configuration, registry, the model as data, run order, cache groups, tensor names."""

import copy

import numpy as np
import pytest
import torch

import plain_luporax as plain

_MOE = {"kind": "moe", "router": {"experts": 6, "top": 2}, "expert": {"ff": 20, "limit": 2.0}, "shared": {"ff": 12, "limit": 1.0}}
_ATT = {"type": "attention", "mlp": _MOE,
        "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 10, "rot": {"dims": 8, "base": 1000.0}, "scale": 0.3, "softcap": 25.0}}
_GRU = {"type": "mingru", "mlp": None, "mixer": {"width": 56}}
_LRU = {"type": "rglru", "mlp": _MOE, "mixer": {"width": 64, "blocks": 4, "conv": 3}}
BASE = {"architecture": "Luporax", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 0.5, "logit_scale": 0.4,
        "layers": [_GRU, _ATT, _LRU, {**_ATT, "weights_of": 1}, {**_GRU, "weights_of": 0}, {**_ATT, "weights_of": 1}]}


def build(document, dtype=torch.bfloat16):
    from ayaka_py_b200 import models, parts  # noqa: F401
    from ayaka_py_b200.models.model import Model
    from ayaka_py_b200.registry import architecture_for
    arch = architecture_for(document)
    config = arch.config_class.from_dict(document)
    return arch, config, Model(arch.build_spec(config), dtype, "meta")


def test_registry_takes_the_single_architecture_key_and_round_trips():
    arch, config, _ = build(BASE)
    assert arch.name == "Luporax"
    again = arch.config_class.from_dict(config.to_dict())
    assert again.to_dict() == config.to_dict() and again.to_dict()["architecture"] == "Luporax"


def test_tensor_names_and_shapes_follow_the_layers_that_have_tensors():
    _, _, model = build(BASE)
    rows = {r.source.name: tuple(r.decl.shape) for r in model.tensor_rows()}
    assert rows == plain.tensor_shapes(BASE)
    assert not any(name.startswith(("l3.", "l4.", "l5.")) for name in rows)
    # the head reads the embedding table
    assert [r.source.name for r in model.tensor_rows() if r.part is model.head] == ["embed"]
    assert model.head.scale == 0.4 and model.final_norm.offset == 1.0


def test_layers_that_run_again_share_parts_and_keep_caches_of_their_own():
    from ayaka_py_b200.parts import KVNeed, StateNeed
    _, _, model = build(BASE)
    assert [s.layer for s in model.spec.order] == [0, 1, 2, 1, 0, 1] and len(model.blocks) == 3
    assert [b.KIND for b in model.blocks] == ["post_norm_mixer_only", "post_norm", "post_norm"]
    layers = {g.need: g.layers for g in model.groups}
    assert layers[KVNeed(2, 12, None, 2, 10)] == 3                       # three runs of the attention layer
    assert layers[StateNeed((48,), torch.float32)] == 6                  # a token shift in every run
    assert layers[StateNeed((56,), torch.float32)] == 2
    assert layers[StateNeed((3, 64), torch.float32)] == 1                # recurrence and two convolution inputs
    mixers = [b["mixer"] for b in model.bindings]
    assert all(b.writes for b in mixers)
    assert [(b.group, b.layer) for b in (mixers[1], mixers[3], mixers[5])] == [(mixers[1].group, 0), (mixers[1].group, 1), (mixers[1].group, 2)]
    assert model.max_positions is None


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads|key/value"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].update(softcap=0), "softcap"),
    (lambda c: c["layers"][2]["mixer"].update(blocks=5), "blocks"),
    (lambda c: c["layers"][2]["mlp"].update(kind="dense"), "mlp.kind"),
    (lambda c: c["layers"][2]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][2]["mlp"]["shared"].pop("limit"), "shared.limit"),
    (lambda c: c["layers"][3].update(weights_of=4), "weights_of"),
    (lambda c: c["layers"][4].update(weights_of=1), "weights_of|another layer"),
    (lambda c: c["norm"].update(eps=0), "norm.eps"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_bad_configurations_are_refused_with_the_key(change, word):
    from ayaka_py_b200.config.model import ConfigError
    document = copy.deepcopy(BASE)
    change(document)
    with pytest.raises(ConfigError, match=word.replace(".", r"\.")):
        build(document)


def test_random_weights_are_written_and_read_back(tmp_path):
    from ayaka_py_b200.config.model import LuporaxConfig
    from ayaka_py_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "m", LuporaxConfig.from_dict(BASE), seed=1)
    import plain_gpt2
    tensors = plain_gpt2.read_safetensors(folder / "model.safetensors")
    assert {k: tuple(v.shape) for k, v in tensors.items()} == plain.tensor_shapes(BASE)
    assert abs(float(np.asarray(tensors["l0.norm1"], dtype=np.float64).mean())) < 0.1     # stored around zero


def test_the_plain_model_does_not_look_ahead():
    """The oracle itself: logits of a prefix equal the logits of the whole at those places."""
    cfg = copy.deepcopy(BASE)
    t = {k: v.astype(np.float64) for k, v in plain.random_tensors(cfg, 5).items()}
    toks = np.random.RandomState(0).randint(0, cfg["vocab"], 24).tolist()
    whole, part = plain.forward(cfg, t, toks), plain.forward(cfg, t, toks[:15])
    assert np.abs(whole[:15] - part).max() < 1e-9
