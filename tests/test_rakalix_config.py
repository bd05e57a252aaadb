"""Rakalix on the host: configuration, registry, the model as data, cache groups, tensor names."""

import copy

import pytest
import torch

import plain_rakalix as plain

BASE = {"architecture": "Rakalix", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "canon": {"taps": 3},
        "embedding": {"scale": 2.0}, "residual_mult": 0.5,
        "layers": [
            {"type": "hgrn2", "mixer": {"heads": 2, "dim": 12, "vdim": 20}, "mlp": {"kind": "dense", "ff": 64}},
            {"type": "latent_attention", "mlp": None,
             "mixer": {"heads": 3, "dim": 8, "rot_dim": 6, "vdim": 10, "kv_rank": 14, "scale": 0.3,
                       "rot": {"dims": 4, "base": 1000.0, "scaling": None}}},
            {"type": "hgrn2", "mixer": {"heads": 2, "dim": 12, "vdim": 20}, "mlp": None}]}


def build(document, dtype=torch.bfloat16):
    from ayaka_py_b200 import models, parts  # noqa: F401
    from ayaka_py_b200.models.model import Model
    from ayaka_py_b200.registry import architecture_for
    arch = architecture_for(document)
    config = arch.config_class.from_dict(document)
    return arch, config, Model(arch.build_spec(config), dtype, "meta")


def test_registry_takes_the_single_architecture_key_and_round_trips():
    arch, config, _ = build(BASE)
    assert arch.name == "Rakalix"
    again = arch.config_class.from_dict(config.to_dict())
    assert again.to_dict() == config.to_dict() and again.to_dict()["architecture"] == "Rakalix"


def test_tensor_names_and_shapes_follow_the_layers():
    arch, config, model = build(BASE)
    rows = {r.source.name: tuple(r.decl.shape) for r in model.tensor_rows()}
    assert rows == plain.tensor_shapes(BASE)
    # a layer without feed-forward: its closing tensors are passed over if a file has them
    assert arch.normalize_name("l1.norm2", config) is None and arch.normalize_name("l1.mlp.up", config) is None
    assert arch.normalize_name("l0.norm2", config) == "l0.norm2" and arch.normalize_name("l1.norm1b", config) == "l1.norm1b"


def test_cache_groups_pages_for_the_latent_and_slots_for_states():
    from ayaka_py_b200.parts import KVNeed, StateNeed
    _, _, model = build(BASE)
    needs = {type(g.need).__name__: [] for g in model.groups}
    for g in model.groups:
        needs[type(g.need).__name__].append((g.need, g.layers))
    assert needs["KVNeed"] == [(KVNeed(1, 6, None, 1, 14), 1)]
    states = dict(needs["StateNeed"])
    assert states[StateNeed((2, 48), torch.float32)] == 4             # a convolution in front of every sublayer
    assert states[StateNeed((2, 12, 20), torch.float32)] == 2
    assert model.max_positions is None
    assert [b.KIND for b in model.blocks] == ["sandwich", "sandwich_mixer_only", "sandwich_mixer_only"]


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=8), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
    (lambda c: c["norm"].update(eps=0), "norm.eps"),
    (lambda c: c["canon"].update(taps=0), "canon.taps"),
    (lambda c: c.update(layers=[]), "layers"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(scaling={"factor": 2.0}), "scaling"),
])
def test_bad_configurations_are_refused_with_the_key(change, word):
    from ayaka_py_b200.config.model import ConfigError
    document = copy.deepcopy(BASE)
    change(document)
    with pytest.raises(ConfigError, match=word.replace(".", r"\.")):
        build(document)


def test_rotary_frequencies_with_and_without_scaling():
    from ayaka_py_b200.parts.position import rotary_frequencies
    import numpy as np
    for scaling in (None, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0},
                    {"factor": 3.0, "original": 4096, "fast": 32.0, "slow": 1.0}):
        for dims, base in ((4, 100.0), (16, 50000.0), (64, 10000.0)):
            got, gain = rotary_frequencies(dims, base, scaling)
            want, want_gain = plain.rotary_frequencies(dims, base, scaling)
            assert np.allclose(got, want, rtol=1e-12) and abs(gain - want_gain) < 1e-12
    assert rotary_frequencies(8, 10.0, None)[1] == 1.0


def test_random_weights_are_written_and_read_back(tmp_path):
    from ayaka_py_b200.config.model import RakalixConfig
    from ayaka_py_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "m", RakalixConfig.from_dict(BASE), seed=1)
    import plain_gpt2
    tensors = plain_gpt2.read_safetensors(folder / "model.safetensors")
    assert {k: tuple(v.shape) for k, v in tensors.items()} == plain.tensor_shapes(BASE)
    assert abs(float(tensors["l0.norm1"].mean()) - 1.0) < 0.1
