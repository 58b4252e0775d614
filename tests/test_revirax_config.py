"""Revirax's configuration, description and cache needs, without a GPU."""

import copy

import numpy as np
import pytest
import torch

import plain_revirax as pr
from revirax_cases import CONFIGS, tensor_shapes


def _model(cfg):
    from rusty_llama_b200.models.model import Model
    from rusty_llama_b200.parts.base import Runtime
    from rusty_llama_b200.registry import describe_model

    return Model(describe_model(cfg), Runtime.create("cpu", torch.float32))


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_described_model_asks_for_the_checkpoints_tensors(name):
    cfg = CONFIGS[name]()
    got = {k: tuple(v.shape) for k, v in _model(cfg).param_infos().items()}
    assert got == tensor_shapes(cfg)


def test_every_layer_gets_the_storage_its_mixer_asks_for():
    from rusty_llama_b200.cache import Cache
    from rusty_llama_b200.parts.base import KVNeed, StateNeed

    cfg = CONFIGS["a"]()
    model = _model(cfg)
    needs = dict(model.cache_needs())
    assert needs[0] == KVNeed(2, 20, 0, value_dim=12)
    assert needs[1] == StateNeed((3, 24, 40), torch.float32)
    assert needs[2] == (KVNeed(4, 16, 5, value_dim=24), StateNeed((50,), torch.float32))
    assert needs[3] == KVNeed(1, 32, 70, value_dim=8)
    cache = Cache(model.cache_needs(), 64 * 4, 2, torch.float32, "cpu")
    left, right = cache.view(2)
    assert tuple(left.k_pages.shape) == (4, 4, 64, 16) and tuple(left.v_pages.shape) == (4, 4, 64, 24) and left.window == 5
    assert tuple(right.state.shape) == (2, 50)
    assert tuple(cache.view(1).state.shape) == (2, 3, 24, 40)
    assert cache.owns(2) and cache.owns(5) and not cache.owns(6)
    # a slot that is used again reads zero in every state; its window groups give pages back as the window passes
    s = cache.open_sequence()
    cache.view(1).state[s] += 1.0
    right.state[s] += 1.0
    cache.reserve([s], [200])
    cache.commit([s], [200])
    cache.check_consistent()
    assert model.cache_bytes_per_token() == 4 * (2 * 32 + 4 * 40 + 1 * 40 + 1 * 40)
    cache.close_sequence(s)
    assert cache.open_sequence() == s
    assert float(cache.view(1).state[s].abs().max()) == 0.0 and float(cache.view(2)[1].state[s].abs().max()) == 0.0
    cache.check_consistent()


def test_frequency_tables_follow_the_plain_formulas():
    from rusty_llama_b200.config.revirax import ReviraxConfig
    from rusty_llama_b200.config.rope_scaling import inverse_frequencies, magnitude

    for name in CONFIGS:
        raw = CONFIGS[name]()
        cfg = ReviraxConfig.from_json(raw)
        for layer, parsed in zip(raw["layers"], cfg.layers):
            m, pm = (layer["mixer"], parsed.mixer) if layer["type"] == "attention" else (layer["mixer"].get("left"), getattr(parsed.mixer, "left", None))
            if m is None or not m["rot"]["dims"]:
                continue
            f, mag = pr.rotary_table(m["rot"])
            got = inverse_frequencies(pm.rot_dims, pm.rot_base, pm.rot_scaling)
            assert np.abs(got - f).max() <= 1e-6 * f.max()
            assert abs(magnitude(pm.rot_scaling) - mag) < 1e-12


def test_configuration_errors_name_the_place():
    from rusty_llama_b200.errors import ConfigError
    from rusty_llama_b200.registry import describe_model

    base = CONFIGS["a"]()
    for change, text in (
        (lambda c: c["layers"][0].update(type="conv"), "layers[0].type"),
        (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
        (lambda c: c["layers"][0]["mixer"].update(heads=5), "kv_heads"),
        (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=22), "rot.dims"),
        (lambda c: c["layers"][0]["mixer"]["rot"].update(scaling={"factor": 2.0, "original": 8}), "scaling"),
        (lambda c: c["layers"][2]["mlp"].update(kind="moe"), "mlp.kind"),
        (lambda c: c["layers"][2]["mixer"].pop("left_scale"), "left_scale"),
    ):
        cfg = copy.deepcopy(base)
        change(cfg)
        with pytest.raises(ConfigError) as e:
            describe_model(cfg)
        assert text in str(e.value), (text, str(e.value))
