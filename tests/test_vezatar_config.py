"""Vezatar's configuration, description and plain implementation: what needs no GPU."""

import copy

import numpy as np
import pytest
import torch

import plain_vezatar as pv
from vezatar_cases import CONFIGS, as_float64, random_weights, tensor_shapes


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_description_asks_for_the_checkpoints_tensors(name):
    from rusty_llama_b200.models.model import Model
    from rusty_llama_b200.parts.base import Runtime
    from rusty_llama_b200.registry import describe_model

    cfg = CONFIGS[name]()
    spec = describe_model(cfg)
    assert spec.architecture == "Vezatar" and len(spec.layers) == len(cfg["layers"])
    infos = Model(spec, Runtime.create("cpu", torch.float32)).param_infos()
    assert {k: tuple(v.shape) for k, v in infos.items()} == tensor_shapes(cfg)
    for i, layer in enumerate(cfg["layers"]):
        assert spec.schedule[i].cache_from == layer["mixer"].get("kv_from")
        assert (spec.layers[i].feed_forward is None) == (layer["mlp"] is None)


def test_layers_with_equal_cache_rows_share_a_group():
    from rusty_llama_b200.models.model import Model
    from rusty_llama_b200.parts.base import Runtime
    from rusty_llama_b200.registry import describe_model

    model = Model(describe_model(CONFIGS["a"]()), Runtime.create("cpu", torch.float32))
    needs = model.cache_needs()
    assert [run for run, _ in needs] == [0, 2]  # the layers that read another layer's cache own none
    assert all(not n.values and n.num_kv_heads == 1 and n.head_dim == 56 for _, n in needs)
    cache = model.new_cache(256, 2)
    assert len(cache.kv_groups) == 1 and cache.kv_groups[0].v is None and cache.kv_groups[0].k.shape[0] == 2
    assert model.cache_bytes_per_token() == 2 * 56 * 4


@pytest.mark.parametrize(
    "change, needle",
    [
        (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "does not run before"),
        (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "no cache of its own"),
        (lambda c: c["layers"][1]["mixer"].update(kv_rank=40), "differ"),
        (lambda c: c["layers"][0].update(type="other"), "not a mixer"),
        (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "neither"),
        (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "of 5 experts"),
        (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "at most rot_dim"),
        (lambda c: c["layers"][0]["mixer"].pop("vdim"), "lacks 'vdim'"),
        (lambda c: c.pop("vocab"), "lacks 'vocab'"),
        (lambda c: c["norm"].update(eps=0), "eps"),
    ],
)
def test_bad_configurations_are_named(change, needle):
    from rusty_llama_b200 import ConfigError
    from rusty_llama_b200.registry import describe_model

    cfg = copy.deepcopy(CONFIGS["a"]())
    change(cfg)
    with pytest.raises(ConfigError, match=needle):
        describe_model(cfg)


def test_scaled_frequencies_follow_the_plain_formula():
    from rusty_llama_b200.config.rope_scaling import RopeScaling, inverse_frequencies, magnitude

    for dims, base, sc in ((8, 10000.0, (4.0, 64, 8.0, 2.0)), (64, 1e6, (2.0, 1024, 32.0, 1.0)), (4, 1000.0, (1.5, 32, 4.0, 1.0)), (32, 5e5, (16.0, 4096, 1.0, 1.0))):
        s = RopeScaling(kind="yarn", factor=sc[0], original_max_position_embeddings=sc[1], beta_fast=sc[2], beta_slow=sc[3])
        f, m = pv.yarn_frequencies(dims, base, dict(factor=sc[0], original=sc[1], fast=sc[2], slow=sc[3]))
        got = inverse_frequencies(dims, base, s)
        assert np.abs(got - f).max() <= 1e-7 * f.max() and np.abs(got / f - 1).max() < 1e-6
        assert magnitude(s) == pytest.approx(m)
    f, m = pv.yarn_frequencies(8, 100.0, None)
    assert m == 1.0 and np.allclose(f, 100.0 ** (-np.arange(4) / 4))


def test_plain_model_mechanisms():
    """The oracle itself: causality, the sink lowers every weight, a layer that reads another's cache sees that cache."""
    cfg = CONFIGS["b"]()
    w = as_float64(random_weights(cfg, 3))
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 12).tolist()
    full = pv.forward(cfg, w, toks)
    assert np.allclose(pv.forward(cfg, w, toks[:7]), full[:7], atol=1e-10)
    w2 = dict(w)
    w2["l0.mix.sink"] = w["l0.mix.sink"] + 5.0
    assert not np.allclose(pv.forward(cfg, w2, toks), full, atol=1e-3)
    w3 = dict(w)
    w3["l0.mix.dkv"] = w["l0.mix.dkv"] * 1.5  # the latent is normed, the rotated key part is not: layer 1 must change too
    keep, keep3 = [], []
    pv.forward(cfg, w, toks, keep)
    pv.forward(cfg, w3, toks, keep3)
    assert not np.allclose(keep[1] - keep[0], keep3[1] - keep3[0], atol=1e-6)
