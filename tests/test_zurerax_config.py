"""Zurerax without a GPU: configuration, tensor binding, weight loading, and checks of the plain implementation itself
(properties that follow from the equations, so that the judge of the GPU tests is judged too)."""
import json
import os

import numpy as np
import pytest
import torch

import glassbox_b200
from glassbox_b200.config import ConfigError, parse_config
from glassbox_b200.config.registry import get_architecture
from glassbox_b200.engine.model import DecoderModel
from glassbox_b200.parts.base import PagedKvSpec, StateSpec
from glassbox_b200.weights.loader import load_parameters, open_model_weights
from glassbox_b200.weights.safetensors_io import WeightsError

from plain import zurerax_plain as plain
import zurerax_util as zu


@pytest.mark.parametrize("name", sorted(zu.CONFIGS))
def test_parse_bind_and_load(name, tmp_path):
    cfg = zu.CONFIGS[name]()
    folder = zu.write_model(str(tmp_path / name), cfg, zu.random_weights(cfg, 3))
    config = glassbox_b200.load_config(folder)                      # ranks come from the tensors' shapes
    assert config.architecture == "Zurerax" and config.vocab_size == cfg["vocab"] and config.hidden_size == cfg["width"]
    assert len(config.layers) == len(cfg["layers"])
    model = DecoderModel(config)
    binding = get_architecture("Zurerax").bind(config)
    assert set(binding) == set(model.param_specs())
    named = {n for src in binding.values() for n in src.names}
    assert named == set(zu.tensor_shapes(cfg))                      # every tensor of the file is used, none is invented
    with open_model_weights(folder) as st:
        params = load_parameters(model.param_specs(), binding, st, torch.bfloat16, "cpu")
    model.bind(params)
    for i, L in enumerate(cfg["layers"]):
        run = config.schedule[i]
        assert run.layer == i
        if L["type"] == "latent_attention" and "kv_from" in L["mixer"]:
            assert not run.writes_cache and run.cache == config.schedule[L["mixer"]["kv_from"]].cache
        else:
            assert run.writes_cache
    specs = model.cache_layer_specs()
    assert all(isinstance(s, (PagedKvSpec, StateSpec)) for s in specs)
    # the gain of a norm stored around zero is 1 + weight
    w = zu.random_weights(cfg, 3)["l0.norm1"].float()
    assert torch.equal(model.layers[0].mixer_norm.params["weight"], w + 1.0)


def test_ranks_come_from_shapes_or_keys():
    cfg = zu.CONFIGS["odd"]()
    assert parse_config(cfg).layers[1].mixer.decay_rank == 5       # given as keys (no weights file yet)
    with pytest.raises(ConfigError, match="rank"):
        parse_config(zu.file_config(cfg))                           # neither keys nor shapes
    shapes = zu.tensor_shapes(cfg)
    assert parse_config(zu.file_config(cfg), shapes).layers[1].mixer.gate_rank == 7


@pytest.mark.parametrize("damage, message", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),           # names a delta-rule layer
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),           # names itself
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=48), "kv_rank"),          # another latent size than its source
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0].update(type="sliding"), "unknown layer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "unknown kind"),
    (lambda c: c.pop("logit_scale"), "logit_scale"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
])
def test_bad_configs_are_refused(damage, message):
    cfg = zu.CONFIGS["odd"]()
    damage(cfg)
    with pytest.raises(ConfigError, match=message):
        parse_config(cfg)


def test_wrong_weights_are_reported_together(tmp_path):
    cfg = zu.CONFIGS["ones"]()
    tensors = zu.random_weights(cfg, 1)
    del tensors["l1.mix.sink"]
    tensors["l0.mix.A_log"] = torch.zeros(3, dtype=torch.bfloat16)
    folder = zu.write_model(str(tmp_path / "m"), cfg, tensors)
    config = glassbox_b200.load_config(folder)
    model = DecoderModel(config)
    with open_model_weights(folder) as st, pytest.raises(WeightsError) as e:
        load_parameters(model.param_specs(), get_architecture("Zurerax").bind(config), st, torch.bfloat16, "cpu")
    assert "l1.mix.sink" in str(e.value) and "l0.mix.A_log" in str(e.value)


# ------------------------------------------------------------------ the plain implementation, against its own equations
def test_plain_delta_rule_stores_and_recalls():
    rng = np.random.default_rng(0)
    D, V = 6, 4
    k = rng.standard_normal((3, 1, D))
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    v = rng.standard_normal((3, 1, V))
    ones, beta = np.ones((3, 1, D)), np.ones((3, 1))
    # no decay, beta 1: reading with the key just written returns the value just written (the write is a correction)
    o = plain.delta_rule(k, k, v, ones, beta)
    np.testing.assert_allclose(o, v, atol=1e-12)
    # beta 0: nothing is ever written
    assert np.all(plain.delta_rule(k, k, v, ones, np.zeros((3, 1))) == 0)
    # a decay of zero on every channel forgets everything before the current token
    o = plain.delta_rule(k, k, v, np.zeros((3, 1, D)), beta)
    np.testing.assert_allclose(o, v, atol=1e-12)
    # with orthogonal keys and no decay an old value is still there
    k2 = np.zeros((2, 1, D)); k2[0, 0, 0] = 1; k2[1, 0, 1] = 1
    q2 = np.zeros((2, 1, D)); q2[:, 0, 0] = 1
    o = plain.delta_rule(q2, k2, v[:2], np.ones((2, 1, D)), np.ones((2, 1)))
    np.testing.assert_allclose(o[1], v[0], atol=1e-12)


def test_plain_conv_rotation_and_sink():
    x = np.arange(12, dtype=np.float64).reshape(6, 2)
    w = np.array([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]])        # channel 0: the current token; channel 1: two tokens back
    y = plain.causal_conv(x, w)
    np.testing.assert_allclose(y[:, 0], x[:, 0])
    np.testing.assert_allclose(y[:, 1], [0, 0, 1, 3, 5, 7])
    # a rotation keeps lengths, turns by position * frequency, and leaves position 0 alone
    v = np.array([[1.0, 0.0, 0.0, 2.0]] * 3)
    r = plain.rotate_interleaved(v, np.array([0.0, 1.0, 2.0]), 100.0, 4)
    np.testing.assert_allclose(r[0], v[0])
    np.testing.assert_allclose(np.linalg.norm(r, axis=-1), np.linalg.norm(v, axis=-1))
    np.testing.assert_allclose(r[2, :2], [np.cos(2.0), np.sin(2.0)])
    np.testing.assert_allclose(r[2, 2:], [-2 * np.sin(2 * 0.1), 2 * np.cos(2 * 0.1)])
    # the sink takes its share of the probability and gives nothing back
    s = np.array([[0.0, -np.inf], [0.0, 0.0]])
    p = plain.softmax_with_sink(s, 0.0)
    np.testing.assert_allclose(p, [[0.5, 0.0], [1 / 3, 1 / 3]])
    np.testing.assert_allclose(plain.softmax_with_sink(s, -1e9), [[1.0, 0.0], [0.5, 0.5]])


def test_plain_forward_is_causal_and_deterministic():
    cfg = zu.CONFIGS["odd"]()
    W = zu.as_float64(zu.random_weights(cfg, 5))
    toks = list(np.random.default_rng(1).integers(0, cfg["vocab"], 19))
    a = plain.forward(cfg, W, toks)
    b = plain.forward(cfg, W, toks[:11])
    np.testing.assert_allclose(a[:11], b, atol=1e-9)
    assert np.isfinite(a).all() and a.std() > 0.1
