"""Lonorax without a GPU: the configuration reader (every optional key present and absent, every refusal), the binding of
tensor names to parameters, and properties of the plain implementation that the GPU tests compare against."""
import copy

import numpy as np
import pytest

import glassbox_b200  # noqa: F401  (registers the architectures)
from glassbox_b200.config.registry import get_architecture, parse_config
from glassbox_b200.config.specs import (ConfigError, LayerNormSpec, MinGruSpec, NoPositionSpec, RoutedExpertsSpec,
                                        SigmoidAttentionSpec)
from glassbox_b200.engine.model import DecoderModel
from glassbox_b200.parts.base import PagedKvSpec, StateSpec
from plain import lonorax_plain as plain
import lonorax_util as lu


@pytest.mark.parametrize("name", sorted(lu.CONFIGS))
def test_every_tensor_is_bound_exactly_once(name):
    raw = lu.CONFIGS[name]()
    config = parse_config(raw)
    model = DecoderModel(config)
    specs, binding = model.param_specs(), get_architecture("Lonorax").bind(config)
    assert set(binding) == set(specs)
    shapes = lu.tensor_shapes(raw)
    named = [n for path in specs for n in binding[path].names]
    assert sorted(named) == sorted(shapes)
    for path, spec in specs.items():
        names = binding[path].names
        rows = spec.pieces if len(names) > 1 else (spec.shape[0],)
        for n, r in zip(names, rows):
            assert tuple(shapes[n]) == (r,) + tuple(spec.shape[1:]), n


def test_what_the_reader_makes_of_the_keys():
    config = parse_config(lu.CONFIGS["odd"]())
    assert config.residual_streams == 3 and all(l.arrangement == "hyper_connections" and l.streams == 3 for l in config.layers)
    assert isinstance(config.final_norm, LayerNormSpec) and config.final_norm.eps == 1e-5 and config.final_norm.bias
    a, g = config.layers[0], config.layers[1]
    assert isinstance(a.mixer, SigmoidAttentionSpec) and (a.mixer.num_heads, a.mixer.num_kv_heads, a.mixer.head_dim, a.mixer.value_dim) == (6, 2, 20, 12)
    assert a.mixer.window == 7 and a.mixer.position.rotary_dim == 8 and a.mixer.position.pairing == "interleaved"
    assert a.mixer.position.theta == 500.0 and a.mixer.qk_norm_eps == 1e-5
    assert isinstance(a.ffn, RoutedExpertsSpec) and (a.ffn.num_experts, a.ffn.top_k, a.ffn.expert_size) == (6, 2, 24)
    assert (a.ffn.num_groups, a.ffn.keep_groups, a.ffn.route_scale, a.ffn.shared_size) == (3, 2, 2.5, 40)
    assert isinstance(g.mixer, MinGruSpec) and g.mixer.width == 44 and g.ffn is None and g.ffn_norm is None
    specs = DecoderModel(config).cache_layer_specs()
    assert specs[0] == PagedKvSpec(2, 20, 7, value_dim=12) and specs[1] == StateSpec((44,))
    plain_cfg = parse_config(lu.CONFIGS["plain"]())
    assert plain_cfg.residual_streams == 0 and all(l.arrangement == "pre_norm" for l in plain_cfg.layers)
    m = plain_cfg.layers[0].mixer
    assert m.window is None and isinstance(m.position, NoPositionSpec)
    f = plain_cfg.layers[0].ffn
    assert (f.num_groups, f.keep_groups, f.shared_size, f.route_scale) == (1, 1, 0, 1.0)


def _broken(change):
    raw = lu.CONFIGS["odd"]()
    change(raw)
    return raw


@pytest.mark.parametrize("change, word", [
    (lambda r: r.pop("vocab"), "vocab"),
    (lambda r: r["norm"].pop("eps"), "eps"),
    (lambda r: r.update(streams=0), "streams"),
    (lambda r: r.update(streams=9), "streams"),
    (lambda r: r.update(layers=[]), "layers"),
    (lambda r: r["layers"][0].update(type="conv"), "conv"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=4), "multiple"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=22), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda r: r["layers"][0]["mlp"].update(kind="dense"), "dense"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=7), "do not fit"),
    (lambda r: r["layers"][0]["mlp"]["router"]["groups"].update(count=4), "do not fit"),
    (lambda r: r["layers"][0]["mlp"]["router"]["groups"].update(keep=1, count=6), "do not fit"),
    (lambda r: r["layers"][1]["mixer"].pop("width"), "width"),
])
def test_refusals_name_the_key(change, word):
    with pytest.raises(ConfigError) as e:
        parse_config(_broken(change))
    assert word in str(e.value)


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from glassbox_b200.weights.random_init import random_tensors
    raw = lu.CONFIGS["odd"]()
    tensors = random_tensors(raw, seed=3)
    assert sorted(tensors) == sorted(lu.tensor_shapes(raw))
    mix = tensors["l0.hc1.mix"].float().numpy()
    assert abs(mix.mean() - 1 / 3) < 0.2 and abs(tensors["l0.norm1.b"].float().mean()) < 0.1      # biases around zero, not one


# ------------------------------------------------------------------------------- the plain implementation itself
def test_plain_attention_sums_exactly_the_visible_keys():
    """With scores pushed to +large every visible key weighs 1: the output is the plain sum of the visible values."""
    T, D = 12, 4
    m = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": D, "scale": 50.0, "mask": {"size": 5}}
    h = np.ones((T, D)) + 0.01 * np.arange(T)[:, None]
    W = {"q": np.eye(D), "k": np.eye(D), "v": np.eye(D), "q.norm": np.ones(D), "k.norm": np.ones(D), "pb": np.zeros(1), "o": np.eye(D)}
    out = plain.sigmoid_attention(h, W, "", m, 1e-6)
    for i in range(T):
        np.testing.assert_allclose(out[i], h[max(0, i - 4):i + 1].sum(0), rtol=1e-9)
    assert plain.visible(7, 3, 5) and not plain.visible(7, 2, 5) and plain.visible(7, 7, 1) and not plain.visible(7, 6, 1)
    assert plain.visible(7, 0, None) and not plain.visible(3, 4, None)


def test_plain_rotation_keeps_lengths_and_relative_angles():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((6, 2, 8))
    r = plain.rotate_pairs(x, np.arange(6), 4, 100.0)
    np.testing.assert_allclose((r ** 2).sum(-1), (x ** 2).sum(-1))
    np.testing.assert_array_equal(r[..., 4:], x[..., 4:])                       # channels beyond the rotated ones pass
    np.testing.assert_array_equal(r[0], x[0])                                   # position 0: no rotation
    a = plain.rotate_pairs(np.tile(x[:1], (6, 1, 1)), np.arange(6), 4, 100.0)
    np.testing.assert_allclose((a[5] * a[3]).sum(-1), (a[2] * a[0]).sum(-1))    # dot products depend on the distance only


def test_plain_mingru_limits():
    w = 3
    W = {"z": np.zeros((w, 2)), "x": np.zeros((w, 2)), "g": np.zeros((w, 2)), "o": np.eye(w), "z.b": np.full(w, 50.0),
         "x.b": np.array([-1.0, 0.0, 2.0])}
    h = np.ones((4, 2))
    _, S = plain.mingru(h, W, "")
    np.testing.assert_allclose(S, [plain.logistic(-1.0), 0.5, 2.5])              # gate open: the state is the candidate
    W["z.b"] = np.full(w, -50.0)
    _, S = plain.mingru(h, W, "", state=[1.0, 2.0, 3.0])
    np.testing.assert_allclose(S, [1.0, 2.0, 3.0])                               # gate shut: the state stays
    W["z.b"] = np.zeros(w)
    full, S_full = plain.mingru(np.ones((7, 2)), W, "")
    _, S_a = plain.mingru(np.ones((3, 2)), W, "")
    _, S_b = plain.mingru(np.ones((4, 2)), W, "", state=S_a)
    np.testing.assert_allclose(S_b, S_full)                                      # a portion continues from the state before


def test_plain_streams_reduce_to_a_plain_residual():
    """One stream with read = mix = write = 1 is x + y."""
    x, y = np.arange(6.0).reshape(1, 2, 3), np.ones((2, 3))
    np.testing.assert_array_equal(plain.stream_write(x, np.ones((1, 1)), np.ones(1), y)[0], x[0] + y)
    np.testing.assert_array_equal(plain.stream_read(x, np.ones(1)), x[0])
    xs = np.stack([x[0], 2 * x[0]])
    mix = np.array([[1.0, 0.5], [0.0, 2.0]])                                     # [from, to]
    new = plain.stream_write(xs, mix, np.array([1.0, -1.0]), y)
    np.testing.assert_array_equal(new[0], xs[0] + y)
    np.testing.assert_array_equal(new[1], 0.5 * xs[0] + 2.0 * xs[1] - y)
