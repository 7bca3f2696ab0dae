"""Zurerax: a decoder whose layers mix tokens either with a gated delta rule (a fixed-size recurrent state per head, one
decay per key channel) or with attention over a compressed latent cache (optionally the cache of an earlier layer), each
branch normed on the way in and on the way out, with a squared-ReLU feed-forward, a scaled embedding and scaled logits.

This file only *describes* the architecture: which config.json keys it reads, which sizes it takes from the shapes of the
weights file's tensors, and how tensor names map onto part parameters. The math lives in the parts
(``parts/delta_rule.py``, ``parts/latent_attention.py``, ``parts/block.py``, ``parts/mlp.py``, ``parts/norm.py``).

config.json: ``architecture`` "Zurerax"; ``vocab``, ``width``; ``embedding.scale``; ``logit_scale``; ``norm.eps``;
``layers``: a list of {``type``: "channel_delta" | "latent_attention", ``mixer``: sizes, ``mlp``: {``kind``: "dense",
``ff``} or null}. Tensors of layer i start with ``l<i>.``: ``norm1``, ``norm1b`` around the mixer (``mix.*``), ``norm2``,
``norm2b`` around the feed-forward (``mlp.up``, ``mlp.down``); ``embed``, ``final.norm``, ``head``. The ranks of the
delta-rule mixer's two low-rank maps are written in no key: they are the row counts of ``mix.a1`` and ``mix.g1``
(a config made for random weights may give them as ``mixer.decay_rank`` / ``mixer.gate_rank``).
"""
from __future__ import annotations

from typing import Dict, Optional

from ..config.registry import Architecture, register_architecture
from ..config.specs import (ChannelDeltaSpec, ConfigError, LatentAttentionSpec, LayerSpec, ModelConfig, RopeSpec, RunSpec,
                            ScaledEmbeddingSpec, ScaledLmHeadSpec, SquaredReluSpec, UnitOffsetRmsNormSpec)
from ..weights.binding import Stacked

NAME = "Zurerax"
#: no key limits the length of a sequence; positions are formed on the device, so this only bounds requests
DEFAULT_MAX_POSITION = 1 << 20


def _get(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _pos_int(d: dict, key: str, where: str) -> int:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _number(d: dict, key: str, where: str) -> float:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


def _rank(mixer: dict, key: str, tensor: str, shapes: Optional[Dict[str, tuple]], where: str) -> int:
    if shapes is not None and tensor in shapes and len(shapes[tensor]) == 2:
        return int(shapes[tensor][0])
    if isinstance(mixer.get(key), int) and mixer[key] > 0:
        return mixer[key]
    raise ConfigError(f"config.json: {where}: the rank '{key}' is neither given nor readable from the shape of {tensor}")


def parse_zurerax_config(raw: dict, shapes: Optional[Dict[str, tuple]] = None) -> ModelConfig:
    vocab = _pos_int(raw, "vocab", "top level")
    width = _pos_int(raw, "width", "top level")
    eps = _number(_get(raw, "norm", "top level"), "eps", "norm")
    if not eps > 0:
        raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
    emb_scale = _number(_get(raw, "embedding", "top level"), "scale", "embedding")
    logit_scale = _number(raw, "logit_scale", "top level")
    layers_raw = _get(raw, "layers", "top level")
    if not isinstance(layers_raw, list) or not layers_raw:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    max_pos = raw.get("max_position", DEFAULT_MAX_POSITION)
    if isinstance(max_pos, bool) or not isinstance(max_pos, int) or max_pos <= 0:
        raise ConfigError(f"config.json: 'max_position' must be a positive integer, got {max_pos!r}")
    norm = UnitOffsetRmsNormSpec(eps=eps)
    layers, schedule = [], []
    cache_of: Dict[int, int] = {}          # layer -> the cache layer it writes
    for i, L in enumerate(layers_raw):
        where = f"layers[{i}]"
        kind = _get(L, "type", where)
        m = _get(L, "mixer", where)
        if kind == "channel_delta":
            mixer = ChannelDeltaSpec(
                num_heads=_pos_int(m, "heads", where), num_kv_heads=_pos_int(m, "kv_heads", where),
                key_dim=_pos_int(m, "dim", where), value_dim=_pos_int(m, "vdim", where), conv_taps=_pos_int(m, "conv", where),
                decay_rank=_rank(m, "decay_rank", f"l{i}.mix.a1", shapes, where),
                gate_rank=_rank(m, "gate_rank", f"l{i}.mix.g1", shapes, where), norm_eps=eps)
            if mixer.num_heads % mixer.num_kv_heads:
                raise ConfigError(f"config.json: {where}: heads {mixer.num_heads} is not a multiple of kv_heads {mixer.num_kv_heads}")
            cache_of[i] = len(cache_of)
            run = RunSpec(layer=i, cache=cache_of[i])
        elif kind == "latent_attention":
            rot = _get(m, "rot", where)
            rot_dim = _pos_int(m, "rot_dim", where)
            dims = _pos_int(rot, "dims", where + ".rot")
            if dims % 2 or dims > rot_dim:
                raise ConfigError(f"config.json: {where}: rot.dims {dims} must be even and at most rot_dim {rot_dim}")
            source = m.get("kv_from")
            if source is not None and (isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i
                                       or not isinstance(layers[source].mixer, LatentAttentionSpec)
                                       or layers[source].mixer.kv_source is not None):
                raise ConfigError(f"config.json: {where}: kv_from {source!r} must name an earlier latent_attention layer "
                                  "that projects its own latent")
            mixer = LatentAttentionSpec(
                num_heads=_pos_int(m, "heads", where), nope_dim=_pos_int(m, "dim", where), rope_dim=rot_dim,
                value_dim=_pos_int(m, "vdim", where), latent_dim=_pos_int(m, "kv_rank", where),
                scale=_number(m, "scale", where),
                position=RopeSpec(theta=_number(rot, "base", where + ".rot"), rotary_dim=dims, max_position=max_pos,
                                  pairing="interleaved"),
                latent_eps=eps, sink=True, kv_source=source)
            if source is not None:
                src = layers[source].mixer
                if (src.latent_dim, src.rope_dim, src.position) != (mixer.latent_dim, mixer.rope_dim, mixer.position):
                    raise ConfigError(f"config.json: {where}: kv_rank, rot_dim and rot must equal those of layer {source}, "
                                      "whose cache it reads")
                run = RunSpec(layer=i, cache=cache_of[source], writes_cache=False)
            else:
                cache_of[i] = len(cache_of)
                run = RunSpec(layer=i, cache=cache_of[i])
        else:
            raise ConfigError(f"config.json: {where}: unknown layer type {kind!r}")
        mlp = L.get("mlp")
        ffn = None
        if mlp is not None:
            if _get(mlp, "kind", where + ".mlp") != "dense":
                raise ConfigError(f"config.json: {where}.mlp: unknown kind {mlp['kind']!r}")
            ffn = SquaredReluSpec(intermediate_size=_pos_int(mlp, "ff", where + ".mlp"))
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=norm if ffn is not None else None,
                                arrangement="sandwich_norm", mixer_post_norm=norm,
                                ffn_post_norm=norm if ffn is not None else None))
        schedule.append(run)
    return ModelConfig(architecture=NAME, vocab_size=vocab, hidden_size=width, max_position=max_pos,
                       tie_word_embeddings=False, layers=tuple(layers), schedule=tuple(schedule), final_norm=norm,
                       raw=dict(raw), embedding=ScaledEmbeddingSpec(scale=emb_scale), head=ScaledLmHeadSpec(scale=logit_scale))


def bind_zurerax_weights(config: ModelConfig) -> dict:
    b = {"embed.weight": Stacked(("embed",)), "final_norm.weight": Stacked(("final.norm",)),
         "head.weight": Stacked(("head",))}
    for i, layer in enumerate(config.layers):
        p, t = f"layers.{i}", f"l{i}"
        b[f"{p}.mixer_norm.weight"] = Stacked((f"{t}.norm1",))
        b[f"{p}.mixer_post_norm.weight"] = Stacked((f"{t}.norm1b",))
        m = f"{t}.mix"
        if isinstance(layer.mixer, ChannelDeltaSpec):
            b[f"{p}.mixer.w_in"] = Stacked((f"{m}.q", f"{m}.k", f"{m}.v", f"{m}.a1", f"{m}.g1", f"{m}.b"))
            b[f"{p}.mixer.conv"] = Stacked((f"{m}.q.conv", f"{m}.k.conv", f"{m}.v.conv"))
            b[f"{p}.mixer.w_a2"] = Stacked((f"{m}.a2",))
            b[f"{p}.mixer.w_g2"] = Stacked((f"{m}.g2",))
            b[f"{p}.mixer.dt_bias"] = Stacked((f"{m}.dt_bias",))
            b[f"{p}.mixer.a_log"] = Stacked((f"{m}.A_log",))
            b[f"{p}.mixer.out_norm"] = Stacked((f"{m}.norm",))
            b[f"{p}.mixer.wo"] = Stacked((f"{m}.o",))
        else:
            if layer.mixer.kv_source is None:
                b[f"{p}.mixer.w_in"] = Stacked((f"{m}.q", f"{m}.dkv"))
                b[f"{p}.mixer.latent_norm"] = Stacked((f"{m}.dkv.norm",))
            else:
                b[f"{p}.mixer.w_in"] = Stacked((f"{m}.q",))
            b[f"{p}.mixer.w_uk"] = Stacked((f"{m}.uk",))
            b[f"{p}.mixer.w_uv"] = Stacked((f"{m}.uv",))
            b[f"{p}.mixer.sink"] = Stacked((f"{m}.sink",))
            b[f"{p}.mixer.wo"] = Stacked((f"{m}.o",))
        if layer.ffn is not None:
            b[f"{p}.ffn_norm.weight"] = Stacked((f"{t}.norm2",))
            b[f"{p}.ffn_post_norm.weight"] = Stacked((f"{t}.norm2b",))
            b[f"{p}.ffn.w_up"] = Stacked((f"{t}.mlp.up",))
            b[f"{p}.ffn.w_down"] = Stacked((f"{t}.mlp.down",))
    return b


def make_zurerax_raw_config(*, vocab: int, width: int, layers: list, embedding_scale: float = 1.0, logit_scale: float = 1.0,
                            norm_eps: float = 1e-6) -> dict:
    """``layers``: a list of dicts as config.json holds them ({"type", "mixer", "mlp"}); a delta-rule mixer's dict also
    carries "decay_rank" and "gate_rank", since no weights file exists yet to read them from."""
    return {"architecture": NAME, "vocab": vocab, "width": width, "embedding": {"scale": embedding_scale},
            "logit_scale": logit_scale, "norm": {"eps": norm_eps}, "layers": layers}


register_architecture(Architecture(name=NAME, parse=parse_zurerax_config, bind=bind_zurerax_weights,
                                   make_raw_config=make_zurerax_raw_config, sizes_from_tensors=True), replace=True)
