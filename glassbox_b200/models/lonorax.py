"""Lonorax: a decoder whose layers mix tokens either with a minGRU (a gated recurrence with a fixed-size float32 state per
request) or with sliding-window attention whose weights are sigmoids instead of a softmax (query/key norm per head,
rotation of the leading channels in neighbouring pairs, a learned bias per head), whose feed-forwards are mixtures of small
squared-ReLU experts with sigmoid routing, a choice correction, a limit to the best groups of experts and a gated shared
expert, whose norms are layer norms with bias, and whose residual is kept as several streams (hyper-connections).

This file only *describes* the architecture: which config.json keys it reads and how tensor names map onto part parameters.
The math lives in the parts (``parts/mingru.py``, ``parts/sigmoid_attention.py``, ``parts/moe.py``, ``parts/norm.py``,
``parts/block.py``).

config.json: ``architecture`` "Lonorax"; ``vocab``, ``width``; ``norm.eps``; ``streams`` (absent: one plain residual row,
pre-norm layers); ``layers``: a list of {``type``: "mingru" | "attention", ``mixer``: sizes, ``mlp``: {``kind``: "moe",
``expert.ff``, ``router``: {``experts``, ``top``, ``scale``, ``groups``: {``count``, ``keep``}}, ``shared``: {``ff``}} or
null}. A minGRU mixer gives ``width``; an attention mixer ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
``mask.size`` (absent: every earlier token is visible) and ``rot``: {``base``, ``dims``} (absent: no rotation). Optional
parts of the feed-forward (``groups``, ``shared``, ``router.scale``) may be absent. Tensors of layer i start with ``l<i>.``:
``norm1``, ``norm1.b`` (mixer ``mix.*``), ``norm2``, ``norm2.b`` (feed-forward ``mlp.*``), ``hc1.*`` / ``hc2.*`` (``in``,
``out``, ``mix`` of the two branches' stream mixing); ``embed``, ``final.norm``, ``final.norm.b``, ``head``.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.specs import (ConfigError, LayerNormSpec, LayerSpec, MinGruSpec, ModelConfig, NoPositionSpec, RopeSpec,
                            RoutedExpertsSpec, RunSpec, SigmoidAttentionSpec)
from ..weights.binding import Stacked

NAME = "Lonorax"
#: no key limits the length of a sequence; angles are formed on the device, so this only bounds requests
DEFAULT_MAX_POSITION = 1 << 20


def _get(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _pos_int(d, key: str, where: str) -> int:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _number(d, key: str, where: str) -> float:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


def _mixer(kind: str, m: dict, where: str, eps: float, max_pos: int):
    if kind == "mingru":
        return MinGruSpec(width=_pos_int(m, "width", where))
    if kind == "attention":
        heads, kv_heads = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: heads {heads} is not a multiple of kv_heads {kv_heads}")
        dim = _pos_int(m, "dim", where)
        position = NoPositionSpec()
        if m.get("rot") is not None:
            rot = m["rot"]
            dims = _pos_int(rot, "dims", where + ".rot")
            if dims % 2 or dims > dim:
                raise ConfigError(f"config.json: {where}: rot.dims {dims} must be even and at most dim {dim}")
            position = RopeSpec(theta=_number(rot, "base", where + ".rot"), rotary_dim=dims, max_position=max_pos,
                                pairing="interleaved")
        window = _pos_int(m["mask"], "size", where + ".mask") if m.get("mask") is not None else None
        return SigmoidAttentionSpec(num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=_pos_int(m, "vdim", where),
                                    scale=_number(m, "scale", where), position=position, window=window, qk_norm_eps=eps,
                                    head_bias=True)
    raise ConfigError(f"config.json: {where}: unknown layer type {kind!r}")


def _feed_forward(mlp, where: str):
    if mlp is None:
        return None
    if _get(mlp, "kind", where) != "moe":
        raise ConfigError(f"config.json: {where}: unknown kind {mlp['kind']!r}")
    router = _get(mlp, "router", where)
    experts, top = _pos_int(router, "experts", where + ".router"), _pos_int(router, "top", where + ".router")
    groups = router.get("groups")
    count = _pos_int(groups, "count", where + ".router.groups") if groups is not None else 1
    keep = _pos_int(groups, "keep", where + ".router.groups") if groups is not None else 1
    if top > experts or experts % count or keep > count or keep * (experts // count) < top:
        raise ConfigError(f"config.json: {where}.router: {experts} experts, {top} per token, {keep} of {count} groups do not fit")
    shared = mlp.get("shared")
    return RoutedExpertsSpec(num_experts=experts, top_k=top, expert_size=_pos_int(_get(mlp, "expert", where), "ff", where + ".expert"),
                             route_scale=_number(router, "scale", where + ".router") if "scale" in router else 1.0,
                             num_groups=count, keep_groups=keep, correction=True,
                             shared_size=_pos_int(shared, "ff", where + ".shared") if shared is not None else 0, shared_gate=True)


def parse_lonorax_config(raw: dict) -> ModelConfig:
    vocab = _pos_int(raw, "vocab", "top level")
    width = _pos_int(raw, "width", "top level")
    eps = _number(_get(raw, "norm", "top level"), "eps", "norm")
    if not eps > 0:
        raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
    streams = _pos_int(raw, "streams", "top level") if raw.get("streams") is not None else 0
    if streams > 8:
        raise ConfigError(f"config.json: {streams} streams; at most 8 are supported")
    layers_raw = _get(raw, "layers", "top level")
    if not isinstance(layers_raw, list) or not layers_raw:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    max_pos = raw.get("max_position", DEFAULT_MAX_POSITION)
    if isinstance(max_pos, bool) or not isinstance(max_pos, int) or max_pos <= 0:
        raise ConfigError(f"config.json: 'max_position' must be a positive integer, got {max_pos!r}")
    norm = LayerNormSpec(eps=eps, bias=True)
    layers, schedule = [], []
    for i, L in enumerate(layers_raw):
        where = f"layers[{i}]"
        mixer = _mixer(_get(L, "type", where), _get(L, "mixer", where), where, eps, max_pos)
        ffn = _feed_forward(L.get("mlp"), where + ".mlp")
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=norm if ffn is not None else None,
                                arrangement="hyper_connections" if streams else "pre_norm", streams=streams))
        schedule.append(RunSpec(layer=i, cache=i))
    return ModelConfig(architecture=NAME, vocab_size=vocab, hidden_size=width, max_position=max_pos, tie_word_embeddings=False,
                       layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, raw=dict(raw), residual_streams=streams)


def bind_lonorax_weights(config: ModelConfig) -> dict:
    b = {"embed.weight": Stacked(("embed",)), "final_norm.weight": Stacked(("final.norm",)),
         "final_norm.bias": Stacked(("final.norm.b",)), "head.weight": Stacked(("head",))}
    for i, layer in enumerate(config.layers):
        p, t = f"layers.{i}", f"l{i}"
        m = f"{t}.mix"
        branches = [("mixer", "norm1", "hc1")] + ([("ffn", "norm2", "hc2")] if layer.ffn is not None else [])
        for part, norm, hc in branches:
            b[f"{p}.{part}_norm.weight"] = Stacked((f"{t}.{norm}",))
            b[f"{p}.{part}_norm.bias"] = Stacked((f"{t}.{norm}.b",))
            if config.residual_streams:
                b[f"{p}.{part}_streams.read"] = Stacked((f"{t}.{hc}.in",))
                b[f"{p}.{part}_streams.write"] = Stacked((f"{t}.{hc}.out",))
                b[f"{p}.{part}_streams.mix"] = Stacked((f"{t}.{hc}.mix",))
        if isinstance(layer.mixer, MinGruSpec):
            b[f"{p}.mixer.w_in"] = Stacked((f"{m}.z", f"{m}.x", f"{m}.g"))
            b[f"{p}.mixer.bias_z"] = Stacked((f"{m}.z.b",))
            b[f"{p}.mixer.bias_x"] = Stacked((f"{m}.x.b",))
            b[f"{p}.mixer.wo"] = Stacked((f"{m}.o",))
        else:
            b[f"{p}.mixer.w_in"] = Stacked((f"{m}.q", f"{m}.k", f"{m}.v"))
            b[f"{p}.mixer.q_norm"] = Stacked((f"{m}.q.norm",))
            b[f"{p}.mixer.k_norm"] = Stacked((f"{m}.k.norm",))
            b[f"{p}.mixer.head_bias"] = Stacked((f"{m}.pb",))
            b[f"{p}.mixer.wo"] = Stacked((f"{m}.o",))
        if layer.ffn is not None:
            f = f"{t}.mlp"
            E = layer.ffn.num_experts
            b[f"{p}.ffn.router"] = Stacked((f"{f}.router",))
            b[f"{p}.ffn.correction"] = Stacked((f"{f}.correction",))
            b[f"{p}.ffn.w_up"] = Stacked(tuple(f"{f}.e{j}.up" for j in range(E)))
            b[f"{p}.ffn.w_down"] = Stacked(tuple(f"{f}.e{j}.down" for j in range(E)))
            if layer.ffn.shared_size:
                b[f"{p}.ffn.shared_up"] = Stacked((f"{f}.shared.up",))
                b[f"{p}.ffn.shared_down"] = Stacked((f"{f}.shared.down",))
                b[f"{p}.ffn.shared_gate"] = Stacked((f"{f}.shared.sg",))
    return b


def make_lonorax_raw_config(*, vocab: int, width: int, layers: list, streams=None, norm_eps: float = 1e-6) -> dict:
    """``layers``: a list of dicts as config.json holds them ({"type", "mixer", "mlp"})."""
    raw = {"architecture": NAME, "vocab": vocab, "width": width, "norm": {"eps": norm_eps}, "layers": layers}
    if streams is not None:
        raw["streams"] = streams
    return raw


register_architecture(Architecture(name=NAME, parse=parse_lonorax_config, bind=bind_lonorax_weights,
                                   make_raw_config=make_lonorax_raw_config), replace=True)
