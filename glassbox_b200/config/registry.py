"""One registry from an architecture's name (config.json ``architectures[0]``, or a plain ``architecture`` string) to its model.

An ``Architecture`` is two functions and nothing else: ``parse`` turns the architecture's own
config.json keys into a ``ModelConfig`` (the typed, per-layer description), and ``bind`` says
which safetensors tensor names feed which parameter of which part. The model object itself is
always the generic ``glassbox_b200.engine.model.DecoderModel`` assembled from parts, so adding
an architecture never touches the step function, the cache, the scheduler or the kernels.

Glassbox has no registry: its loader always builds the Llama ``Model``
(crates/glassbox-server/src/main.rs:44-64). The registry is this engine's addition.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

from .specs import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    #: raw config.json dict -> ModelConfig
    parse: Callable[[dict], ModelConfig]
    #: ModelConfig -> {parameter path: weight source}; see glassbox_b200.weights.binding
    bind: Callable[[ModelConfig], dict]
    #: (keyword sizes) -> raw config.json dict, used by the random-weights mode and tests
    make_raw_config: Callable[..., dict] = None
    #: True: ``parse`` takes a second argument, {tensor name: shape} of the weights file (None when there is no file
    #: yet), for architectures some of whose sizes are written nowhere but in their tensors' shapes
    sizes_from_tensors: bool = False


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch


def architecture_names() -> List[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {', '.join(architecture_names()) or '(none)'}") from None


def architecture_of(raw: dict) -> str:
    """The architecture a config.json names: ``architectures[0]`` (the Hugging Face form) or a string ``architecture``."""
    archs = raw.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    if archs is None and isinstance(raw.get("architecture"), str):
        return raw["architecture"]
    raise ConfigError("config.json: 'architectures' must be a non-empty list of names (or 'architecture' one name)")


def parse_config(raw: dict, tensor_shapes: Optional[Dict[str, tuple]] = None) -> ModelConfig:
    """Pick the architecture by name and let it read its own keys (and, if it asks for them, the shapes of the weights
    file's tensors)."""
    arch = get_architecture(architecture_of(raw))
    config = arch.parse(raw, tensor_shapes) if arch.sizes_from_tensors else arch.parse(raw)
    config.validate()
    return config


def load_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    shapes = None
    if get_architecture(architecture_of(raw)).sizes_from_tensors:
        from ..weights.safetensors_io import SafetensorsFile
        weights = os.path.join(model_dir, "model.safetensors")
        if os.path.exists(weights):
            with SafetensorsFile(weights) as st:
                shapes = {name: tuple(st.shape(name)) for name in st.names()}
    return parse_config(raw, shapes)
