"""The one registry from an architecture's name to its configuration class and its model description."""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from ..errors import LoadError, UnsupportedError
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict], Any]      # config.json (dict) -> typed configuration
    build_spec: Callable[[Any], ModelSpec]   # typed configuration -> ModelSpec
    model_types: tuple[str, ...] = ()        # config.json "model_type" values that also select it
    # Sizes that config.json does not give and the checkpoint's tensor shapes do: {tensor name: shape} -> a value
    # that `parse_config(config_json, value)` takes as its second argument. None: the configuration says it all.
    shapes_to_config: Callable[[dict], Any] | None = None


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{arch.name}' is already registered")
    _ARCHITECTURES[arch.name] = arch


def architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(config_json: dict) -> Architecture:
    """Chooses by `architectures[0]` (or the single name under `architecture`), else by `model_type` (the only
    key the reference reads, src/model/config.cpp:39-42)."""
    names = config_json.get("architectures") or []
    if not names and isinstance(config_json.get("architecture"), str):
        names = [config_json["architecture"]]
    if names:
        if names[0] in _ARCHITECTURES:
            return _ARCHITECTURES[names[0]]
        raise UnsupportedError(f"architecture '{names[0]}' is not supported (supported: {', '.join(architectures())})")
    model_type = config_json.get("model_type")
    if model_type is None:
        raise LoadError("config.json has no 'model_type'")
    for arch in _ARCHITECTURES.values():
        if model_type in arch.model_types:
            return arch
    raise UnsupportedError(f"architecture '{model_type}' is not supported (supported: "
                           f"{', '.join(sorted(t for a in _ARCHITECTURES.values() for t in a.model_types))})")


def read_config_json(model_dir) -> dict:
    path = Path(model_dir) / "config.json"
    try:
        text = path.read_text()
    except OSError as e:
        raise LoadError(f"{path}: cannot open ({e.strerror})") from None
    try:
        cfg = json.loads(text)
    except json.JSONDecodeError as e:
        raise LoadError(f"{path}: invalid JSON: {e}") from None
    if not isinstance(cfg, dict):
        raise LoadError(f"{path}: expected a JSON object")
    return cfg


def checkpoint_present(model_dir) -> bool:
    d = Path(model_dir)
    return (d / "model.safetensors").exists() or (d / "model.safetensors.index.json").exists()


def load_config(model_dir):
    """config.json of a folder -> (architecture, typed configuration, model description)."""
    raw = read_config_json(model_dir)
    arch = resolve_architecture(raw)
    if arch.shapes_to_config is not None and checkpoint_present(model_dir):
        from ..weights.loader import SafetensorsSource
        shapes = {n: tuple(s) for n, (s, _) in SafetensorsSource(model_dir).shapes().items()}
        cfg = arch.parse_config(raw, arch.shapes_to_config(shapes))
    else:
        cfg = arch.parse_config(raw)
    spec = arch.build_spec(cfg)
    spec.validate()
    return arch, cfg, spec
