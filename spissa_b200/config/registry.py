"""One registry from an architecture's name to its configuration class and model.

``config.json`` names the architecture in ``architectures[0]`` (and ``model_type``);
the reference dispatches on a normalised string
(crates/spissa-import/src/safetensors.rs:202-232, crates/spissa-cli/src/commands/chat.rs:131-168).
Here an architecture registers a configuration class with two methods,
``from_dict(config_json) -> config`` and ``config.to_spec() -> ModelSpec``.
"""
from __future__ import annotations

import json
from pathlib import Path

_ARCHITECTURES: dict = {}
_MODEL_TYPES: dict = {}


class UnknownArchitecture(ValueError):
    pass


def register_architecture(name: str, config_cls, model_type: str | None = None) -> None:
    """Make ``config_cls`` the configuration of architecture ``name``.

    ``config_cls`` needs ``from_dict(dict)``, ``to_dict()`` and ``to_spec()``.
    """
    _ARCHITECTURES[name] = config_cls
    if model_type:
        _MODEL_TYPES[model_type] = config_cls


def unregister_architecture(name: str) -> None:
    cls = _ARCHITECTURES.pop(name, None)
    for k in [k for k, v in _MODEL_TYPES.items() if v is cls]:
        del _MODEL_TYPES[k]


def known_architectures() -> list:
    return sorted(_ARCHITECTURES)


def config_class_for(config_json: dict):
    names = list(config_json.get("architectures") or [])
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = config_json.get("model_type")
    if mt in _MODEL_TYPES:
        return _MODEL_TYPES[mt]
    asked = names or ([mt] if mt else ["<none given>"])
    raise UnknownArchitecture(
        f"no architecture registered for {asked}; known architectures: {known_architectures()}")


def config_from_dict(config_json: dict):
    return config_class_for(config_json).from_dict(config_json)


def load_config(folder_or_file):
    p = Path(folder_or_file)
    if p.is_dir():
        p = p / "config.json"
    if not p.exists():
        raise FileNotFoundError(f"no config.json at {p}")
    return config_from_dict(json.loads(p.read_text()))
