"""One registry from an architecture's name to its configuration class.

The name is `architectures[0]` of config.json; a folder without that key falls
back on `model_type`, the only key the reference dispatches on
(src/model/model_config.cpp:31).  A configuration class has `from_dict`,
`to_dict` and `build_spec() -> ModelSpec`; registering one is all that adding an
architecture needs at this level.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, Mapping, Type

from .qwen2 import ConfigError, Qwen2Config

_ARCHITECTURES: Dict[str, Type] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(name: str, config_class: Type, model_type: str = "") -> None:
    """Make `name` (as written in config.json `architectures`) resolve to `config_class`."""
    for attribute in ("from_dict", "to_dict", "build_spec"):
        if not hasattr(config_class, attribute):
            raise TypeError(f"{config_class.__name__} lacks {attribute}()")
    _ARCHITECTURES[name] = config_class
    if model_type:
        _MODEL_TYPES[model_type] = name


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)
    for model_type in [k for k, v in _MODEL_TYPES.items() if v == name]:
        del _MODEL_TYPES[model_type]


def registered_architectures():
    return sorted(_ARCHITECTURES)


def architecture_name(data: Mapping[str, Any]) -> str:
    names = data.get("architectures")
    if isinstance(names, (list, tuple)) and names:
        return str(names[0])
    model_type = str(data.get("model_type", ""))
    if model_type in _MODEL_TYPES:
        return _MODEL_TYPES[model_type]
    raise ConfigError("config.json names no architecture: neither 'architectures' nor a known "
                      f"'model_type' (registered: {', '.join(registered_architectures())})")


def config_from_dict(data: Mapping[str, Any]):
    name = architecture_name(data)
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture '{name}' is not registered "
                          f"(registered: {', '.join(registered_architectures())})")
    return _ARCHITECTURES[name].from_dict(data)


def load_config(model_dir) -> Any:
    path = Path(model_dir) / "config.json"
    try:
        text = path.read_text(encoding="utf-8")
    except OSError as error:
        raise ConfigError(f"cannot read {path}: {error}") from error
    try:
        data = json.loads(text)
    except json.JSONDecodeError as error:
        raise ConfigError(f"{path} is not valid JSON: {error}") from error
    if not isinstance(data, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return config_from_dict(data)


register_architecture("Qwen2ForCausalLM", Qwen2Config, model_type="qwen2")
