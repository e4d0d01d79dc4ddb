"""Registries: architecture name -> (config class, spec builder); part kind -> class.

Adding an architecture is one ``register_architecture`` call with a typed config
class and a function from that config to a ``ModelSpec``; adding a part is one
``register_part`` call.  Nothing else in the package names an architecture.
"""
from __future__ import annotations

from typing import Any, Callable

from .config.base import ConfigError, read_config_json

_ARCHITECTURES: dict[str, tuple[Any, Callable]] = {}
_MODEL_TYPES: dict[str, str] = {}
_PARTS: dict[str, dict[str, type]] = {"norm": {}, "position": {}, "mixer": {}, "ffn": {}, "block": {}}


def register_architecture(name: str, config_cls, build_spec: Callable, model_type: str | None = None) -> None:
    """``config_cls.from_dict(raw) -> config``; ``build_spec(config) -> ModelSpec``."""
    _ARCHITECTURES[name] = (config_cls, build_spec)
    if model_type:
        _MODEL_TYPES[model_type] = name


def architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def architecture_of(raw: dict) -> str:
    """The registry key named by a config.json: ``architectures[0]``, else ``model_type``."""
    _ensure_builtin()
    archs = raw.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        name = archs[0]
    elif isinstance(raw.get("model_type"), str) and raw["model_type"] in _MODEL_TYPES:
        name = _MODEL_TYPES[raw["model_type"]]
    else:
        raise ConfigError("config.json names no architecture (keys 'architectures' / 'model_type'); "
                          f"registered: {architectures()}")
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not registered; registered: {architectures()}")
    return name


def resolve(raw_or_path):
    """(architecture name, typed config, ModelSpec) for a config dict or a model folder."""
    raw = read_config_json(raw_or_path) if isinstance(raw_or_path, str) else raw_or_path
    name = architecture_of(raw)
    config_cls, build_spec = _ARCHITECTURES[name]
    cfg = config_cls.from_dict(raw)
    return name, cfg, build_spec(cfg)


def spec_of_config(cfg):
    """ModelSpec of an already typed config (its class says which architecture it is)."""
    _ensure_builtin()
    for name, (config_cls, build_spec) in _ARCHITECTURES.items():
        if type(cfg) is config_cls:
            return build_spec(cfg)
    raise ConfigError(f"no registered architecture uses config class {type(cfg).__name__}")


def register_part(kind: str, name: str, cls: type) -> None:
    if kind not in _PARTS:
        raise KeyError(f"unknown part kind {kind!r}; kinds: {sorted(_PARTS)}")
    _PARTS[kind][name] = cls


def build_part(kind: str, spec) -> Any:
    """Instantiates ``spec.kind`` of the given kind with ``spec.params``."""
    _ensure_builtin()
    table = _PARTS[kind]
    if spec.kind not in table:
        raise KeyError(f"no {kind} named {spec.kind!r}; registered: {sorted(table)}")
    return table[spec.kind](**spec.params)


_builtin_done = False


def _ensure_builtin() -> None:
    global _builtin_done
    if _builtin_done:
        return
    _builtin_done = True
    from . import parts  # noqa: F401  registers the built-in parts
    from .models import qwen2_moe  # noqa: F401  registers the architecture
