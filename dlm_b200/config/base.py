"""Typed configuration helpers shared by every architecture's config class.

A config class is a dataclass whose fields carry the key names of the
architecture's own ``config.json``.  ``read_config_json`` only finds and parses
the file; which class interprets it is decided by the architecture registry.
"""
from __future__ import annotations

import json
import os
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot describe a runnable model (mirrors the
    reference's ``InvalidConfig``, src/error.rs:12-87)."""


def read_config_json(path: str) -> dict[str, Any]:
    """Read ``config.json`` from a model folder (or the file itself) and merge
    the EOS ids of a neighbouring ``generation_config.json`` the way the
    reference does (src/model/config.rs:366-421)."""
    cfg_path = os.path.join(path, "config.json") if os.path.isdir(path) else path
    if not os.path.isfile(cfg_path):
        raise ConfigError(f"no config.json at {cfg_path!r}")
    try:
        with open(cfg_path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{cfg_path}: not valid JSON ({e})") from e
    if not isinstance(raw, dict):
        raise ConfigError(f"{cfg_path}: top level must be a JSON object")
    gen_path = os.path.join(os.path.dirname(cfg_path), "generation_config.json")
    if os.path.isfile(gen_path):
        try:
            with open(gen_path, "r", encoding="utf-8") as f:
                gen = json.load(f)
            extra = gen.get("eos_token_id")
            if extra is not None:
                ids = eos_list(raw.get("eos_token_id"))
                for t in eos_list(extra):
                    if t not in ids:
                        ids.append(t)
                raw["eos_token_id"] = ids
        except (json.JSONDecodeError, AttributeError):
            pass  # an unreadable generation_config.json never blocks loading
    return raw


def eos_list(v: Any) -> list[int]:
    """``eos_token_id`` is one id or a list (src/model/config.rs:277-282)."""
    if v is None:
        return []
    if isinstance(v, bool):
        raise ConfigError("eos_token_id must be an integer or a list of integers")
    if isinstance(v, int):
        return [v]
    if isinstance(v, (list, tuple)) and all(isinstance(t, int) and not isinstance(t, bool) for t in v):
        return list(v)
    raise ConfigError("eos_token_id must be an integer or a list of integers")


def require_int(raw: dict, key: str, *, minimum: int = 1) -> int:
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks required key {key!r}")
    return as_int(raw[key], key, minimum=minimum)


def as_int(v: Any, key: str, *, minimum: int | None = None) -> int:
    if isinstance(v, bool) or not isinstance(v, int):
        if isinstance(v, float) and v.is_integer():
            v = int(v)
        else:
            raise ConfigError(f"{key} must be an integer, got {v!r}")
    if minimum is not None and v < minimum:
        raise ConfigError(f"{key} must be >= {minimum}, got {v}")
    return v


def as_float(v: Any, key: str) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{key} must be a number, got {v!r}")
    return float(v)


def as_bool(v: Any, key: str) -> bool:
    if not isinstance(v, bool):
        raise ConfigError(f"{key} must be true or false, got {v!r}")
    return v
