"""Registries: architecture name -> (configuration class, model builder), and part
name -> part class for mixers, feed-forwards, norms and position encodings.

A model is never chosen by an ``if`` on its name: ``config.json`` names the
architecture, the architecture's builder reads its typed configuration and asks the
part registries for the parts each layer names.  Code outside this package can add to
every registry (a test registers a toy mixer and a toy architecture this way).
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

from .config.model_config import ConfigError, read_config_json

_ARCHITECTURES: Dict[str, Tuple[type, Callable]] = {}
_PARTS: Dict[str, Dict[str, type]] = {"mixer": {}, "ffn": {}, "norm": {}, "position": {}}

#: when config.json has no "architecture" key (a folder written with the upstream
#: project's field names only) this one is meant: it is the only model upstream has.
DEFAULT_ARCHITECTURE = "gqa_mtp_transformer"


def register_architecture(name: str, config_cls: type, builder: Callable) -> None:
    """``builder(config) -> ModelSpec``-like object understood by ``engine.ModelRunner``."""
    _ARCHITECTURES[name] = (config_cls, builder)


def architecture(name: str):
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture {name!r}; registered: {sorted(_ARCHITECTURES)}")
    return _ARCHITECTURES[name]


def architectures():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def register_part(kind: str, name: str, cls: type) -> None:
    if kind not in _PARTS:
        raise KeyError(f"part kind must be one of {sorted(_PARTS)}, got {kind!r}")
    _PARTS[kind][name] = cls


def part(kind: str, name: str) -> type:
    _ensure_builtin()
    try:
        return _PARTS[kind][name]
    except KeyError:
        raise ConfigError(f"unknown {kind} {name!r}; registered: {sorted(_PARTS.get(kind, {}))}") from None


def config_from_folder(folder: str):
    """Read ``config.json`` and return the typed configuration of its architecture."""
    raw = read_config_json(folder)
    return config_from_dict(raw)


def config_from_dict(raw: dict):
    name = raw.get("architecture", DEFAULT_ARCHITECTURE)
    cfg_cls, _ = architecture(name)
    return cfg_cls.from_dict(raw)


def build_model(cfg):
    """The model description (layers made of parts, schedule, heads) for a configuration."""
    _, builder = architecture(cfg.architecture)
    return builder(cfg)


_builtin_done = False


def _ensure_builtin():
    global _builtin_done
    if _builtin_done:
        return
    _builtin_done = True
    from . import parts as _parts  # noqa: F401  (registers the built-in parts)
    from . import models as _models  # noqa: F401  (registers the built-in architecture)
