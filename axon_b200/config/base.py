"""Typed model configurations and the registry of architectures.

A configuration is read from the keys of an architecture's own ``config.json``
and nothing else: every size and constant the model code uses comes from here.
The registry maps an architecture name (``architectures[0]`` or ``model_type``
of ``config.json``) to its configuration class and to the function that turns
a configuration into a :class:`axon_b200.parts.spec.ModelSpec`.

The resolution rule follows the reference's ``arch_of``
(src/safetensors.rs:437-463): ``model_type`` decides when present, else
``architectures[0]``; an unknown name is an error that lists what is known.
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, fields
from typing import Any, Callable, ClassVar, Dict, Mapping, Optional, Tuple, Type


class ConfigError(ValueError):
    """A config.json that this engine cannot run; the message says why."""


def whole_number(cfg: Mapping[str, Any], key: str, default: Optional[int] = None,
                 minimum: int = 1) -> Optional[int]:
    """``cfg[key]`` as a whole number >= ``minimum``.

    JSON numbers like ``2.0`` are accepted, ``2.5``, booleans, strings and
    negatives are not (reference: ``cfg_u32``, src/safetensors.rs:466-474;
    positivity checks src/model.rs:1283-1292).
    """
    v = cfg.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json {key} = {v!r} is not a whole number")
    if isinstance(v, float):
        if not math.isfinite(v) or v != int(v):
            raise ConfigError(f"config.json {key} = {v!r} is not a whole number")
        v = int(v)
    if v < minimum or v > 0xFFFFFFFF:
        raise ConfigError(f"config.json {key} = {v} must be a whole number >= {minimum}")
    return v


def real_number(cfg: Mapping[str, Any], key: str, default: Optional[float] = None) -> Optional[float]:
    """``cfg[key]`` as a finite float (reference: ``cfg_f64``, src/safetensors.rs:476-485)."""
    v = cfg.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"config.json {key} = {v!r} is not a number")
    return float(v)


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration."""

    #: the name under which the architecture is registered
    architecture: ClassVar[str] = ""
    #: ``model_type`` strings that select this architecture
    model_types: ClassVar[Tuple[str, ...]] = ()

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "ModelConfig":  # pragma: no cover - abstract
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        """The ``config.json`` that reads back as this configuration."""
        d: Dict[str, Any] = {f.name: getattr(self, f.name) for f in fields(self)}
        d["architectures"] = [self.architecture]
        if self.model_types:
            d["model_type"] = self.model_types[0]
        return d


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Type[ModelConfig]
    build_spec: Callable[[ModelConfig], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(config_cls: Type[ModelConfig], build_spec: Callable[[Any], Any]) -> None:
    """Make an architecture known: its name, its ``model_type`` strings, its
    configuration class and the function ``config -> ModelSpec``."""
    name = config_cls.architecture
    if not name:
        raise ValueError("a configuration class must name its architecture")
    _ARCHITECTURES[name] = Architecture(name, config_cls, build_spec)
    for mt in config_cls.model_types:
        _MODEL_TYPES[mt] = name


def known_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def architecture_of(cfg: Mapping[str, Any]) -> Architecture:
    """The registered architecture a ``config.json`` dictionary names."""
    if not isinstance(cfg, Mapping):
        raise ConfigError("config.json is not a JSON object")
    mt = cfg.get("model_type") or ""
    archs = cfg.get("architectures") or []
    hf = archs[0] if isinstance(archs, list) and archs and isinstance(archs[0], str) else ""
    if isinstance(mt, str) and mt in _MODEL_TYPES:
        return _ARCHITECTURES[_MODEL_TYPES[mt]]
    if (not mt) and hf in _ARCHITECTURES:
        return _ARCHITECTURES[hf]
    if mt and hf in _ARCHITECTURES and mt not in _MODEL_TYPES:
        # model_type decides when present (reference rule), and it is unknown
        pass
    shown = mt if mt else hf
    raise ConfigError(
        f"model_type '{shown}' is not supported ({', '.join(known_architectures())})")


def config_from_dict(cfg: Mapping[str, Any]) -> ModelConfig:
    return architecture_of(cfg).config_cls.from_dict(cfg)


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            cfg = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{folder}: no config.json") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not JSON ({e})") from None
    if not isinstance(cfg, dict):
        raise ConfigError(f"{path}: config.json is not a JSON object")
    return cfg


def load_config(folder: str) -> ModelConfig:
    """Read ``folder/config.json`` into the typed configuration of its architecture."""
    return config_from_dict(read_config_json(folder))


def write_config_json(folder: str, config: ModelConfig) -> None:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1, sort_keys=True)
        f.write("\n")
