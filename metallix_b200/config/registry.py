"""One registry from an architecture's name to its model family.

The reference has no ``architectures``-keyed table: each adapter gates on
``model_type`` (``crates/models/qwen/src/lib.rs:91-98``) and the serve registry
names the adapter by kind, ``"qwen"`` (``crates/app/cli/src/serve_registry.rs:32-99``).
Here one table answers all three spellings, and a new family is one
``register`` call with a configuration class that can parse its own
``config.json`` and describe itself as a ``ModelSpec``.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Type

from .qwen3 import ConfigError, Qwen3Config


@dataclass(frozen=True)
class ModelFamily:
    """What the engine needs of a family: how to read its configuration.

    ``config_class`` must offer ``from_dict(raw)``, ``to_dict()``,
    ``to_model_spec()``, ``tensor_shapes()``, ``ignored_tensors()`` and
    ``norm_tensor(name)``.
    """

    architecture: str
    model_type: str
    kind: str
    config_class: Type


_BY_ARCHITECTURE: Dict[str, ModelFamily] = {}
_BY_MODEL_TYPE: Dict[str, ModelFamily] = {}
_BY_KIND: Dict[str, ModelFamily] = {}


def register(family: ModelFamily) -> None:
    for table, key in ((_BY_ARCHITECTURE, family.architecture),
                       (_BY_MODEL_TYPE, family.model_type), (_BY_KIND, family.kind)):
        if key in table and table[key] is not family:
            raise ValueError(f"{key!r} is already registered")
        table[key] = family


def unregister(family: ModelFamily) -> None:
    for table, key in ((_BY_ARCHITECTURE, family.architecture),
                       (_BY_MODEL_TYPE, family.model_type), (_BY_KIND, family.kind)):
        if table.get(key) is family:
            del table[key]


def family_by_kind(kind: str) -> ModelFamily:
    if kind not in _BY_KIND:
        raise ConfigError("UnsupportedModelType", f"no model family of kind {kind!r}; "
                          f"known kinds: {sorted(_BY_KIND)}")
    return _BY_KIND[kind]


def resolve(raw: Mapping[str, Any]) -> ModelFamily:
    """The family a ``config.json`` names, by ``architectures[0]`` or ``model_type``."""
    architectures = raw.get("architectures") or []
    if not isinstance(architectures, list):
        raise ConfigError("Json", "architectures must be a list of names")
    for name in architectures:
        if name in _BY_ARCHITECTURE:
            return _BY_ARCHITECTURE[name]
    model_type = raw.get("model_type", "")
    if model_type in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[model_type]
    raise ConfigError(
        "UnsupportedModelType",
        f"architectures {architectures!r} / model_type {model_type!r}; "
        f"this engine builds {sorted(_BY_ARCHITECTURE)}")


def parse_config(raw: Mapping[str, Any]):
    """Typed configuration of whatever family ``raw`` names."""
    return resolve(raw).config_class.from_dict(raw)


def read_config(model_dir: str):
    """Reads ``<model_dir>/config.json``; stop ids of ``generation_config.json``
    are added to the configuration's own (``chat-format/src/lib.rs:207-253``)."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isdir(model_dir):
        raise ConfigError("NotDirectory", model_dir)
    try:
        with open(path, "r", encoding="utf-8") as handle:
            raw = json.load(handle)
    except OSError as error:
        raise ConfigError("ReadConfig", f"{path}: {error}") from None
    except json.JSONDecodeError as error:
        raise ConfigError("Json", f"{path}: {error}") from None
    if not isinstance(raw, dict):
        raise ConfigError("Json", f"{path} must hold one JSON object")
    config = parse_config(raw)
    extra = _generation_eos(os.path.join(model_dir, "generation_config.json"))
    if extra and hasattr(config, "eos_token_ids"):
        merged = tuple(dict.fromkeys(tuple(config.eos_token_ids) + extra))
        config = dataclasses.replace(config, eos_token_ids=merged)
    return config


def _generation_eos(path: str) -> tuple:
    try:
        with open(path, "r", encoding="utf-8") as handle:
            eos = json.load(handle).get("eos_token_id")
    except (OSError, json.JSONDecodeError, AttributeError):
        return ()
    if isinstance(eos, int) and not isinstance(eos, bool):
        return (eos,)
    if isinstance(eos, list):
        return tuple(e for e in eos if isinstance(e, int) and not isinstance(e, bool))
    return ()


QWEN3 = ModelFamily(architecture=Qwen3Config.ARCHITECTURE, model_type=Qwen3Config.MODEL_TYPE,
                    kind="qwen", config_class=Qwen3Config)
register(QWEN3)
