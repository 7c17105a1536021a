"""Typed configurations, the architecture-independent model description and
the architecture registry."""
from .qwen3 import ConfigError, Qwen3Config
from .registry import (ModelFamily, family_by_kind, parse_config, read_config, register,
                       resolve, unregister)
from .spec import CacheNeed, LayerRun, LayerSpec, ModelSpec, PartSpec

__all__ = ["ConfigError", "Qwen3Config", "ModelFamily", "family_by_kind", "parse_config",
           "read_config", "register", "resolve", "unregister", "CacheNeed", "LayerRun",
           "LayerSpec", "ModelSpec", "PartSpec"]
