"""Architecture-independent description of a decoder.

A model family turns its own ``config.json`` into a :class:`ModelSpec`: plain
data that says, layer by layer, which mixer, feed-forward, norms and position
encoding to build, with every size and constant as a parameter, and in which
order the layers run. Nothing below this file knows a family's name; the
parts are built from the spec by kind (``metallix_b200.parts.registry``).

The reference engine hard-codes one arrangement in
``crates/models/qwen/src/forward.rs:1856-1922`` (pre-norm attention, residual,
pre-norm SwiGLU, residual). Here the same arrangement is one value of
``LayerSpec.block``, and the loop over layers (``forward.rs:1562-1582``) is the
``order`` list.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One buildable part: a registered ``kind`` and its parameters.

    ``params`` holds sizes, constants and tensor names; a part reads nothing
    else. Two parts of the same kind with different params may sit in
    different layers of one model.
    """

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: what it is made of and how the pieces are arranged."""

    name: str  # tensor-name prefix, e.g. "model.layers.3"
    block: PartSpec  # the arrangement (pre-norm residual, ...)
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution order.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named twice; its
    second run then needs a cache entry of its own, any unused index).
    ``cache`` is the cache entry the mixer uses; by default a layer owns the
    entry with its own index. ``write_cache=False`` lets a layer read the
    entry another layer has written in the same step without writing to it.
    """

    layer: int
    cache: Optional[int] = None
    write_cache: bool = True

    def cache_entry(self) -> int:
        return self.layer if self.cache is None else self.cache


@dataclass(frozen=True)
class CacheNeed:
    """What one cache entry needs from the cache manager.

    ``kind == "kv_pages"``: keys and values of ``kv_heads`` heads of width
    ``head_dim`` for every position (``window is None``) or for the last
    ``window`` positions. ``kind == "state"``: ``state_shape`` values of fixed
    size per request, zeroed when the request is admitted. ``kind == "none"``:
    the mixer keeps nothing between steps.
    """

    kind: str
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: str = "float32"

    def group_key(self) -> tuple:
        return (self.kind, self.kv_heads, self.head_dim, self.window,
                tuple(self.state_shape), self.state_dtype)


@dataclass(frozen=True)
class ModelSpec:
    """Everything the engine needs to build a decoder, and nothing family-specific."""

    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[LayerRun, ...]
    final_norm: PartSpec
    head: PartSpec

    def num_cache_entries(self) -> int:
        return max(run.cache_entry() for run in self.order) + 1

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        written = set()
        for run in self.order:
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"order names layer {run.layer}, the model has {len(self.layers)}")
            entry = run.cache_entry()
            if entry < 0:
                raise ValueError(f"order names cache entry {entry}")
            if run.write_cache:
                written.add(entry)
            elif entry not in written:
                raise ValueError(
                    f"layer {run.layer} reads cache entry {entry} before any layer has written it")
