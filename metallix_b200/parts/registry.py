"""Registry of buildable parts and what every part may rely on.

A part is built from a ``PartSpec`` (kind + parameters), a ``WeightStore``
(tensors by name) and a ``Runtime`` (device, compute dtype, capacity). It
never learns which model it is in. Five categories exist: ``mixer``,
``feed_forward``, ``norm``, ``position`` and ``block``; plus ``embedding`` and
``head`` at the model's two ends. Registering a new kind is one call::

    register_part("mixer", "my_mixer", lambda spec, weights, runtime: MyMixer(...))

and a model spec that names ``PartSpec("my_mixer", {...})`` then builds it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..config.spec import CacheNeed, PartSpec

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_BUILDERS: Dict[Tuple[str, str], Callable] = {}


def register_part(category: str, kind: str, builder: Callable, replace: bool = False) -> None:
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")
    if (category, kind) in _BUILDERS and not replace:
        raise ValueError(f"{category} part {kind!r} is already registered")
    _BUILDERS[(category, kind)] = builder


def unregister_part(category: str, kind: str) -> None:
    _BUILDERS.pop((category, kind), None)


def build_part(category: str, spec: Optional[PartSpec], weights: "WeightStore", runtime: "Runtime"):
    if spec is None:
        return None
    builder = _BUILDERS.get((category, spec.kind))
    if builder is None:
        known = sorted(kind for cat, kind in _BUILDERS if cat == category)
        raise KeyError(f"no {category} part of kind {spec.kind!r}; registered: {known}")
    return builder(spec, weights, runtime)


@dataclass
class Runtime:
    """What the engine tells every part it builds."""

    device: torch.device
    dtype: torch.dtype          # compute dtype: torch.bfloat16 or torch.float32
    max_positions: int          # longest context the engine will run
    gemm_backend: str = "auto"  # how bfloat16 matrix products run: auto | tcgen05 | cublas | simple


class WeightStore:
    """Tensors by name, as stored; remembers which names parts have taken."""

    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self._tensors = tensors
        self.taken: List[str] = []

    def take(self, name: str) -> torch.Tensor:
        if name not in self._tensors:
            raise KeyError(f"weight {name!r} is not in the checkpoint")
        self.taken.append(name)
        return self._tensors[name]

    def has(self, name: str) -> bool:
        return name in self._tensors


@dataclass
class CacheView:
    """What one layer run sees of the cache.

    For ``kv_pages`` entries: ``pool`` is this entry's
    ``[pages, 2, kv_heads, page_tokens, head_dim]`` tensor, ``block_tables``
    ``[requests, max_pages]`` and ``slots`` ``[tokens]`` belong to the entry's
    group (``slots`` is None when the run may not write). For ``state``
    entries: ``state`` is ``[request_slots, *state_shape]``, indexed by
    ``StepContext.request_slots``.
    """

    need: CacheNeed
    pool: Optional[torch.Tensor] = None
    block_tables: Optional[torch.Tensor] = None
    slots: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None
    write: bool = True


@dataclass
class StepContext:
    """One step's batch, as the parts see it. Tokens of all requests are
    packed one after another; request row r owns tokens
    ``request_offsets[r] .. request_offsets[r + 1] - 1`` at consecutive
    positions starting at ``request_positions[r]``."""

    device: torch.device
    dtype: torch.dtype
    num_tokens: int
    num_requests: int
    positions: torch.Tensor            # int32 [tokens], absolute position of each token
    token_request: torch.Tensor        # int32 [tokens], request row of each token
    request_slots: torch.Tensor        # int32 [requests], state slot of each request row
    request_offsets: List[int]         # host, [requests + 1]
    request_positions: List[int]       # host, first position of each row's tokens
    tile_request: torch.Tensor         # int32 [tiles], attention query tiles of every request
    tile_start: torch.Tensor
    tile_length: torch.Tensor
    # The same batch split by kind of request, for mixers with a kernel of
    # their own for single decoded tokens: tiles of the requests that bring
    # several tokens, and (token, request row) of those that bring one.
    # ``decode_token`` may hold negative entries (padding rows).
    multi_tiles: int = 0               # the first ``multi_tiles`` tiles belong to multi-token requests
    decode_token: Optional[torch.Tensor] = None    # int32 [decode rows]
    decode_request: Optional[torch.Tensor] = None  # int32 [decode rows]
    longest_context: int = 0           # upper bound of position + 1 over the decode rows
    longest_keys: int = 0              # upper bound of the keys a wide tile sees (0: no bound known, taken as few)
    # Tiles of up to 64 tokens over the multi-token requests, for the
    # tensor-core prompt kernel; longest keys first.
    wide_tile_request: Optional[torch.Tensor] = None
    wide_tile_start: Optional[torch.Tensor] = None
    wide_tile_length: Optional[torch.Tensor] = None
    extras: Dict[str, object] = field(default_factory=dict)
