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
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple

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
    # Read-only tensors that parts built from equal parameters may share
    # (tables of a position encoding, say), by a key of those parameters.
    shared: Dict[tuple, object] = field(default_factory=dict)


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

    def drop_taken(self, keep=()) -> None:
        """Forgets the tensors that parts have taken (except ``keep``), for an
        owner that hands its dictionary over: a part that stacked or cast a
        weight holds a copy, and the original's memory is wanted back while a
        large model is still being built."""
        for name in set(self.taken):
            if name not in keep:
                self._tensors.pop(name, None)


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
class StepPlan:
    """A step as the host knows it, handed to the parts that keep integers
    of their own for it (``prepare_step``): request row r brings
    ``counts[r]`` tokens at positions ``starts[r]`` onwards; rows from
    ``live`` on are padding of a captured graph (they bring a token that
    nothing may read or write). ``context_bound`` bounds position + 1 of every
    token. ``replayable``: the integers go into a captured graph that later
    steps of the same shape replay with other positions, so sizes of the
    arrays may depend on ``counts`` (and on the part's ``graph_key``) only, and
    bounds that kernels are launched with must be ``context_bound``, not
    what this one step needs."""

    counts: Sequence[int]
    starts: Sequence[int]
    live: int
    context_bound: int
    replayable: bool = False


@dataclass
class Prepared:
    """What a part's ``prepare_step(plan)`` returns. ``arrays``: int32 numpy
    arrays by name, which travel to the device with the step's other integers
    (one copy) and come back as device tensors under the same names;
    ``facts``: host values for the part's ``forward``; ``graph_key``: what,
    beyond the shape of the step, decides which kernels the part launches (two
    steps may share a captured graph only if it is equal)."""

    arrays: Dict[str, "object"] = field(default_factory=dict)
    facts: Dict[str, object] = field(default_factory=dict)
    graph_key: Hashable = None


@dataclass
class StepContext:
    """One step's batch, as the parts see it. Tokens of all requests are
    packed one after another; request row r owns tokens
    ``request_offsets[r] .. request_offsets[r + 1] - 1`` at consecutive
    positions starting at ``request_positions[r]``. The two host lists are
    None while a graph is captured or replayed: a part that needs them on the
    host cannot ride in a graph (it says ``graph_safe = False``).

    A part that needs integers of its own for a step (tile lists of an
    attention kernel, say) defines ``step_key`` (parts with the same key share
    one preparation) and ``prepare_step(plan) -> Prepared``; the engine calls
    it once per step and leaves the result, arrays on the device, in
    ``extras[step_key]``: a dict of the arrays and the facts by name."""

    device: torch.device
    dtype: torch.dtype
    num_tokens: int
    num_requests: int
    positions: torch.Tensor            # int32 [tokens], absolute position of each token
    token_request: torch.Tensor        # int32 [tokens], request row of each token
    request_slots: torch.Tensor        # int32 [requests], state slot of each request row
    request_offsets: Optional[List[int]]    # host, [requests + 1]
    request_positions: Optional[List[int]]  # host, first position of each row's tokens
    extras: Dict[str, object] = field(default_factory=dict)


def step_preparers(blocks) -> Dict[str, object]:
    """The parts of ``blocks`` that prepare integers for a step, one per
    ``step_key``."""
    found: Dict[str, object] = {}
    for block in blocks:
        for part in block_parts(block):
            key = getattr(part, "step_key", None)
            if key is not None and key not in found and hasattr(part, "prepare_step"):
                found[key] = part
    return found


def block_parts(block) -> List[object]:
    """Every part a block holds: what its ``parts()`` names (else its
    ``mixer``, ``feed_forward`` and the two norms), and what those parts name
    in turn through a ``parts()`` of their own (an attention mixer holds head
    norms and a position encoding)."""
    def own(holder):
        if hasattr(holder, "parts"):
            return [p for p in holder.parts() if p is not None]
        return []
    first = own(block) or [getattr(block, name) for name in
                           ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")
                           if getattr(block, name, None) is not None]
    found, queue = [], list(first)
    while queue:
        part = queue.pop(0)
        if any(part is other for other in found):
            continue
        found.append(part)
        queue.extend(own(part))
    return found


def graph_safe(part) -> bool:
    """Whether a part may ride in a captured graph: it launches the same work
    whatever the step's integers and the device's values are (no host reads).
    A mixer must say so (``graph_safe = True``); any other part is taken at
    its word only when it says no (``graph_safe = False``)."""
    return bool(getattr(part, "graph_safe", not hasattr(part, "cache_need")))
