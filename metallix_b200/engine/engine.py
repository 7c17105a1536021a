"""The engine: a model, its cache and the one step function.

``Engine.step`` takes a batch of (request, its next tokens) entries: portions
of prompts beside single decoded tokens, cut anywhere. It runs only those
tokens, as one packed batch, against the cache that earlier steps left, and
returns float32 logits at the wanted places. The reference runs prompt
portions and decode rows as separate forward passes
(crates/models/qwen/src/forward/paged.rs:570 and :741); here they share one.

Protocol per step, as in crates/core/engine/src/blocks.rs:17-45: everything is
checked first and nothing changes on a refusal; then pages are reserved for
every entry, the forward pass writes them, and the positions are committed. A
failure after the reservation rolls every entry of the step back.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache import PagedCache
from ..config import read_config
from ..parts.registry import Runtime, StepContext, StepPlan, step_preparers
from ..weights import load_tensors, random_tensors
from .model import DecoderModel

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}
STEP_GRAPHS = 32      # how many shapes of general steps keep a captured graph
STEP_GRAPH_TOKENS = 8192   # ... of steps up to this many tokens (a graph keeps its activations)
# A graph saves the launches of a step (some 250 kernels from Python, a
# millisecond or two of the host's time): worth it while the step itself is
# short. Steps whose matrix products alone would take longer than this at the
# rate below are launched kernel by kernel, which the device then hides.
STEP_GRAPH_SECONDS = 5e-3
DEVICE_FLOPS = 1.4e15      # a B200's sustained bfloat16 matrix rate
CONTEXT_BUCKET = 2048  # a captured graph serves contexts up to a power of two times this many positions


class StepError(ValueError):
    """A batch the step function refuses; nothing was changed."""


@dataclass
class StepEntry:
    """One request's share of a step: its next ``tokens`` and the indices
    among them (``want``) whose logits are asked for."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)
    # True: ``request`` is an id a scheduler has already admitted to the cache
    # manager; the step reserves and commits for it but neither admits nor
    # releases it.
    managed: bool = False


def resolve_dtype(dtype) -> torch.dtype:
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")
    return _DTYPES[dtype]


class Engine:
    def __init__(self, config, tensors: Dict[str, torch.Tensor], dtype="bfloat16",
                 page_tokens: int = 16, num_pages: Optional[int] = None,
                 max_tokens: Optional[int] = None, max_requests: int = 64,
                 max_context: Optional[int] = None, device="cuda:0", gemm_backend: str = "auto",
                 spec=None, cuda_graphs: bool = True, chained_launches: bool = True,
                 pool_bytes: Optional[int] = None, pool_fraction: Optional[float] = None,
                 consume_tensors: bool = False):
        """The cache pool is sized by the first of these that is given:
        ``num_pages``; ``max_tokens`` (positions all live requests may hold);
        ``pool_bytes``; ``pool_fraction`` of the device memory that is free
        once the weights are resident (what a large model on one GPU wants);
        else four contexts of up to 4,096 positions."""
        ops.require_cuda()
        self.chained_launches = bool(chained_launches)
        ops.set_chained_launches(self.chained_launches)
        self.config = config
        self.device = torch.device(device)
        self.dtype = resolve_dtype(dtype)
        self.spec = spec if spec is not None else config.to_model_spec()
        self.max_context = min(max_context or self.spec.max_positions, self.spec.max_positions)
        if self.dtype == torch.float32:
            # True 32-bit everywhere: no reduced-precision matrix mode for
            # anything torch may run on this path.
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
        self.runtime = Runtime(device=self.device, dtype=self.dtype, max_positions=self.max_context,
                               gemm_backend=gemm_backend)
        self.model = DecoderModel(self.spec, tensors, self.runtime, consume=consume_tensors)
        if num_pages is None and max_tokens is None and (pool_bytes is not None or pool_fraction is not None):
            if pool_bytes is None:
                if not 0.0 < pool_fraction <= 1.0:
                    raise ValueError(f"pool_fraction must lie in (0, 1], got {pool_fraction}")
                torch.cuda.empty_cache()   # what building the model freed goes back to the device first
                free, _ = torch.cuda.mem_get_info(self.device)     # the weights are on the device by now
                pool_bytes = int(free * pool_fraction)
            per_page = PagedCache.page_bytes(self.model.cache_needs(), page_tokens, self.dtype)
            num_pages = max(int(pool_bytes) // per_page, 1) if per_page else 1
        if num_pages is None:
            tokens = max_tokens if max_tokens is not None else min(self.max_context, 4096) * 4
            num_pages = -(-tokens // page_tokens)
        self.cache = PagedCache(self.model.cache_needs(), page_tokens, num_pages, max_requests,
                                self.dtype, self.device)
        self.manager = self.cache.manager
        from .decode_graph import DecodeGraphs
        self._preparers = step_preparers(self.model.blocks)   # parts with integers of their own per step
        self.graphs = DecodeGraphs(self) if cuda_graphs and DecodeGraphs.usable(self.model) else None
        # Graphs of general steps by shape (see _run). Such a graph is warmed
        # up and captured on a live step, which therefore runs more than once:
        # harmless where a step only writes pages (written again with the
        # same values), not where a part keeps state that a step advances.
        stateless = all(need is None or need.kind != "state" for need in self.cache.needs)
        self._step_graphs: Optional[Dict] = {} if self.graphs is not None and stateless else None
        self.replay_general_steps = True   # False: general steps are launched kernel by kernel (measurements)
        values = self.model.weight_bytes() / torch.empty((), dtype=self.dtype).element_size()
        self.step_graph_tokens = int(min(STEP_GRAPH_TOKENS, max(256, STEP_GRAPH_SECONDS * DEVICE_FLOPS / (2.0 * values))))
        self._shapes_seen: Dict = {}
        self._ids: Dict[Hashable, int] = {}   # request name -> manager id
        self._next_id = 1 << 40               # above any id a scheduler hands out
        self.steps = 0

    # ----------------------------------------------------------- construction
    @classmethod
    def from_folder(cls, model_dir: str, **options) -> "Engine":
        """A model folder (config.json + *.safetensors); the model class is
        chosen by config.json."""
        config = read_config(model_dir)
        device = options.get("device", "cuda:0")
        ops.require_cuda()
        tensors = load_tensors(model_dir, config, device=device)
        return cls(config, tensors, consume_tensors=True, **options)

    @classmethod
    def from_random(cls, config, seed: int, **options) -> "Engine":
        """Random weights from ``seed`` made directly on the device."""
        ops.require_cuda()
        dtype = resolve_dtype(options.get("dtype", "bfloat16"))
        name = "bfloat16" if dtype == torch.bfloat16 else "float32"
        tensors = random_tensors(config, seed, dtype=name, device=options.get("device", "cuda:0"))
        return cls(config, tensors, consume_tensors=True, **options)

    # ---------------------------------------------------------------- requests
    def live(self, request: Hashable) -> bool:
        return request in self._ids

    def context_length(self, request: Hashable) -> int:
        return self.manager.computed(self._ids[request]) if request in self._ids else 0

    def _rid(self, entry: StepEntry) -> Optional[int]:
        """The cache manager's id of an entry's request, None if not admitted."""
        if entry.managed:
            return int(entry.request)
        return self._ids.get(entry.request)

    def release(self, request: Hashable) -> None:
        """Gives back everything the request holds."""
        if request in self._ids:
            self.manager.release(self._ids.pop(request))

    def fork(self, parent: Hashable, child: Hashable) -> None:
        """A new request ``child`` that has ``parent``'s whole context in the
        cache without computing it again: full pages are shared, the partly
        filled last page and the state are copied on the device (the
        reference's reference-counted blocks, crates/core/engine/src/manager.rs:614-628,
        749-763). Both go on independently afterwards; either may end first."""
        if parent not in self._ids:
            raise KeyError(f"request {parent!r} is not live")
        if child in self._ids:
            raise ValueError(f"request {child!r} is already live")
        rid = self._next_id
        self.cache.fork(self._ids[parent], rid)
        self._ids[child] = rid
        self._next_id += 1

    def release_all(self) -> None:
        for request in list(self._ids):
            self.release(request)

    # -------------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs one batch. Returns float32 logits ``[wanted, vocab]`` on the
        device in the order of the entries and of each entry's ``want``, or
        None if nothing is wanted. The tensor may be a view of a buffer that
        the next step overwrites: read it before stepping again. Call
        ``check()`` after reading results."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(**e) for e in entries]
        ops.set_chained_launches(self.chained_launches)   # another engine may have chosen otherwise
        self._validate(entries)
        manager, fresh = self.manager, []
        try:
            for entry in entries:
                if self._rid(entry) is None:
                    self._ids[entry.request] = self._next_id
                    self._next_id += 1
                    manager.admit(self._ids[entry.request])
                    fresh.append(entry.request)
                rid = self._rid(entry)
                if manager.computed(rid) == 0:
                    self.cache.zero_state(manager.slot(rid))  # a sequence starts from zero state
                manager.reserve(rid, len(entry.tokens))
            logits = self._run_graph(entries) if self._all_decode(entries) else self._run(entries)
            for entry in entries:
                manager.commit(self._rid(entry), len(entry.tokens))
        except BaseException:
            for entry in entries:
                rid = self._rid(entry)
                if rid is None or not manager.has(rid):
                    continue
                if not entry.managed and entry.request in fresh:
                    manager.release(self._ids.pop(entry.request))
                else:
                    manager.rollback(rid)
            raise
        self.steps += 1
        return logits

    def _all_decode(self, entries: List[StepEntry]) -> bool:
        """Every request brings one token after earlier ones: a decode step,
        which runs as a captured graph."""
        if self.graphs is None or self.graphs.bucket_for(len(entries)) is None:
            return False
        return all(len(e.tokens) == 1 and self.manager.computed(self._rid(e)) > 0 for e in entries)

    def _run_graph(self, entries: List[StepEntry]) -> Optional[torch.Tensor]:
        manager = self.manager
        rows, wanted = [], []
        for row, entry in enumerate(entries):
            rid = self._rid(entry)
            rows.append((rid, int(entry.tokens[0]), manager.computed(rid), manager.slot(rid)))
            if len(entry.want):
                wanted.append(row)
        logits = self.graphs.run(rows)
        if not wanted:
            return None
        if len(wanted) == len(entries):
            return logits
        return logits[torch.tensor(wanted, device=self.device)]

    # ------------------------------------------------- a decode step run ahead
    def ahead_possible(self) -> bool:
        """Whether a decode step may be launched before the tokens it runs on
        have reached the host, to be confirmed or dropped afterwards: only
        when dropping leaves no trace, i.e. every cache entry is pages without
        a window (a page written in vain is simply written again) and no part
        keeps state of its own."""
        if self.graphs is None:
            return False
        return all(need is None or (need.kind == "kv_pages" and not need.window) or need.kind == "none"
                   for need in self.cache.needs)

    def launch_ahead(self, requests: Sequence[int], fed_ids: torch.Tensor) -> Optional[torch.Tensor]:
        """One decoded token for each of the managed ``requests``, the token
        ids taken from ``fed_ids`` on the device (int32, same order). Reserves
        the positions and launches; commits nothing. Returns the logits, or
        None (and changes nothing) where such a step cannot run now.
        ``commit_ahead`` or ``drop_ahead`` must follow."""
        manager = self.manager
        if not self.ahead_possible() or self.graphs.bucket_for(len(requests)) is None:
            return None
        for rid in requests:
            if (not manager.has(rid) or manager.computed(rid) == 0 or manager.reserved(rid) != manager.computed(rid)
                    or manager.computed(rid) + 1 > self.max_context):
                return None
        if not manager.fits([(rid, 1) for rid in requests]):
            return None
        for rid in requests:
            manager.reserve(rid, 1)
        try:
            rows = [(rid, 0, manager.computed(rid), manager.slot(rid)) for rid in requests]
            return self.graphs.run(rows, fed_ids=fed_ids)
        except BaseException:
            self.drop_ahead(requests)
            raise

    def commit_ahead(self, requests: Sequence[int]) -> None:
        for rid in requests:
            self.manager.commit(rid, 1)
        self.steps += 1

    def drop_ahead(self, requests: Sequence[int]) -> None:
        """The step launched ahead does not count: its positions are given
        back (what it wrote is written again by the step that replaces it)."""
        manager = self.manager
        for rid in requests:
            if manager.has(rid) and manager.reserved(rid) != manager.computed(rid):
                manager.rollback(rid)

    def check(self) -> None:
        """Raises if any kernel since the last check refused its input
        (synchronises the device)."""
        ops.check_status(self.device)

    def check_later(self) -> None:
        """Queues the read of the kernels' status behind what has been
        launched; ``check_now`` raises on it after the caller has synchronised
        anyway (by reading tokens or logits)."""
        ops.fetch_status(self.device)

    def check_now(self) -> None:
        ops.raise_status(self.device)

    # ------------------------------------------------------------------ pieces
    def _validate(self, entries: List[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        asks = []
        new_requests = 0
        vocab = self.spec.vocab_size
        for entry in entries:
            if entry.request in seen:
                raise StepError(f"request {entry.request!r} appears twice in one step")
            seen.add(entry.request)
            count = len(entry.tokens)
            if count == 0:
                raise StepError(f"request {entry.request!r} brings no tokens")
            if count == 1:   # a decoded token: no array needed
                token = entry.tokens[0]
                if isinstance(token, bool) or not isinstance(token, (int, np.integer)) or not 0 <= token < vocab:
                    raise StepError(f"request {entry.request!r}: token ids must lie in 0..{vocab - 1}")
            else:
                tokens = np.asarray(entry.tokens)
                if tokens.dtype.kind not in "iu" or tokens.min() < 0 or tokens.max() >= vocab:
                    raise StepError(f"request {entry.request!r}: token ids must lie in 0..{vocab - 1}")
            for index in entry.want:
                if not 0 <= index < count:
                    raise StepError(f"request {entry.request!r}: want index {index} outside its {count} tokens")
            rid = self._rid(entry)
            if entry.managed and not self.manager.has(rid):
                raise StepError(f"request {entry.request!r} is not admitted to the cache manager")
            held = self.manager.computed(rid) if rid is not None else 0
            if rid is not None and self.manager.reserved(rid) != held:
                raise StepError(f"request {entry.request!r} has uncommitted positions")
            if held + count > self.max_context:
                raise StepError(f"request {entry.request!r}: {held + count} positions exceed the "
                                f"context limit of {self.max_context}")
            if rid is None:
                new_requests += 1
                asks.append((-1 - new_requests, count))  # an unknown id is costed from zero
            else:
                asks.append((rid, count))
        if new_requests > self.manager.free_slots():
            raise StepError(f"{new_requests} new requests but {self.manager.free_slots()} free request slots")
        if not self.manager.fits(asks):
            free = [self.manager.free_pages(g) for g in range(self.manager.num_groups())]
            raise StepError(f"out of cache pages: the step does not fit (free pages per group: {free})")

    def context_bucket(self, longest: int) -> int:
        """The bound a captured graph is laid out for when its longest request
        holds ``longest`` positions: 2,048 times a power of two, at most the
        engine's limit. Block tables, split counts and scratch of a graph
        follow the contexts that are live, not the longest one allowed."""
        bound = CONTEXT_BUCKET
        while bound < longest:
            bound *= 2
        return min(bound, self.max_context)

    def _run(self, entries: List[StepEntry]) -> Optional[torch.Tensor]:
        """A general step: any mix of portions of prompts and decoded tokens.

        The step's integers (token ids, positions, block tables, slots, and
        what the parts prepare for themselves, such as the attention's tile
        lists) go to the device as one packed buffer. A step whose *shape*
        (the token counts of its entries, how many logits are wanted, the
        bucket of its longest context, and what the parts say decides their
        launches) has been seen before replays a CUDA graph captured for that
        shape, with its integers copied into the graph's buffer: a prompt cut
        into equal portions, or the same batch again, then costs one launch
        instead of some two hundred."""
        manager, cache = self.manager, self.cache
        page_tokens = cache.page_tokens
        counts = [len(e.tokens) for e in entries]
        total = sum(counts)
        rows = len(entries)
        offsets = np.zeros(rows + 1, dtype=np.int64)
        np.cumsum(counts, out=offsets[1:])
        token_ids = np.empty(total, dtype=np.int32)
        positions = np.empty(total, dtype=np.int32)
        token_request = np.empty(total, dtype=np.int32)
        request_slots = np.empty(rows, dtype=np.int32)
        starts, wanted = [], []
        group_tables = [[] for _ in cache.groups]
        for row, entry in enumerate(entries):
            rid = self._rid(entry)
            begin, count = int(offsets[row]), counts[row]
            start = manager.computed(rid)
            starts.append(start)
            token_ids[begin:begin + count] = np.asarray(entry.tokens, dtype=np.int32)
            positions[begin:begin + count] = np.arange(start, start + count, dtype=np.int32)
            token_request[begin:begin + count] = row
            request_slots[row] = manager.slot(rid)
            wanted.extend(begin + index for index in entry.want)
            for group in cache.groups:
                group_tables[group.index].append(manager.table(rid, group.index))
        longest = max(start + count for start, count in zip(starts, counts))
        plan = StepPlan(counts, starts, rows, longest)
        prepared = {key: part.prepare_step(plan) for key, part in self._preparers.items()}
        # A step that may be replayed as a graph has block tables as wide as
        # its context bucket, so that its buffer has one layout whatever the
        # contexts inside the bucket are.
        bound = self.context_bucket(longest)
        shape_key = (tuple(counts), len(wanted), bound, tuple(p.graph_key for p in prepared.values()))
        graphed = self._step_graphs is not None and self.replay_general_steps and total <= self.step_graph_tokens and (
            shape_key in self._step_graphs or self._shapes_seen.get(shape_key, 0) >= 1)
        if graphed:   # the parts' integers and bounds for every step of this shape
            plan = StepPlan(counts, starts, rows, bound, replayable=True)
            prepared = {key: part.prepare_step(plan) for key, part in self._preparers.items()}
        # One packed int32 buffer, one copy to the device.
        pieces = [token_ids, positions, token_request, request_slots, np.asarray(wanted, dtype=np.int32)]
        shapes = [None] * len(pieces)
        for key, result in prepared.items():
            for array in result.arrays.values():
                pieces.append(np.ascontiguousarray(array, dtype=np.int32).reshape(-1))
                shapes.append(tuple(array.shape) if array.ndim > 1 else None)
        first_table = len(pieces)
        full_width = -(-bound // page_tokens)
        for group in cache.groups:
            tables = group_tables[group.index]
            width = full_width if graphed else max(len(t) for t in tables)
            table = np.full((rows, width), -1, dtype=np.int32)
            slots = np.empty(total, dtype=np.int32)
            for row, pages in enumerate(tables):
                table[row, :len(pages)] = pages
                begin, count = int(offsets[row]), counts[row]
                where = positions[begin:begin + count]
                slots[begin:begin + count] = table[row, where // page_tokens] * page_tokens + where % page_tokens
            pieces.extend([table.reshape(-1), slots])
            shapes.extend([(rows, width), None])
        sizes = [p.size for p in pieces]
        packed = torch.empty(sum(sizes), dtype=torch.int32, pin_memory=True)
        packed_np = packed.numpy()
        cursor = 0
        for piece, size in zip(pieces, sizes):
            packed_np[cursor:cursor + size] = piece
            cursor += size
        self._keep = packed  # the pinned buffer must outlive the asynchronous copy

        def forward(on_device: torch.Tensor) -> Optional[torch.Tensor]:
            views, cursor = [], 0
            for size, shape in zip(sizes, shapes):
                view = on_device[cursor:cursor + size]
                views.append(view.view(shape) if shape is not None else view)
                cursor += size
            d_ids, d_positions, d_token_request, d_request_slots, d_wanted = views[:5]
            extras, at = {}, 5
            for key, result in prepared.items():
                extras[key] = dict(result.facts)
                for name in result.arrays:
                    extras[key][name] = views[at]
                    at += 1
            tables = {g.index: views[first_table + 2 * g.index] for g in cache.groups}
            slots = {g.index: views[first_table + 1 + 2 * g.index] for g in cache.groups}
            ctx = StepContext(
                device=self.device, dtype=self.dtype, num_tokens=total, num_requests=rows,
                positions=d_positions, token_request=d_token_request, request_slots=d_request_slots,
                # inside a graph the host's view of one step would be baked in for all
                request_offsets=None if graphed else [int(v) for v in offsets],
                request_positions=None if graphed else starts, extras=extras)
            return self.model.forward(
                d_ids, ctx, lambda entry, write: cache.view(entry, write, tables, slots),
                d_wanted if wanted else None)

        if not graphed:
            if self._step_graphs is not None and self.replay_general_steps:
                self._shapes_seen[shape_key] = self._shapes_seen.get(shape_key, 0) + 1
                if len(self._shapes_seen) > 4096:
                    self._shapes_seen.clear()
            return forward(packed.to(self.device, non_blocking=True))
        return self._replay_step(shape_key, packed, forward)

    def _replay_step(self, shape_key, packed: torch.Tensor, forward) -> Optional[torch.Tensor]:
        """Replays (after capturing it, the first time) the graph of a general
        step of this shape with the integers in ``packed``."""
        from .decode_graph import capture_quietly
        held = self._step_graphs.get(shape_key)
        if held is None:
            # A step of this shape has run before, kernel by kernel: libraries
            # and lazily loaded kernels have settled, the capture needs no
            # warm-up run of its own.
            static = packed.to(self.device)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            pool = self.graphs.pool if self.graphs is not None else None
            with capture_quietly(graph, pool):
                logits = forward(static)
            if self.graphs is not None and self.graphs.pool is None:
                self.graphs.pool = graph.pool()
            held = {"graph": graph, "static": static, "logits": logits, "kernels": ops.launch_count() - before}
            if len(self._step_graphs) >= STEP_GRAPHS:
                self._step_graphs.pop(next(iter(self._step_graphs)))   # the oldest shape makes room
            self._step_graphs[shape_key] = held
        held["static"].copy_(packed, non_blocking=True)
        held["graph"].replay()
        ops.count_launches(held["kernels"])
        return held["logits"]

