"""Decode steps as CUDA graphs.

A step in which every request brings exactly one token launches the same
kernels every time; only ids, positions, slots and block tables change. Such a
step is captured once per (batch-size bucket, context bucket) and replayed: one
copy of the step's integers into the graph's static buffer, one graph launch.
The reference hides the same launch cost by queueing step t+1 before step t is
read (crates/models/qwen/src/forward/paged.rs:784-858); here the launches
themselves go away.

Rows beyond the live requests are padding: id 0, position 0, slot -1 (no cache
write), and whatever the parts' own integers say of a padding row (the
attention: a tile of no tokens, a negative decode row). Block tables are as
wide as the context bucket: the longest live context rounded up to 2,048 times
a power of two, so that table width, split counts and scratch follow the
contexts that are live, not the longest one the engine allows.
"""
from __future__ import annotations

import contextlib
import gc
import weakref
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.registry import StepContext, StepPlan, block_parts, graph_safe

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
# A captured decode step runs in one of two times some 4% apart (0.87 or 0.90
# ms for 8 requests at the 0.6B shapes): the same engine recaptures the same
# step faster or slower, with the weights, the cache and the kernels' own
# times unchanged; what differs lies between the kernels of the replayed graph.
# So a step is captured several times, each capture alive beside the others,
# each timed on the step's own rows, and the fastest kept.
PLACEMENTS = 8             # at most; fewer once one capture has come out 2% faster than another
PLACEMENT_REPLAYS = 6
PLACEMENT_WORTH_MS = 2.0   # a step that takes longer is bound by what it reads, not by where its buffers lie
_GENERIC = ("ids", "positions", "token_request", "request_slots", "wanted")


@contextlib.contextmanager
def capture_quietly(graph: torch.cuda.CUDAGraph, pool):
    """Captures into ``graph`` with the garbage collector off: freeing another
    engine's graph or device memory in the middle would invalidate the capture."""
    collecting = gc.isenabled()
    gc.collect()
    gc.disable()
    try:
        with torch.cuda.graph(graph, pool=pool):
            yield
    finally:
        if collecting:
            gc.enable()


class _Bucket:
    def __init__(self, size: int, bound: int, table_width: int):
        self.size, self.bound, self.table_width = size, bound, table_width
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.static: Optional[torch.Tensor] = None   # int32 metadata on the device
        self.logits: Optional[torch.Tensor] = None
        self.layout: Dict[str, slice] = {}
        self.facts: Dict[str, dict] = {}              # per preparing part: the host values baked into the graph
        self.prepared: Dict[int, list] = {}           # live rows -> [(layout name, array)] of the parts' integers
        self.kernels = 0                              # our kernel launches inside the graph
        self.staging: List[dict] = []                 # pinned host buffers for the step's integers
        self.turn = 0


class DecodeGraphs:
    def __init__(self, engine):
        self._engine = weakref.ref(engine)   # the engine owns this object, not the reverse
        self.buckets: Dict[Tuple[int, int], _Bucket] = {}
        self.pool = None                        # unused since every kept capture has memory of its own
        self.placements = PLACEMENTS
        self.placement_ms: Dict[Tuple[int, int], List[float]] = {}   # what each placement of a step took
        cache = engine.cache
        self._windowed = any(g.need.window for g in cache.groups)
        self.h2d_bytes = 0
        # Mirrors of the manager's tables: manager id -> (epoch, pages, per-group rows)
        self._host_tables: Dict[int, tuple] = {}

    @property
    def engine(self):
        return self._engine()

    @staticmethod
    def usable(model) -> bool:
        """Every part of every block must launch the same work whatever the
        step's integers and the device's values are (no host reads): a mixer
        has to promise it (``graph_safe = True``), any other part may deny it
        (``graph_safe = False``)."""
        return all(graph_safe(part) for block in model.blocks for part in block_parts(block))

    def bucket_for(self, rows: int) -> Optional[int]:
        for size in BUCKETS:
            if size >= rows:
                return size
        return None

    def sizes_captured(self) -> List[int]:
        return sorted({size for size, _ in self.buckets})

    # ----------------------------------------------------------------- layout
    def _plan(self, bucket: _Bucket, live: int) -> StepPlan:
        # positions are not given: what a part prepares for a replayed decode
        # step may depend on which rows are live only
        return StepPlan([1] * bucket.size, None, live, bucket.bound, replayable=True)

    def _prepare(self, bucket: _Bucket, live: int) -> list:
        """[(layout name, int32 array)] of the parts' own integers for a step
        with ``live`` requests; kept per ``live``."""
        held = bucket.prepared.get(live)
        if held is None:
            held = []
            for key, part in self.engine._preparers.items():
                result = part.prepare_step(self._plan(bucket, live))
                for name, array in result.arrays.items():
                    held.append((f"{key}/{name}", np.ascontiguousarray(array, dtype=np.int32).reshape(-1)))
                bucket.facts.setdefault(key, dict(result.facts))
            bucket.prepared[live] = held
        return held

    def _layout(self, bucket: _Bucket) -> None:
        size, layout, cursor = bucket.size, {}, 0
        for name in _GENERIC:
            layout[name] = slice(cursor, cursor + size)
            cursor += size
        for name, array in self._prepare(bucket, 0):
            layout[name] = slice(cursor, cursor + array.size)
            cursor += array.size
        for g in range(len(self.engine.cache.groups)):
            layout[f"slots{g}"] = slice(cursor, cursor + size)
            cursor += size
            layout[f"table{g}"] = slice(cursor, cursor + size * bucket.table_width)
            cursor += size * bucket.table_width
        layout["end"] = slice(cursor, cursor)
        bucket.layout = layout

    def _context(self, bucket: _Bucket) -> StepContext:
        s, size, engine = bucket.static, bucket.size, self.engine
        cut = lambda name: s[bucket.layout[name]]
        extras = {}
        for key in engine._preparers:
            extras[key] = dict(bucket.facts[key])
            for name, _ in bucket.prepared[0]:
                if name.startswith(key + "/"):
                    extras[key][name[len(key) + 1:]] = cut(name)
        return StepContext(
            device=engine.device, dtype=engine.dtype, num_tokens=size, num_requests=size,
            positions=cut("positions"), token_request=cut("token_request"),
            request_slots=cut("request_slots"), request_offsets=None, request_positions=None,
            extras=extras)

    def _views(self, bucket: _Bucket):
        s, size, cache = bucket.static, bucket.size, self.engine.cache
        tables = {g.index: s[bucket.layout[f"table{g.index}"]].view(size, bucket.table_width)
                  for g in cache.groups}
        slots = {g.index: s[bucket.layout[f"slots{g.index}"]] for g in cache.groups}
        return lambda entry, write: cache.view(entry, write, tables, slots)

    def _host_constants(self, bucket: _Bucket, out: np.ndarray) -> None:
        """What never changes in a bucket's integers, with every row padding."""
        size, layout, cache = bucket.size, bucket.layout, self.engine.cache
        index = np.arange(size, dtype=np.int32)
        out[:] = 0
        for name in ("token_request", "wanted"):
            out[layout[name]] = index
        for name, array in self._prepare(bucket, 0):
            out[layout[name]] = array
        for g in cache.groups:
            out[layout[f"slots{g.index}"]] = -1
            out[layout[f"table{g.index}"]] = -1

    def _host_fill(self, bucket: _Bucket, rows: Sequence, stage: dict) -> None:
        """rows: (manager id, token id, position, state slot) of the live
        requests; fills one step's integers into the staging buffer, which
        holds the constants and, in its first ``stage["filled"]`` rows, an
        earlier step. ``stage["held"][row]`` remembers whose block table a row
        holds, so that a table is copied again only when it has changed."""
        out, held_rows, filled = stage["array"], stage["held"], stage["filled"]
        layout, cache = bucket.layout, self.engine.cache
        manager, page_tokens = self.engine.manager, cache.page_tokens
        live, width = len(rows), bucket.table_width
        ids, positions, request_slots = (out[layout[k]] for k in ("ids", "positions", "request_slots"))
        if stage["live"] != live:    # the parts' integers change only with the number of live rows
            for name, array in self._prepare(bucket, live):
                out[layout[name]] = array
            stage["live"] = live
        if filled > live:   # rows an earlier, larger step left behind become padding again
            ids[live:filled] = 0
            positions[live:filled] = 0
            request_slots[live:filled] = 0
            for g in cache.groups:
                out[layout[f"slots{g.index}"]][live:filled] = -1
        for row, (rid, token, position, slot) in enumerate(rows):
            ids[row], positions[row], request_slots[row] = token, position, slot
            pages = -(-(position + 1) // page_tokens)
            epoch = manager.epoch(rid)
            mirror = self._host_tables.get(rid)
            if mirror is None or mirror[0] != epoch or mirror[1] < pages or self._windowed:
                held = [np.asarray(manager.table(rid, g.index), dtype=np.int32) for g in cache.groups]
                if len(self._host_tables) > 4 * manager.max_requests():
                    self._host_tables.clear()   # requests that left long ago
                mirror = self._host_tables[rid] = (epoch, pages, held)
            held = mirror[2]
            copy_table = held_rows[row] is not held
            held_rows[row] = held
            for g in cache.groups:
                pages_held = held[g.index]
                if copy_table:
                    table = out[layout[f"table{g.index}"]]
                    count = min(len(pages_held), width)
                    table[row * width:row * width + count] = pages_held[:count]
                    table[row * width + count:(row + 1) * width] = -1
                out[layout[f"slots{g.index}"]][row] = \
                    pages_held[position // page_tokens] * page_tokens + position % page_tokens

    # ---------------------------------------------------------------- capture
    def _capture(self, size: int, bound: int, pool=None) -> _Bucket:
        from .. import ops
        engine = self.engine
        bucket = _Bucket(size, bound, -(-bound // engine.cache.page_tokens))
        self._layout(bucket)
        total = bucket.layout["end"].start
        host = np.zeros(total, dtype=np.int32)
        self._host_constants(bucket, host)   # all padding: nothing is read or written
        bucket.static = torch.from_numpy(host).to(engine.device)
        # Two pinned staging buffers taken in turn, each with the constants in
        # place; an event says when the copy out of a buffer is done.
        for _ in range(2):
            pinned = torch.empty(total, dtype=torch.int32, pin_memory=True)
            pinned.numpy()[:] = host
            bucket.staging.append({"pinned": pinned, "array": pinned.numpy(), "copied": None,
                                   "filled": 0, "live": 0, "held": [None] * size})
        ctx, views = self._context(bucket), self._views(bucket)
        ids, wanted = bucket.static[bucket.layout["ids"]], bucket.static[bucket.layout["wanted"]]
        stream = torch.cuda.Stream(device=engine.device)
        stream.wait_stream(torch.cuda.current_stream(engine.device))
        with torch.cuda.stream(stream):
            for _ in range(2):   # libraries and lazily loaded kernels settle before the capture
                engine.model.forward(ids, ctx, views, wanted)
        torch.cuda.current_stream(engine.device).wait_stream(stream)
        torch.cuda.synchronize(engine.device)
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with capture_quietly(graph, pool):
            bucket.logits = engine.model.forward(ids, ctx, views, wanted)
        bucket.kernels = ops.launch_count() - before
        bucket.graph = graph
        return bucket

    def _settle(self, size: int, bound: int, rows: Sequence, fed_ids: Optional[torch.Tensor]) -> _Bucket:
        """Captures the step in several placements and keeps the fastest. Each
        candidate replays the real step of ``rows`` a few times: the same
        token at the same position writes the same keys and values again and
        gives the same logits, so nothing changes; a model with state of its
        own per request (which a replay would advance) gets one capture."""
        engine = self.engine
        stateless = all(need is None or need.kind != "state" for need in engine.cache.needs)
        tries = self.placements if stateless else 1
        first = self._capture(size, bound, pool=None)
        if tries <= 1:
            return first
        best, best_ms, timings = None, None, []
        candidate = first
        for attempt in range(tries):
            if candidate is None:
                try:
                    candidate = self._capture(size, bound, pool=None)   # memory of its own, beside the others'
                except torch.cuda.OutOfMemoryError:
                    break   # no room for another placement: the best so far serves
            stage = candidate.staging[0]
            self._host_fill(candidate, rows, stage)
            stage["filled"] = len(rows)
            candidate.static.copy_(stage["pinned"], non_blocking=True)
            if fed_ids is not None:
                candidate.static[candidate.layout["ids"]][:len(rows)].copy_(fed_ids[:len(rows)], non_blocking=True)
            candidate.graph.replay()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            for _ in range(PLACEMENT_REPLAYS):
                candidate.graph.replay()
            end.record()
            end.synchronize()
            ms = begin.elapsed_time(end) / PLACEMENT_REPLAYS
            timings.append(ms)
            if best_ms is None or ms < best_ms:
                best, best_ms = candidate, ms       # the one before goes when its last reference does
            candidate = None
            if ms >= PLACEMENT_WORTH_MS or best_ms <= 0.98 * max(timings):
                break   # too long a step to gain, or both of the two times have been seen
        self.placement_ms[(size, bound)] = timings
        return best

    # -------------------------------------------------------------------- run
    def run(self, rows: Sequence, fed_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """rows: (manager id, token id, position, state slot). Returns float32
        logits [len(rows), vocab]: a view of the graph's output that the next
        replay of the same bucket overwrites. ``fed_ids`` (int32, on the
        device, one per row) replaces the rows' token ids without the host
        ever seeing them: the tokens an earlier step picked."""
        from .. import ops
        size = self.bucket_for(len(rows))
        bound = self.engine.context_bucket(max(row[2] for row in rows) + 1)
        bucket = self.buckets.get((size, bound))
        if bucket is None:
            bucket = self.buckets[(size, bound)] = self._settle(size, bound, rows, fed_ids)
        total = bucket.layout["end"].start
        stage = bucket.staging[bucket.turn]
        bucket.turn ^= 1
        if stage["copied"] is not None:
            stage["copied"].synchronize()   # the copy of two steps ago out of this buffer (long done)
        self._host_fill(bucket, rows, stage)
        stage["filled"] = len(rows)
        bucket.static.copy_(stage["pinned"], non_blocking=True)
        if stage["copied"] is None:
            stage["copied"] = torch.cuda.Event()
        stage["copied"].record()
        if fed_ids is not None:
            bucket.static[bucket.layout["ids"]][:len(rows)].copy_(fed_ids[:len(rows)], non_blocking=True)
        bucket.graph.replay()
        ops.count_launches(bucket.kernels)
        self.h2d_bytes = total * 4
        return bucket.logits[:len(rows)]
