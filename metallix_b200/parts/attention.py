"""Grouped-query attention over the paged cache.

q = a Wq^T, k = a Wk^T, v = a Wv^T; optional per-head norms of q and k before
the position encoding; K and V written into the cache; s = (q k^T) * scale with
a causal mask (and an optional window), softmax over keys, query head j reading
key/value head j // (heads / kv_heads); then the output projection
(crates/models/qwen/src/forward.rs:2012-2065, :1967-1989, :2070-2093).

Every size and constant is a parameter. When the head norms are RMSNorms (or
absent) and the position encoding offers cos/sin tables (or is absent), norm,
rotation and cache write run as one kernel; any other norm or position part is
called through its own interface and only the cache write stays here.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from .. import ops
from ..config.spec import CacheNeed, PartSpec
from .linear import Linear
from .norm import RMSNorm
from .registry import (CacheView, Prepared, Runtime, StepContext, StepPlan, WeightStore, build_part,
                       register_part)

TILE_TOKENS = 16     # query tokens per tile of the general kernel (csrc/kernels/attention_tile.cu)
WIDE_TOKENS = 128    # ... of the tensor-core prompt kernels (csrc/kernels/attention_prefill*.cu)
PROJECT_TOKENS = 32  # decode steps of up to this many tokens merge their splits and project in one kernel
LONG_CONTEXT = 2048  # a portion of a prompt that sees this many keys or more counts as behind a long context


def attention_tiles(plan: StepPlan) -> Prepared:
    """The lists the attention kernels walk, for one step.

    ``tile_*``: query tiles of up to 16 consecutive tokens of one request,
    those of the requests that bring several tokens first (``multi_tiles`` of
    them), then one per request that brings a single token. ``decode_token`` /
    ``decode_request``: (token, request row) of the requests that bring one
    token, for the split-key kernel (a negative token is a padding row).
    ``wide_*``: tiles of up to 128 tokens over the requests that bring
    several, those with most keys first, for the tensor-core prompt kernels.
    Facts: ``longest_context`` bounds position + 1 of the single tokens,
    ``longest_keys`` the keys a wide tile sees. A portion of a prompt behind
    ``LONG_CONTEXT`` keys or more runs other launches (its keys are shared out
    among blocks) than the same portion at a prompt's start: that is the
    ``graph_key``."""
    counts, starts, live = plan.counts, plan.starts, plan.live
    rows = len(counts)
    if all(count == 1 for count in counts):     # a decode step: no loop over the rows
        index = np.arange(rows, dtype=np.int32)
        alive = index < live
        arrays = {"tile_request": index, "tile_start": index, "tile_length": alive.astype(np.int32),
                  "decode_token": np.where(alive, index, -1).astype(np.int32), "decode_request": index}
        empty = np.empty(0, dtype=np.int32)
        arrays.update(wide_request=empty, wide_start=empty, wide_length=empty)
        longest = plan.context_bound if plan.replayable else max(
            [starts[row] + 1 for row in range(min(live, rows))], default=1)
        return Prepared(arrays, {"multi_tiles": 0, "decode_rows": rows, "longest_context": longest,
                                 "longest_keys": 0}, graph_key=False)
    tile_request, tile_start, tile_length = [], [], []
    singles, wide = [], []
    longest, longest_keys, begin = 0, 0, 0
    for row, (count, start) in enumerate(zip(counts, starts)):
        if count == 1:
            singles.append((row, begin, 1 if row < live else 0))
            longest = max(longest, start + 1)
        else:
            for first in range(0, count, TILE_TOKENS):
                tile_request.append(row)
                tile_start.append(begin + first)
                tile_length.append(min(TILE_TOKENS, count - first))
            longest_keys = max(longest_keys, start + count)
            for first in range(0, count, WIDE_TOKENS):
                size = min(WIDE_TOKENS, count - first)
                wide.append((start + first + size, row, begin + first, size))
        begin += count
    multi_tiles = len(tile_request)
    wide.sort(key=lambda item: -item[0])   # the tiles with most keys start first
    for row, token, length in singles:
        tile_request.append(row)
        tile_start.append(token)
        tile_length.append(length)
    many_keys = longest_keys >= LONG_CONTEXT
    if plan.replayable:   # a graph serves every context of its kind
        longest = plan.context_bound
        longest_keys = plan.context_bound if many_keys else LONG_CONTEXT - 1
    as_array = lambda values: np.asarray(values, dtype=np.int32)
    arrays = {"tile_request": as_array(tile_request), "tile_start": as_array(tile_start),
              "tile_length": as_array(tile_length),
              "decode_token": as_array([token if length else -1 for _, token, length in singles]),
              "decode_request": as_array([row for row, _, _ in singles]),
              "wide_request": as_array([w[1] for w in wide]), "wide_start": as_array([w[2] for w in wide]),
              "wide_length": as_array([w[3] for w in wide])}
    return Prepared(arrays, {"multi_tiles": multi_tiles, "decode_rows": len(singles), "longest_context": longest,
                             "longest_keys": longest_keys}, graph_key=many_keys)


class GQAttention:
    kind = "gqa_attention"
    graph_safe = True  # launches the same kernels whatever the step's integers are
    step_key = "attention_tiles"   # every attention layer of a model walks the same lists
    prepare_step = staticmethod(attention_tiles)

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        self.hidden_size = spec["hidden_size"]
        self.num_heads = spec["num_heads"]
        self.num_kv_heads = spec["num_kv_heads"]
        self.head_dim = spec["head_dim"]
        self.scale = float(spec["scale"])
        self.window = spec.get("window") or 0
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} query heads cannot share {self.num_kv_heads} key/value heads")
        if self.head_dim % 2 or not 0 < self.head_dim <= 256:
            raise ValueError(f"head_dim {self.head_dim}: the attention kernels take even sizes up to 256")
        q, k, v = (weights.take(spec[name]) for name in ("q_proj", "k_proj", "v_proj"))
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        for name, weight, rows in (("q_proj", q, self.q_size), ("k_proj", k, self.kv_size),
                                   ("v_proj", v, self.kv_size)):
            if tuple(weight.shape) != (rows, self.hidden_size):
                raise ValueError(f"{spec[name]} is {tuple(weight.shape)}, expected {(rows, self.hidden_size)}")
        self.qkv = Linear.stacked([q, k, v], runtime)  # rows: all q heads, then k heads, then v heads
        self.o = Linear(weights.take(spec["o_proj"]), runtime)
        if (self.o.out_features, self.o.in_features) != (self.hidden_size, self.q_size):
            raise ValueError(f"{spec['o_proj']} is {tuple(self.o.weight.shape)}")
        self.q_norm = build_part("norm", spec.get("q_norm"), weights, runtime)
        self.k_norm = build_part("norm", spec.get("k_norm"), weights, runtime)
        self.position = build_part("position", spec.get("position"), weights, runtime)
        norms_fuse = all(n is None or isinstance(n, RMSNorm) for n in (self.q_norm, self.k_norm))
        eps_agree = (self.q_norm is None or self.k_norm is None or self.q_norm.eps == self.k_norm.eps)
        position_fuses = self.position is None or getattr(self.position, "fused_tables", False)
        self.fused = norms_fuse and eps_agree and position_fuses
        self.dtype = runtime.dtype
        self.split_decode = ops.decode_attention_supported(self.head_dim, self.num_heads,
                                                           self.num_kv_heads, self.dtype)
        self.flash = ops.flash_prefill_supported(self.head_dim, self.num_heads, self.num_kv_heads,
                                                 self.dtype)

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="kv_pages", kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                         window=self.window or None)

    def parts(self):
        return [self.q_norm, self.k_norm, self.position]

    def _tiles(self, ctx: StepContext) -> Dict[str, object]:
        """The step's tile lists: what the engine prepared, or (for a caller
        that built a context by hand) made here from the host lists."""
        tiles = ctx.extras.get(self.step_key)
        if tiles is None:
            if ctx.request_offsets is None:
                raise ValueError("the attention's tile lists were not prepared for this step")
            counts = [ctx.request_offsets[row + 1] - ctx.request_offsets[row] for row in range(ctx.num_requests)]
            ends = [start + count for start, count in zip(ctx.request_positions, counts)]
            prepared = attention_tiles(StepPlan(counts, ctx.request_positions, len(counts), max(ends)))
            tiles = dict(prepared.facts)
            for name, array in prepared.arrays.items():
                tiles[name] = torch.from_numpy(array).to(ctx.device)
            ctx.extras[self.step_key] = tiles
        return tiles

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        return self._attend(x, ctx, cache, summands=False)

    def forward_summands(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        """``forward`` for a caller that adds up summands: where one kernel can
        put the splits of a decode step together and project them head by head,
        the result is float32 ``[heads, tokens, hidden]`` whose sum over the
        heads is ``forward``'s output; otherwise ``forward``'s output itself."""
        return self._attend(x, ctx, cache, summands=True)

    def _attend(self, x: torch.Tensor, ctx: StepContext, cache: CacheView, summands: bool) -> torch.Tensor:
        tokens = x.shape[0]
        qkv = self.qkv.forward(x)
        q = qkv[:, :self.q_size]
        k = qkv[:, self.q_size:self.q_size + self.kv_size]
        v = qkv[:, self.q_size + self.kv_size:]
        q_heads = torch.empty((tokens, self.num_heads, self.head_dim), dtype=self.dtype, device=x.device)
        write = cache.write and cache.slots is not None
        if self.fused:
            eps = self.q_norm.eps if self.q_norm is not None else (self.k_norm.eps if self.k_norm else 0.0)
            ops.qk_norm_rope_cache(
                q, k, v, q_heads, cache.pool if write else None, cache.slots if write else None,
                ctx.positions,
                self.q_norm.weight if self.q_norm is not None else None,
                self.k_norm.weight if self.k_norm is not None else None,
                self.position.cos if self.position is not None else None,
                self.position.sin if self.position is not None else None, eps)
        else:
            if self.q_norm is not None:
                q = self.q_norm.forward(q.reshape(tokens * self.num_heads, self.head_dim).contiguous(),
                                        self.dtype).view(tokens, self.q_size)
            if self.k_norm is not None:
                k = self.k_norm.forward(k.reshape(tokens * self.num_kv_heads, self.head_dim).contiguous(),
                                        self.dtype).view(tokens, self.kv_size)
            if self.position is not None:
                q_rot, k_rot = self.position.apply(q, k, ctx.positions)
                q_heads = q_rot.contiguous().view(tokens, self.num_heads, self.head_dim)
                k = k_rot.contiguous().view(tokens, self.kv_size)
            else:
                q_heads = q.contiguous().view(tokens, self.num_heads, self.head_dim)
            if write:
                ops.write_cache(k, v, cache.pool, cache.slots, ctx.positions)
        tiles = self._tiles(ctx)
        multi_tiles = tiles["multi_tiles"]
        split = tiles["decode_rows"] and self.split_decode
        if (summands and split and multi_tiles == 0 and tokens <= PROJECT_TOKENS and self.o.rows_are_short()
                and ops.decode_project_supported(self.head_dim, self.num_heads, self.num_kv_heads, self.dtype,
                                                 tokens, self.o.weight)):
            # Only single tokens, at most 64 of them: the splits are merged
            # and projected by one kernel, one summand per head.
            return ops.paged_attention_decode_project(
                q_heads, cache.pool, cache.block_tables, tiles["decode_token"], tiles["decode_request"],
                ctx.positions, self.scale, tiles["longest_context"], self.o.weight, self.window)
        out = torch.empty_like(q_heads)
        if split:
            # Requests that bring one token: split along the keys.
            ops.paged_attention_decode(q_heads, cache.pool, out, cache.block_tables, tiles["decode_token"],
                                       tiles["decode_request"], ctx.positions, self.scale,
                                       tiles["longest_context"], self.window)
        if self.flash:
            # Requests that bring several tokens: tensor cores, tiles of 128.
            if tiles["wide_request"].numel():
                ops.flash_prefill(q_heads, cache.pool, out, cache.block_tables, tiles["wide_request"],
                                  tiles["wide_start"], tiles["wide_length"], ctx.positions, self.scale,
                                  self.window, longest_context=tiles["longest_keys"])
            rest = None if split else slice(multi_tiles, None)   # single tokens not yet served
        else:
            rest = slice(0, multi_tiles) if split else slice(0, None)
        if rest is not None and tiles["tile_request"][rest].numel():
            ops.paged_attention_tile(q_heads, cache.pool, out, cache.block_tables, tiles["tile_request"][rest],
                                     tiles["tile_start"][rest], tiles["tile_length"][rest], ctx.positions,
                                     self.scale, self.window)
        return self.o.forward(out.view(tokens, self.q_size))

    def weight_bytes(self) -> int:
        return self.qkv.weight_bytes() + self.o.weight_bytes()


register_part("mixer", "gqa_attention", lambda spec, weights, runtime: GQAttention(spec, weights, runtime))
