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

from typing import Optional

import torch

from .. import ops
from ..config.spec import CacheNeed, PartSpec
from .linear import Linear
from .norm import RMSNorm
from .registry import CacheView, Runtime, StepContext, WeightStore, build_part, register_part


class GQAttention:
    kind = "gqa_attention"
    graph_safe = True  # launches the same kernels whatever the step's integers are

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

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
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
        out = torch.empty_like(q_heads)
        decode_rows = 0 if ctx.decode_token is None else ctx.decode_token.numel()
        split = decode_rows and self.split_decode
        if split:
            # Requests that bring one token: split along the keys.
            ops.paged_attention_decode(q_heads, cache.pool, out, cache.block_tables, ctx.decode_token,
                                       ctx.decode_request, ctx.positions, self.scale,
                                       ctx.longest_context, self.window)
        if self.flash and ctx.wide_tile_request is not None:
            # Requests that bring several tokens: tensor cores, tiles of 64.
            if ctx.wide_tile_request.numel():
                ops.flash_prefill(q_heads, cache.pool, out, cache.block_tables, ctx.wide_tile_request,
                                  ctx.wide_tile_start, ctx.wide_tile_length, ctx.positions, self.scale,
                                  self.window, longest_context=ctx.longest_keys)
            rest = None if split else slice(ctx.multi_tiles, None)   # single tokens not yet served
        else:
            rest = slice(0, ctx.multi_tiles) if split else slice(0, None)
        if rest is not None and ctx.tile_request[rest].numel():
            ops.paged_attention_tile(q_heads, cache.pool, out, cache.block_tables, ctx.tile_request[rest],
                                     ctx.tile_start[rest], ctx.tile_length[rest], ctx.positions,
                                     self.scale, self.window)
        return self.o.forward(out.view(tokens, self.q_size))

    def weight_bytes(self) -> int:
        return self.qkv.weight_bytes() + self.o.weight_bytes()


register_part("mixer", "gqa_attention", lambda spec, weights, runtime: GQAttention(spec, weights, runtime))
