"""A decoder put together from a ``ModelSpec``: embedding, blocks in the
spec's order, final norm on the wanted rows only, output head
(crates/models/qwen/src/forward.rs:1562-1606)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.spec import CacheNeed, ModelSpec
from ..parts.registry import (CacheView, Runtime, StepContext, WeightStore, _BUILDERS, build_part)


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], runtime: Runtime,
                 consume: bool = False):
        """``consume``: the caller gives ``tensors`` away; entries are removed
        as the parts take them, so that a model close to the device's memory
        never holds its weights twice."""
        spec.validate()
        self.spec, self.runtime = spec, runtime
        weights = WeightStore(tensors)
        self.embedding = build_part("embedding", spec.embedding, weights, runtime)
        self.blocks = []
        for layer in spec.layers:
            builder = _BUILDERS.get(("block", layer.block.kind))
            if builder is None:
                raise KeyError(f"no block arrangement of kind {layer.block.kind!r}")
            self.blocks.append(builder(layer, weights, runtime))
            if consume:
                weights.drop_taken(keep=(spec.embedding.get("weight"), spec.head.get("weight")))
        self.final_norm = build_part("norm", spec.final_norm, weights, runtime)
        head_builder = _BUILDERS.get(("head", spec.head.kind))
        if head_builder is None:
            raise KeyError(f"no head of kind {spec.head.kind!r}")
        self.head = head_builder(spec.head, weights, runtime, self.embedding)
        if consume:
            weights.drop_taken()
        self.order = list(spec.order)
        self.vocab_size = spec.vocab_size

    def cache_needs(self) -> List[Optional[CacheNeed]]:
        """What each cache entry (one per layer index) must hold."""
        needs: List[Optional[CacheNeed]] = [None] * self.spec.num_cache_entries()
        for run in self.order:
            entry = run.cache_entry()
            need = self.blocks[run.layer].mixer.cache_need()
            if run.write_cache or needs[entry] is None:
                if needs[entry] is not None and needs[entry].group_key() != need.group_key() \
                        and run.write_cache:
                    raise ValueError(f"cache entry {entry} is written by layers with different needs")
                needs[entry] = need
        return needs

    def weight_bytes(self) -> int:
        """Bytes of every weight one step reads once."""
        total = self.head.weight_bytes() if not self.head.tied else self.embedding.weight_bytes()
        for block in self.blocks:
            for part in (block.mixer, block.feed_forward):
                total += part.weight_bytes() if hasattr(part, "weight_bytes") else 0
        return total

    def forward(self, token_ids: torch.Tensor, ctx: StepContext, views, wanted_rows: Optional[torch.Tensor]):
        """``views(entry, write) -> CacheView``. Returns float32 logits
        [wanted, vocab], or None when no row is wanted."""
        residual = self.embedding.forward(token_ids)
        pending = None
        for run in self.order:
            block = self.blocks[run.layer]
            pending = block.forward(residual, pending, ctx, views(run.cache_entry(), run.write_cache))
        if wanted_rows is None or wanted_rows.numel() == 0:
            return None
        if pending is not None:
            ops.add_(residual, pending)
        normed = self.final_norm.forward(residual, self.runtime.dtype, rows_index=wanted_rows)
        return self.head.forward(normed)
