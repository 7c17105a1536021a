"""Arrangement of one layer's parts.

``prenorm_residual`` is the reference's layer
(crates/models/qwen/src/forward.rs:1856-1885, :1889-1922):
r = x + mixer(norm1(x)); x' = r + feed_forward(norm2(r)). The residual stream
is float32; a block receives the previous block's output not yet added
(``pending``) so that every residual sum runs inside the norm kernel that
follows it.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.spec import LayerSpec
from .registry import CacheView, Runtime, StepContext, WeightStore, build_part, register_part


class PreNormResidualBlock:
    kind = "prenorm_residual"

    def __init__(self, layer: LayerSpec, weights: WeightStore, runtime: Runtime):
        self.name = layer.name
        self.mixer_norm = build_part("norm", layer.mixer_norm, weights, runtime)
        self.mixer = build_part("mixer", layer.mixer, weights, runtime)
        self.feed_forward_norm = build_part("norm", layer.feed_forward_norm, weights, runtime)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, weights, runtime)
        self.dtype = runtime.dtype
        # A mixer may leave its output as summands [parts, tokens, hidden] when
        # the norm that takes it next adds them up in its own pass over the row.
        summands = getattr(self.mixer, "forward_summands", None)
        self.mix = summands if summands is not None and getattr(self.feed_forward_norm, "adds_summands", False) \
            else self.mixer.forward

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, residual: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: CacheView) -> torch.Tensor:
        """``residual`` (float32, updated in place) plus ``pending`` is the
        layer's input; returns the feed-forward output, to be added by
        whoever runs next."""
        mixer_in = self.mixer_norm.add_forward(residual, pending, self.dtype)
        mixed = self.mix(mixer_in, ctx, cache)
        feed_in = self.feed_forward_norm.add_forward(residual, mixed, self.dtype)
        return self.feed_forward.forward(feed_in, ctx)


register_part("block", "prenorm_residual",
              lambda layer, weights, runtime: PreNormResidualBlock(layer, weights, runtime))
