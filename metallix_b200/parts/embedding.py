"""The model's two ends: token embedding (row gather,
crates/models/qwen/src/forward/projection.rs:208-216) and the output head
(logits = n W^T through the embedding when tied, else lm_head,
crates/models/qwen/src/forward.rs:574-580), whose logits leave in float32."""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .linear import Linear
from .registry import Runtime, WeightStore, register_part



class TokenEmbedding:
    kind = "token_embedding"

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        table = weights.take(spec["weight"])
        if tuple(table.shape) != (spec["vocab_size"], spec["hidden_size"]):
            raise ValueError(f"{spec['weight']} is {tuple(table.shape)}")
        self.table = table.to(device=runtime.device, dtype=runtime.dtype).contiguous()
        self.vocab_size = spec["vocab_size"]
        self.name = spec["weight"]

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.embed(ids, self.table)

    def weight_bytes(self) -> int:
        return self.table.numel() * self.table.element_size()


class LinearHead:
    kind = "linear_head"

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime, embedding=None):
        if embedding is not None and embedding.name == spec["weight"]:
            self.linear = Linear.__new__(Linear)  # tied: one tensor serves both ends
            self.linear.weight = embedding.table
            self.linear.out_features, self.linear.in_features = embedding.table.shape
            self.linear.dtype = runtime.dtype
            self.linear.backend = runtime.gemm_backend
            weights.take(spec["weight"])
            self.tied = True
        else:
            self.linear = Linear(weights.take(spec["weight"]), runtime)
            self.tied = False
        if self.linear.out_features != spec["vocab_size"] or self.linear.in_features != spec["hidden_size"]:
            raise ValueError(f"{spec['weight']} is {tuple(self.linear.weight.shape)}")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.linear.forward(x, out_dtype=torch.float32)

    def weight_bytes(self) -> int:
        return 0 if self.tied else self.linear.weight_bytes()


register_part("embedding", "token_embedding",
              lambda spec, weights, runtime: TokenEmbedding(spec, weights, runtime))
register_part("head", "linear_head",
              lambda spec, weights, runtime, embedding=None: LinearHead(spec, weights, runtime, embedding))
