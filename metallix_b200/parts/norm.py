"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, the weight multiplying
directly (crates/models/qwen/src/forward.rs:2442-2449). Sum of squares and
scale are float32 in both precisions."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.spec import PartSpec
from .registry import Runtime, WeightStore, register_part


class RMSNorm:
    kind = "rmsnorm"
    adds_summands = True   # add_forward also takes [parts, rows, size]: a sum its producer left in parts

    def __init__(self, weight: torch.Tensor, eps: float, runtime: Runtime):
        self.weight = weight.to(device=runtime.device, dtype=torch.float32).contiguous()
        self.size = self.weight.numel()
        self.eps = float(eps)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype,
                rows_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype, rows_index=rows_index)

    def add_forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor],
                    out_dtype: torch.dtype) -> torch.Tensor:
        """residual += delta (float32, in place), then the norm of the sum.
        ``delta`` may be float32 ``[parts, rows, size]``: its parts are added up first."""
        if delta is None:
            return ops.rmsnorm(residual, self.weight, self.eps, out_dtype)
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out_dtype)


def _build(spec: PartSpec, weights: WeightStore, runtime: Runtime) -> RMSNorm:
    weight = weights.take(spec["weight"])
    if weight.numel() != spec["size"]:
        raise ValueError(f"{spec['weight']} has {weight.numel()} values, the norm is over {spec['size']}")
    return RMSNorm(weight, spec["eps"], runtime)


register_part("norm", "rmsnorm", _build)
