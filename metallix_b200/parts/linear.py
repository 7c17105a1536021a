"""x @ W^T for a weight ``[out, in]`` (the reference's one path from a weight
name to a matmul, crates/models/qwen/src/forward/projection.rs:257-265).

float32 runs on the hand-written CUDA-core kernel (true 32-bit, fixed order).
bfloat16 runs on the hand-written tcgen05 kernel where its shape rules hold,
else on the library product (the reference itself calls a library matmul
here), or on the plain CUDA-core kernel when asked.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import ops
from .registry import Runtime


class Linear:
    def __init__(self, weight: torch.Tensor, runtime: Runtime):
        if weight.dim() != 2:
            raise ValueError(f"a linear weight must be [out, in], got {tuple(weight.shape)}")
        self.weight = weight.to(device=runtime.device, dtype=runtime.dtype).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.dtype = runtime.dtype
        self.backend = runtime.gemm_backend

    @classmethod
    def stacked(cls, weights: Sequence[torch.Tensor], runtime: Runtime) -> "Linear":
        """Several weights over the same input, rows one after another, so
        that one product yields all their outputs side by side."""
        return cls(torch.cat([w.to(runtime.device) for w in weights], dim=0), runtime)

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out_dtype = out_dtype or self.dtype
        if self.dtype == torch.float32:
            return ops.gemm_simple(x, self.weight, out_dtype=torch.float32, out=out)
        return ops.gemm_bf16(x, self.weight, out_dtype=out_dtype, backend=self.backend, out=out)

    def rows_are_short(self) -> bool:
        """Whether this is a weight of the kind whose decode-step products are
        short, overlapped kernels (rows of at most ``ops.STREAM_K`` values, the
        kernel chosen by this library), where a hand-over between kernels costs
        as much as the work."""
        return self.dtype == torch.bfloat16 and self.backend == "auto" and self.in_features <= ops.STREAM_K

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()
