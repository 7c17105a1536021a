"""The tcgen05 / TMEM / TMA matrix product (sm_100a), or the reason it is not
used for a given call."""
from __future__ import annotations

from typing import Optional

import torch


def why_not(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> str:
    return "the tensor-core kernel is not built yet"


def supports(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> bool:
    return False


def gemm(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    raise NotImplementedError(why_not(a, w, out_dtype))
