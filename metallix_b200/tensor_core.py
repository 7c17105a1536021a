"""The tcgen05 / TMEM / TMA matrix product (sm_100a), or the reason it is not
used for a given call."""
from __future__ import annotations

from typing import Optional

import torch

from . import ops

STORE_BF16, STORE_F32, SWIGLU = 0, 1, 2


def why_not(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> str:
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return "operands must be bfloat16"
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        return "operands must be [m, k] and [n, k]"
    if a.stride(1) != 1 or w.stride(1) != 1:
        return "rows must be contiguous"
    if a.data_ptr() % 16 or w.data_ptr() % 16:
        return "operands must start on 16-byte boundaries"
    if not ops._fn("mxb_gemm_tcgen05_supported")(a.shape[0], w.shape[0], a.shape[1], a.stride(0), w.stride(0)):
        return "k and the row strides must be multiples of 8"
    if out_dtype not in (torch.bfloat16, torch.float32):
        return "the result must be bfloat16 or float32"
    return ""


def supports(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> bool:
    return why_not(a, w, out_dtype) == ""


def _launch(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, n: int, epilogue: int) -> torch.Tensor:
    ops._call("mxb_gemm_tcgen05", out.data_ptr(), a.data_ptr(), w.data_ptr(), a.shape[0], n, a.shape[1],
              a.stride(0), w.stride(0), out.stride(0), epilogue, ops.status_word(a.device).data_ptr(),
              ops._stream())
    return out


def gemm(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [m, k] times w [n, k] transposed on tcgen05 tensor cores."""
    reason = why_not(a, w, out_dtype)
    if reason:
        raise ops.KernelError("the tcgen05 kernel does not take this call: " + reason)
    m, n = a.shape[0], w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    ops._need(out.shape == (m, n) and out.dtype == out_dtype and out.stride(1) == 1, "out does not fit")
    return _launch(out, a, w, n, STORE_BF16 if out_dtype == torch.bfloat16 else STORE_F32)


def gemm_swiglu(a: torch.Tensor, gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(a gate^T) * (a up^T) for gate_up = [gate rows; up rows], without
    gate and up ever reaching memory. Returns bfloat16 [m, inter]."""
    reason = why_not(a, gate_up, torch.bfloat16)
    if reason:
        raise ops.KernelError("the tcgen05 kernel does not take this call: " + reason)
    ops._need(gate_up.shape[0] % 2 == 0, "gate and up rows must pair up")
    m, inter = a.shape[0], gate_up.shape[0] // 2
    if out is None:
        out = torch.empty((m, inter), dtype=torch.bfloat16, device=a.device)
    ops._need(out.shape == (m, inter) and out.dtype == torch.bfloat16 and out.stride(1) == 1, "out does not fit")
    return _launch(out, a, gate_up, inter, SWIGLU)
