"""Rotate-half rotary position encoding over the first ``rotary_dim`` values
of a head (crates/models/qwen/src/forward.rs:2031-2054: dims = head_dim,
traditional = false, base = rope_theta, scale 1). For i < rotary_dim / 2:
f_i = theta^(-2i / rotary_dim), out[i] = x[i] cos(p f_i) - x[i + half] sin(p f_i),
out[i + half] = x[i + half] cos(p f_i) + x[i] sin(p f_i).

Angles are formed in float64 (position times frequency), cos and sin are
rounded once to float32 tables that the kernels index by position.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .registry import Runtime, WeightStore, register_part


class RotaryHalf:
    kind = "rope_half"
    fused_tables = True  # the attention mixer may hand cos/sin to its fused kernel

    def __init__(self, theta: float, rotary_dim: int, head_dim: int, runtime: Runtime):
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and within head_dim {head_dim}")
        self.theta, self.rotary_dim, self.head_dim = float(theta), rotary_dim, head_dim
        # Layers with the same parameters share one pair of tables.
        key = ("rope_half", self.theta, rotary_dim, runtime.max_positions, str(runtime.device))
        if key not in runtime.shared:
            half = rotary_dim // 2
            index = torch.arange(half, dtype=torch.float64, device=runtime.device)
            frequency = torch.pow(torch.tensor(self.theta, dtype=torch.float64, device=runtime.device),
                                  -2.0 * index / rotary_dim)
            position = torch.arange(runtime.max_positions, dtype=torch.float64, device=runtime.device)
            angle = position[:, None] * frequency[None, :]
            runtime.shared[key] = (torch.cos(angle).to(torch.float32).contiguous(),
                                   torch.sin(angle).to(torch.float32).contiguous())
        self.cos, self.sin = runtime.shared[key]

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor):
        """Rotates q [tokens, heads * head_dim] and k [tokens, kv_heads * head_dim];
        returns (q_rotated [tokens, heads, head_dim], k_rotated [tokens, kv_heads, head_dim])."""
        q_out = ops.norm_rotate_heads(q, self.head_dim, positions, cos=self.cos, sin=self.sin)
        k_out = ops.norm_rotate_heads(k, self.head_dim, positions, cos=self.cos, sin=self.sin)
        return q_out, k_out


def _build(spec: PartSpec, weights: WeightStore, runtime: Runtime) -> RotaryHalf:
    return RotaryHalf(spec["theta"], spec["rotary_dim"], spec["head_dim"], runtime)


register_part("position", "rope_half", _build)
