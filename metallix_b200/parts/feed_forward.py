"""SwiGLU feed-forward: d = ((sigmoid(g) * g) * u) Wd^T with g = m Wg^T and
u = m Wu^T (crates/models/qwen/src/forward.rs:1904-1920). Gate and up weights
are stacked so that one product yields both; SiLU and the product with u are
float32 inside the kernel."""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .linear import Linear
from .registry import Runtime, StepContext, WeightStore, register_part

FUSED_ACTIVATION_ROWS = 1536   # from here on "auto" takes the tcgen05 product with the SwiGLU epilogue


class SwiGLU:
    kind = "swiglu"

    def __init__(self, spec: PartSpec, weights: WeightStore, runtime: Runtime):
        hidden, inter = spec["hidden_size"], spec["intermediate_size"]
        gate, up = weights.take(spec["gate_proj"]), weights.take(spec["up_proj"])
        down = weights.take(spec["down_proj"])
        for name, weight, shape in (("gate_proj", gate, (inter, hidden)), ("up_proj", up, (inter, hidden)),
                                    ("down_proj", down, (hidden, inter))):
            if tuple(weight.shape) != shape:
                raise ValueError(f"{spec[name]} is {tuple(weight.shape)}, expected {shape}")
        self.gate_up = Linear.stacked([gate, up], runtime)  # rows: gate, then up
        self.down = Linear(down, runtime)
        self.intermediate_size = inter

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        few = ops.SKINNY_ROWS if x.shape[1] <= ops.STREAM_K else ops.SKINNY_ROWS // 2   # as ops.gemm_bf16
        if (x.shape[0] <= few and self.gate_up.backend in ("auto", "skinny")
                and ops.gemm_skinny_takes(x, self.gate_up.weight, swiglu=True)):
            # A decode step: gate, up and the activation in one pass over the weights.
            return self.down.forward(ops.gemm_skinny(x, self.gate_up.weight, swiglu=True))
        # From about 1,500 rows on the tcgen05 product with the activation in its
        # epilogue beats the library's product followed by an activation pass
        # (28 against 31 us at 2,048 rows of this model; 21 against 19 at 1,024,
        # 10 against 8 at 128): below that the library keeps the product, as in
        # the reference, unless the part is told to use the tcgen05 kernel.
        fused = self.gate_up.backend == "tcgen05" or (self.gate_up.backend == "auto"
                                                      and x.shape[0] >= FUSED_ACTIVATION_ROWS)
        if self.gate_up.dtype == torch.bfloat16 and fused:
            from .. import tensor_core
            if tensor_core.supports(x, self.gate_up.weight, torch.bfloat16):
                # gate, up and the activation in the product's epilogue
                return self.down.forward(tensor_core.gemm_swiglu(x, self.gate_up.weight))
        return self.down.forward(ops.silu_mul(self.gate_up.forward(x)))

    def weight_bytes(self) -> int:
        return self.gate_up.weight_bytes() + self.down.weight_bytes()


register_part("feed_forward", "swiglu", lambda spec, weights, runtime: SwiGLU(spec, weights, runtime))
