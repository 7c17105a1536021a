"""Picking the next token of every row of a batch, on the device.

Greedy (temperature 0 or absent, crates/app/cli/src/chat_generation.rs:391-410),
inverse-CDF temperature sampling (crates/core/engine/src/sampling.rs:56-103)
and the race sampler (crates/core/engine/src/sampling/race.rs), optionally
inside the top-k / top-p nucleus (crates/app/cli/src/qwen_forward.rs:474-549).
What a row draws depends only on its own seed, stream and generated position,
never on the rest of the batch.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Sequence

import torch

from .. import ops

GREEDY, ICDF, RACE = 0, 1, 2
SAMPLERS = {"icdf": ICDF, "race": RACE}


@dataclass(frozen=True)
class SamplingParams:
    """How one request picks tokens. ``temperature`` 0 means greedy; otherwise
    it must be finite and positive (crates/app/cli/src/cli.rs:98-109)."""

    temperature: float = 0.0
    seed: int = 0
    stream: int = 0        # tells apart requests that share a seed
    top_p: float = 1.0
    top_k: int = 0         # 0: off
    sampler: str = "icdf"  # "icdf" or "race"

    def validate(self) -> None:
        if not math.isfinite(self.temperature) or self.temperature < 0.0:
            raise ValueError("temperature must be finite and not negative")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must lie in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")
        if self.sampler not in SAMPLERS:
            raise ValueError(f"sampler must be one of {sorted(SAMPLERS)}")
        if not 0 <= self.seed < 1 << 64 or not 0 <= self.stream < 1 << 64:
            raise ValueError("seed and stream must fit 64 bits")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    @property
    def truncates(self) -> bool:
        return self.top_p < 1.0 or self.top_k > 0


def _u64(values: Sequence[int], device) -> torch.Tensor:
    signed = [v - (1 << 64) if v >= 1 << 63 else v for v in values]
    return torch.tensor(signed, dtype=torch.int64, device=device)


def pick(logits: torch.Tensor, params: Sequence[SamplingParams],
         generated_positions: Sequence[int]) -> torch.Tensor:
    """Token ids (int32, on the device) for logits ``[rows, vocab]``; row r is
    drawn with ``params[r]`` at generated position ``generated_positions[r]``."""
    rows = logits.shape[0]
    if len(params) != rows or len(generated_positions) != rows:
        raise ValueError("one SamplingParams and one position per row")
    methods = [GREEDY if p.greedy else SAMPLERS[p.sampler] for p in params]
    if all(m == GREEDY for m in methods):
        return ops.argmax(logits)
    device = logits.device
    temperature = torch.tensor([p.temperature if not p.greedy else 1.0 for p in params],
                               dtype=torch.float64, device=device)
    seed = _u64([p.seed for p in params], device)
    stream = _u64([p.stream for p in params], device)
    position = torch.tensor(list(generated_positions), dtype=torch.int32, device=device)
    legal = None
    if any(p.truncates and not p.greedy for p in params):
        top_p = torch.tensor([p.top_p if not p.greedy else 1.0 for p in params],
                             dtype=torch.float64, device=device)
        top_k = torch.tensor([p.top_k if not p.greedy else 0 for p in params],
                             dtype=torch.int32, device=device)
        legal = ops.nucleus_mask(logits, temperature, top_p, top_k)
    result = None
    method = torch.tensor(methods, dtype=torch.int32, device=device)
    for code in sorted(set(methods)):
        if code == GREEDY:
            ids = ops.argmax(logits)
        elif code == ICDF:
            ids = ops.sample_icdf(logits, temperature, seed, stream, position, legal)
        else:
            ids = ops.sample_race(logits, temperature, seed, position, legal)
        result = ids if result is None else torch.where(method == code, ids, result)
    return result
