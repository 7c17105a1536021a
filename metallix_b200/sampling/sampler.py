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


class _RowTensors:
    """What the kernels want to know about the rows of a batch, on the device.
    Everything but the generated positions is a function of the rows'
    SamplingParams, which stay the same from step to step while the same
    requests decode: it is built once per batch composition. The positions go
    through pinned memory, without a stop of the host."""

    def __init__(self, params: Sequence[SamplingParams], device):
        self.methods = [GREEDY if p.greedy else SAMPLERS[p.sampler] for p in params]
        self.codes = sorted(set(self.methods))
        self.temperature = torch.tensor([p.temperature if not p.greedy else 1.0 for p in params],
                                        dtype=torch.float64, device=device)
        self.seed = _u64([p.seed for p in params], device)
        self.stream = _u64([p.stream for p in params], device)
        self.truncates = any(p.truncates and not p.greedy for p in params)
        if self.truncates:
            self.top_p = torch.tensor([p.top_p if not p.greedy else 1.0 for p in params],
                                      dtype=torch.float64, device=device)
            self.top_k = torch.tensor([p.top_k if not p.greedy else 0 for p in params],
                                      dtype=torch.int32, device=device)
        self.method = torch.tensor(self.methods, dtype=torch.int32, device=device)
        self.is_code = {code: self.method == code for code in self.codes} if len(self.codes) > 1 else {}
        self.position = torch.zeros(len(params), dtype=torch.int32, device=device)
        # two staging buffers: the copy out of one may still be queued while the next step fills the other
        self.staging = [torch.zeros(len(params), dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.turn = 0

    def positions(self, generated_positions: Sequence[int]) -> torch.Tensor:
        staging = self.staging[self.turn]
        self.turn ^= 1
        staging.numpy()[:] = generated_positions
        self.position.copy_(staging, non_blocking=True)
        return self.position


_ROWS: "dict[tuple, _RowTensors]" = {}
_ROWS_KEPT = 64


def _row_tensors(params: Sequence[SamplingParams], device) -> _RowTensors:
    key = (str(device), tuple(params))
    found = _ROWS.get(key)
    if found is None:
        if len(_ROWS) >= _ROWS_KEPT:
            _ROWS.pop(next(iter(_ROWS)))   # the oldest composition
        found = _ROWS[key] = _RowTensors(params, device)
    return found


def pick(logits: torch.Tensor, params: Sequence[SamplingParams],
         generated_positions: Sequence[int]) -> torch.Tensor:
    """Token ids (int32, on the device) for logits ``[rows, vocab]``; row r is
    drawn with ``params[r]`` at generated position ``generated_positions[r]``."""
    rows = logits.shape[0]
    if len(params) != rows or len(generated_positions) != rows:
        raise ValueError("one SamplingParams and one position per row")
    if all(p.greedy for p in params):
        return ops.argmax(logits)
    row = _row_tensors(params, logits.device)
    position = row.positions(generated_positions)
    legal = ops.nucleus_mask(logits, row.temperature, row.top_p, row.top_k) if row.truncates else None
    result = None
    for code in row.codes:
        if code == GREEDY:
            ids = ops.argmax(logits)
        elif code == ICDF:
            ids = ops.sample_icdf(logits, row.temperature, row.seed, row.stream, position, legal)
        else:
            ids = ops.sample_race(logits, row.temperature, row.seed, position, legal)
        result = ids if result is None else torch.where(row.is_code[code], ids, result)
    return result
