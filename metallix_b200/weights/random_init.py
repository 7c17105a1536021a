"""Random weights for a configuration and a seed, and the model folder they
are written to (``config.json`` + ``model.safetensors``).

The reference has only test-local generators (an arithmetic pattern at
``crates/models/qwen/src/forward.rs:4548-4555``, an LCG at
``forward/tests/paged_kv.rs:49-128`` with norm weights near one). Here linear
and embedding weights are drawn from N(0, 0.02) and every norm weight,
q/k-norms included, from 1 + U(-0.1, 0.1).

The generator is counter-based, as the reference's sampling noise is
(Philox4x32-10, ``crates/core/engine/src/sampling/race.rs:40-86``): element
``i`` of a tensor is a function of (seed, tensor name, i) alone. A tensor's
values therefore do not depend on which other tensors exist, in which order
they are made, or on which device: the words are integer arithmetic, and the
way from words to values uses only operations that IEEE 754 rounds exactly
(+, -, x, /, square root) one at a time, so a CPU and a GPU give the same bits.
``log`` and ``sin``/``cos`` of the Box-Muller transform are series written in
those operations in float64 for that reason.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from typing import Dict, Tuple

import torch

from .safetensors_io import write_file

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}

_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
_MASK32 = 0xFFFFFFFF
_DOMAIN = 0x77677473          # "wgts": keeps these streams apart from the samplers'
_CHUNK_BLOCKS = 1 << 22       # counters worked on at a time (four values each)


def _tensor_key(seed: int, name: str) -> Tuple[int, int]:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:4], "little"), int.from_bytes(digest[4:8], "little")


def _mulhilo(constant: int, value: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """High and low 32-bit words of constant x value (both below 2^32), in
    int64 arithmetic that never leaves 63 bits."""
    low_half, high_half = value & 0xFFFF, value >> 16
    t, u = low_half * constant, high_half * constant
    low_sum = ((u & 0xFFFF) << 16) + (t & _MASK32)
    return (u >> 16) + (t >> 32) + (low_sum >> 32), low_sum & _MASK32


def philox_words(key: Tuple[int, int], first_block: int, blocks: int, device) -> torch.Tensor:
    """int64 [4, blocks]: the four 32-bit output words of Philox4x32-10 for the
    counters (block low word, block high word, 0, domain), block =
    first_block .. first_block + blocks - 1."""
    block = torch.arange(first_block, first_block + blocks, dtype=torch.int64, device=device)
    c0, c1 = block & _MASK32, block >> 32
    c2 = torch.zeros_like(block)
    c3 = torch.full_like(block, _DOMAIN)
    k0, k1 = key
    for round_index in range(10):
        if round_index:
            k0, k1 = (k0 + _W0) & _MASK32, (k1 + _W1) & _MASK32
        high0, low0 = _mulhilo(_M0, c0)
        high1, low1 = _mulhilo(_M1, c2)
        c0, c1, c2, c3 = high1 ^ c1 ^ k0, low1, high0 ^ c3 ^ k1, low0
    return torch.stack([c0, c1, c2, c3])


def _log_unit(u: torch.Tensor) -> torch.Tensor:
    """ln(u) for float64 u in (0, 1): u = m 2^e with m in [sqrt(1/2), sqrt(2)),
    ln m = 2 atanh(s), s = (m - 1) / (m + 1), by its series."""
    m, e = torch.frexp(u)                       # m in [0.5, 1)
    small = m < math.sqrt(0.5)
    m = torch.where(small, m * 2.0, m)
    e = e.to(torch.float64) - small.to(torch.float64)
    s = (m - 1.0) / (m + 1.0)
    s2 = s * s
    p = torch.full_like(s, 1.0 / 25.0)
    for k in range(11, -1, -1):
        p = p * s2 + 1.0 / (2 * k + 1)
    return e * math.log(2.0) + (s * p) * 2.0


def _unit_circle(word: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(cos, sin) of 2 pi word / 2^32: the top two bits choose the quadrant,
    the rest is an angle in [0, pi/2) whose sine and cosine are Taylor sums."""
    quadrant = word >> 30
    theta = (word & ((1 << 30) - 1)).to(torch.float64) * (math.pi / 2.0 / (1 << 30))
    t2 = theta * theta
    terms = 15   # (pi/2)^30 / 30! is below 1e-26
    c = torch.full_like(theta, (-1.0) ** terms / math.factorial(2 * terms))
    s = torch.full_like(theta, (-1.0) ** terms / math.factorial(2 * terms + 1))
    for k in range(terms - 1, -1, -1):
        c = c * t2 + (-1.0) ** k / math.factorial(2 * k)
        s = s * t2 + (-1.0) ** k / math.factorial(2 * k + 1)
    s = s * theta
    cos = torch.where(quadrant == 0, c, torch.where(quadrant == 1, -s, torch.where(quadrant == 2, -c, s)))
    sin = torch.where(quadrant == 0, s, torch.where(quadrant == 1, c, torch.where(quadrant == 2, -s, -c)))
    return cos, sin


def _uniform_values(words: torch.Tensor) -> torch.Tensor:
    """float32 [4 * blocks] in 1 + [-0.1, 0.1): the top 24 bits of each word."""
    unit = (words >> 8).to(torch.float32) * (1.0 / (1 << 24))
    return ((unit * 0.2 - 0.1) + 1.0).t().reshape(-1)


def _normal_values(words: torch.Tensor) -> torch.Tensor:
    """float32 [4 * blocks] of N(0, 0.02): Box-Muller on the word pairs
    (0, 1) and (2, 3) of each counter, radius from the first word of a pair
    (u = (word + 1/2) 2^-32, never 0 or 1), angle from the second."""
    out = []
    for first in (0, 2):
        u = (words[first].to(torch.float64) + 0.5) * (1.0 / (1 << 32))
        radius = torch.sqrt(_log_unit(u) * -2.0)
        cos, sin = _unit_circle(words[first + 1])
        out.extend([(radius * cos).to(torch.float32) * 0.02, (radius * sin).to(torch.float32) * 0.02])
    return torch.stack(out).t().reshape(-1)


def random_tensor(seed: int, name: str, shape, norm: bool, device="cpu") -> torch.Tensor:
    """One tensor's float32 values: element i (row-major) comes from counter
    i // 4, word i % 4 of the stream keyed by (seed, name)."""
    count = 1
    for size in shape:
        count *= int(size)
    key = _tensor_key(seed, name)
    blocks = -(-count // 4)
    flat = torch.empty(blocks * 4, dtype=torch.float32, device=device)
    for first in range(0, blocks, _CHUNK_BLOCKS):
        size = min(_CHUNK_BLOCKS, blocks - first)
        words = philox_words(key, first, size, device)
        flat[first * 4:(first + size) * 4] = _uniform_values(words) if norm else _normal_values(words)
    return flat[:count].reshape(tuple(shape))


def random_tensors(config, seed: int, dtype: str = "bfloat16", device: str = "cpu",
                   norm_dtype: str = None) -> Dict[str, torch.Tensor]:
    """Every tensor of ``config.tensor_shapes()``: float32 values made on
    ``device`` (the same on every device), then rounded to ``dtype`` (norm
    weights to ``norm_dtype``, which defaults to ``dtype``)."""
    matrix_dtype = _DTYPES[dtype]
    vector_dtype = _DTYPES[norm_dtype or dtype]
    tensors: Dict[str, torch.Tensor] = {}
    for name, shape in config.tensor_shapes().items():
        norm = bool(config.norm_tensor(name))
        value = random_tensor(seed, name, shape, norm, device)
        tensors[name] = value.to(vector_dtype if norm else matrix_dtype)
    return tensors


def write_model_folder(model_dir: str, config, seed: int, dtype: str = "bfloat16",
                       norm_dtype: str = None, device: str = "cpu") -> str:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` with
    random weights from ``seed``; returns ``model_dir``. ``device`` is where
    the values are made (a GPU is faster for large models; the file is the
    same)."""
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(config.to_dict(), handle, indent=1)
    tensors = random_tensors(config, seed, dtype=dtype, norm_dtype=norm_dtype, device=device)
    tensors = {name: value.cpu() for name, value in tensors.items()}
    write_file(os.path.join(model_dir, "model.safetensors"), tensors,
               metadata={"format": "pt", "seed": str(seed)},
               order=list(config.tensor_shapes()))
    return model_dir
