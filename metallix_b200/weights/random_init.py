"""Random weights for a configuration and a seed, and the model folder they
are written to (``config.json`` + ``model.safetensors``).

The reference has only test-local generators (an arithmetic pattern at
``crates/models/qwen/src/forward.rs:4548-4555``, an LCG at
``forward/tests/paged_kv.rs:49-128`` with norm weights near one). Here linear
and embedding weights are drawn from N(0, 0.02) and every norm weight,
q/k-norms included, from 1 + U(-0.1, 0.1). Each tensor has a generator of its
own, seeded from the seed and the tensor's name, so a tensor's values do not
depend on which other tensors exist or in which order they are made.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict

import torch

from .safetensors_io import write_file

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensors(config, seed: int, dtype: str = "bfloat16", device: str = "cpu",
                   norm_dtype: str = None) -> Dict[str, torch.Tensor]:
    """Every tensor of ``config.tensor_shapes()``. Values are drawn in float32
    on ``device`` and then rounded to ``dtype`` (norm weights to ``norm_dtype``,
    which defaults to ``dtype``). CPU and CUDA generators differ, so a seed
    names one set of values per device type."""
    matrix_dtype = _DTYPES[dtype]
    vector_dtype = _DTYPES[norm_dtype or dtype]
    tensors: Dict[str, torch.Tensor] = {}
    for name, shape in config.tensor_shapes().items():
        generator = torch.Generator(device=device)
        generator.manual_seed(_tensor_seed(seed, name))
        if config.norm_tensor(name):
            value = torch.rand(shape, generator=generator, device=device, dtype=torch.float32)
            tensors[name] = (1.0 + (value * 0.2 - 0.1)).to(vector_dtype)
        else:
            value = torch.randn(shape, generator=generator, device=device, dtype=torch.float32)
            tensors[name] = (value * 0.02).to(matrix_dtype)
    return tensors


def write_model_folder(model_dir: str, config, seed: int, dtype: str = "bfloat16",
                       norm_dtype: str = None) -> str:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` with
    random weights from ``seed``; returns ``model_dir``."""
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(config.to_dict(), handle, indent=1)
    tensors = random_tensors(config, seed, dtype=dtype, norm_dtype=norm_dtype)
    write_file(os.path.join(model_dir, "model.safetensors"), tensors,
               metadata={"format": "pt", "seed": str(seed)},
               order=list(config.tensor_shapes()))
    return model_dir
