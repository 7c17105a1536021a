"""Loads a model folder's tensors by name.

Discovery, naming and the required-tensor check follow the reference's
``Qwen3CheckpointInspection`` (``crates/models/qwen/src/checkpoint.rs:51-134``):
every regular ``*.safetensors`` file of the folder in sorted order (``:235-269``),
bare or ``model.``-prefixed names made canonical (``:193-233``), every required
tensor present with the configured shape (``:772-875``). Unlike the reference,
which stops at the first problem, all problems of a folder are gathered into
one error that lists missing tensors, unexpected tensors and wrong shapes.

Tensors keep the dtype they are stored with: bfloat16 stays bfloat16, a tensor
stored in 32 bits stays in 32 bits, integer tables become int32. The parts cast
what they need when they are built.
"""
from __future__ import annotations

import mmap
import os
from typing import Dict, List, Mapping, Tuple

import torch

from .safetensors_io import DTYPES, CheckpointError, TensorEntry, read_header

_FLOATS = ("F32", "BF16", "F16")
_INTEGERS = ("I64", "I32", "I16", "I8", "U8")


def discover(model_dir: str) -> List[str]:
    if not os.path.isdir(model_dir):
        raise CheckpointError("NotDirectory", model_dir)
    paths = sorted(
        os.path.join(model_dir, name) for name in os.listdir(model_dir)
        if name.endswith(".safetensors") and os.path.isfile(os.path.join(model_dir, name)))
    if not paths:
        raise CheckpointError("NoSafetensors", f"{model_dir} holds no *.safetensors file")
    return paths


def canonical_names(entries: Mapping[str, TensorEntry]) -> Dict[str, TensorEntry]:
    """Bare names (``embed_tokens.weight``) become ``model.``-prefixed; a folder
    that holds both spellings is ambiguous (``checkpoint.rs:193-233``)."""
    bare = "embed_tokens.weight" in entries
    prefixed = "model.embed_tokens.weight" in entries
    if bare and prefixed:
        raise CheckpointError("AmbiguousTensorNaming",
                              "both embed_tokens.weight and model.embed_tokens.weight")
    if not bare:
        return dict(entries)
    out = {}
    for name, entry in entries.items():
        canonical = name if name.startswith("lm_head.") else f"model.{name}"
        out[canonical] = entry
    return out


def inspect(model_dir: str, config) -> Dict[str, TensorEntry]:
    """Headers of the whole folder, checked against ``config.tensor_shapes()``."""
    entries: Dict[str, TensorEntry] = {}
    for path in discover(model_dir):
        found, _ = read_header(path)
        for name, entry in found.items():
            if name in entries:
                raise CheckpointError("DuplicateTensorName", f"{name} in two files")
            entries[name] = entry
    entries = canonical_names(entries)
    required = config.tensor_shapes()
    ignored = set(config.ignored_tensors())
    missing = [name for name in required if name not in entries]
    unexpected = sorted(name for name in entries if name not in required and name not in ignored)
    wrong_shape = [
        f"{name}: expected {list(shape)}, found {list(entries[name].shape)}"
        for name, shape in required.items()
        if name in entries and tuple(entries[name].shape) != tuple(shape)]
    wrong_dtype = [
        f"{name}: {entries[name].dtype}" for name in required
        if name in entries and entries[name].dtype not in _FLOATS + _INTEGERS]
    if missing or unexpected or wrong_shape or wrong_dtype:
        lines = [f"the tensors of {model_dir} do not fit its config.json"]
        for title, items in (("missing", missing), ("unexpected", unexpected),
                             ("wrong shape", wrong_shape), ("unsupported dtype", wrong_dtype)):
            if items:
                lines.append(f"  {title} ({len(items)}): " + "; ".join(items))
        error = CheckpointError("TensorMismatch", "\n".join(lines))
        error.missing, error.unexpected = missing, unexpected
        error.wrong_shape, error.wrong_dtype = wrong_shape, wrong_dtype
        raise error
    return {name: entries[name] for name in required}


def load_tensors(model_dir: str, config, device: str = "cpu") -> Dict[str, torch.Tensor]:
    """All required tensors by canonical name, on ``device``, dtype as stored."""
    entries = inspect(model_dir, config)
    by_path: Dict[str, List[Tuple[str, TensorEntry]]] = {}
    for name, entry in entries.items():
        by_path.setdefault(entry.path, []).append((name, entry))
    tensors: Dict[str, torch.Tensor] = {}
    for path, items in by_path.items():
        with open(path, "rb") as handle, \
                mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_READ) as mapped:
            whole = memoryview(mapped)
            try:
                for name, entry in items:
                    dtype, _ = DTYPES[entry.dtype]
                    start = entry.payload_start + entry.begin
                    piece = whole[start:start + (entry.end - entry.begin)]
                    try:
                        if entry.element_count() == 0:
                            value = torch.empty(entry.shape, dtype=dtype)
                        else:
                            value = torch.frombuffer(bytearray(piece), dtype=torch.uint8) \
                                .view(dtype).reshape(entry.shape)
                    finally:
                        piece.release()
                    if entry.dtype in _INTEGERS:
                        value = value.to(torch.int32)
                    tensors[name] = value.to(device)
            finally:
                whole.release()
    return tensors
