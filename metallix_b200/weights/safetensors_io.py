"""Reading and writing the safetensors container, with the header checks of
the reference's ``crates/models/qwen/src/checkpoint.rs:363-445`` (header) and
``:553-646`` (payload ranges): 8-byte little-endian header length, one JSON map
``name -> {dtype, shape, data_offsets}``, unique names, every range inside the
payload with ``bytes == elements * dtype size``, ranges neither overlapping nor
leaving gaps, and together covering the whole payload.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

HEADER_LIMIT = 100 * 1024 * 1024  # checkpoint.rs: a header beyond 100 MiB is refused

DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {dtype: name for name, (dtype, _) in DTYPES.items()}


class CheckpointError(ValueError):
    """A model folder or file this loader refuses; ``kind`` names the reason
    (the error kinds of ``checkpoint.rs:878`` onward)."""

    def __init__(self, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.kind = kind


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int  # byte offsets inside the payload
    end: int
    path: str
    payload_start: int  # file offset of the payload

    def element_count(self) -> int:
        count = 1
        for extent in self.shape:
            count *= extent
        return count


def _unique_pairs(pairs):
    seen = {}
    for key, value in pairs:
        if key in seen:
            raise CheckpointError("DuplicateTensorName", key)
        seen[key] = value
    return seen


def read_header(path: str) -> Tuple[Dict[str, TensorEntry], Dict[str, str]]:
    """Parses and validates one file's header; returns entries and metadata."""
    size = os.path.getsize(path)
    with open(path, "rb") as handle:
        prefix = handle.read(8)
        if len(prefix) != 8:
            raise CheckpointError("TruncatedHeader", f"{path}: shorter than the 8-byte length")
        (length,) = struct.unpack("<Q", prefix)
        if length > HEADER_LIMIT:
            raise CheckpointError("HeaderTooLarge", f"{path}: header of {length} bytes")
        if 8 + length > size:
            raise CheckpointError("TruncatedHeader",
                                  f"{path}: header of {length} bytes, file of {size}")
        text = handle.read(length)
    try:
        header = json.loads(text.decode("utf-8"), object_pairs_hook=_unique_pairs)
    except (UnicodeDecodeError, json.JSONDecodeError) as error:
        raise CheckpointError("InvalidHeader", f"{path}: {error}") from None
    if not isinstance(header, dict):
        raise CheckpointError("InvalidHeader", f"{path}: the header is not a JSON object")
    metadata = header.pop("__metadata__", {}) or {}
    if not isinstance(metadata, dict) or not all(
            isinstance(k, str) and isinstance(v, str) for k, v in metadata.items()):
        raise CheckpointError("InvalidHeader", f"{path}: __metadata__ must map strings to strings")

    payload_start = 8 + length
    payload = size - payload_start
    entries: Dict[str, TensorEntry] = {}
    for name, info in header.items():
        if not isinstance(info, dict):
            raise CheckpointError("InvalidHeader", f"{path}: entry {name!r} is not an object")
        dtype, shape, offsets = info.get("dtype"), info.get("shape"), info.get("data_offsets")
        if dtype not in DTYPES:
            raise CheckpointError("UnsupportedTensorDtype", f"{name}: dtype {dtype!r}")
        if not (isinstance(shape, list) and all(
                isinstance(e, int) and not isinstance(e, bool) and e >= 0 for e in shape)):
            raise CheckpointError("InvalidHeader", f"{name}: shape {shape!r}")
        if not (isinstance(offsets, list) and len(offsets) == 2 and all(
                isinstance(e, int) and not isinstance(e, bool) and e >= 0 for e in offsets)):
            raise CheckpointError("InvalidHeader", f"{name}: data_offsets {offsets!r}")
        begin, end = offsets
        entry = TensorEntry(name, dtype, tuple(shape), begin, end, path, payload_start)
        if begin > end or end > payload:
            raise CheckpointError("TensorOutOfRange",
                                  f"{name}: bytes {begin}..{end} of a {payload}-byte payload")
        if end - begin != entry.element_count() * DTYPES[dtype][1]:
            raise CheckpointError(
                "TensorSizeMismatch",
                f"{name}: {end - begin} bytes for shape {list(shape)} of {dtype}")
        entries[name] = entry
    cursor = 0
    for entry in sorted(entries.values(), key=lambda e: (e.begin, e.end)):
        if entry.begin < cursor:
            raise CheckpointError("OverlappingTensors", f"{entry.name} starts inside another tensor")
        if entry.begin > cursor:
            raise CheckpointError("PayloadGap", f"bytes {cursor}..{entry.begin} before {entry.name}")
        cursor = entry.end
    if cursor != payload:
        raise CheckpointError("PayloadGap", f"{path}: bytes {cursor}..{payload} belong to no tensor")
    return entries, metadata


def read_tensor(entry: TensorEntry) -> torch.Tensor:
    """One tensor's values as stored, copied out of the file (CPU)."""
    dtype, _ = DTYPES[entry.dtype]
    count = entry.element_count()
    if count == 0:
        return torch.empty(entry.shape, dtype=dtype)
    with open(entry.path, "rb") as handle:
        with mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_READ) as mapped:
            start = entry.payload_start + entry.begin
            view = memoryview(mapped)[start:start + (entry.end - entry.begin)]
            try:
                flat = torch.frombuffer(bytearray(view), dtype=torch.uint8)
            finally:
                view.release()
    return flat.view(dtype).reshape(entry.shape)


def write_file(path: str, tensors: Mapping[str, torch.Tensor],
               metadata: Mapping[str, str] = None, order: Iterable[str] = None) -> None:
    """Writes ``tensors`` (CPU, any listed dtype) as one safetensors file."""
    names: List[str] = list(order) if order is not None else sorted(tensors)
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    cursor = 0
    blobs = []
    for name in names:
        tensor = tensors[name].detach().cpu().contiguous()
        if tensor.dtype not in _NAMES:
            raise CheckpointError("UnsupportedTensorDtype", f"{name}: {tensor.dtype}")
        blob = tensor.reshape(-1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [cursor, cursor + len(blob)]}
        cursor += len(blob)
        blobs.append(blob)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)  # keep the payload 8-byte aligned
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(text)))
        handle.write(text)
        for blob in blobs:
            handle.write(blob)
