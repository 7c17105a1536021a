"""Safetensors container, by-name loading and its one clear error, random
weights (no GPU). Cases after the reference's header tests in
crates/models/qwen/src/checkpoint/tests.rs."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from conftest import TINY_A, TINY_B
from metallix_b200 import Qwen3Config, load_tensors, random_tensors, write_model_folder
from metallix_b200.weights import CheckpointError, inspect, read_header, write_file


def _write_raw(path, header, payload):
    text = json.dumps(header).encode()
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(text)) + text + payload)


def test_round_trip_all_dtypes(tmp_path):
    tensors = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
               "b": torch.tensor([1.5, -2.25], dtype=torch.bfloat16),
               "c": torch.tensor([[1, 2], [3, 4]], dtype=torch.int64)}
    path = str(tmp_path / "x.safetensors")
    write_file(path, tensors, metadata={"format": "pt"})
    entries, metadata = read_header(path)
    assert metadata == {"format": "pt"} and set(entries) == {"a", "b", "c"}
    assert entries["a"].shape == (2, 3) and entries["b"].dtype == "BF16"
    theirs = plain.read_safetensors(path)  # the plain reader agrees on the bytes
    assert np.array_equal(theirs["a"], tensors["a"].double().numpy())
    assert np.array_equal(theirs["b"], tensors["b"].double().numpy())


@pytest.mark.parametrize("header, payload, kind", [
    ({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4, "TensorOutOfRange"),
    ({"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8, "TensorSizeMismatch"),
    ({"t": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
      "u": {"dtype": "F32", "shape": [1], "data_offsets": [2, 6]}}, b"\0" * 6, "OverlappingTensors"),
    ({"t": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
      "u": {"dtype": "F32", "shape": [1], "data_offsets": [8, 12]}}, b"\0" * 12, "PayloadGap"),
    ({"t": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 8, "PayloadGap"),
    ({"t": {"dtype": "Q4", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4, "UnsupportedTensorDtype"),
    ({"__metadata__": {"n": 1}, "t": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}},
     b"\0" * 4, "InvalidHeader"),
])
def test_header_refusals(tmp_path, header, payload, kind):
    path = str(tmp_path / "bad.safetensors")
    _write_raw(path, header, payload)
    with pytest.raises(CheckpointError) as error:
        read_header(path)
    assert error.value.kind == kind


def test_truncated_and_duplicate(tmp_path):
    path = str(tmp_path / "short.safetensors")
    with open(path, "wb") as handle:
        handle.write(b"\x10\0\0")
    with pytest.raises(CheckpointError) as error:
        read_header(path)
    assert error.value.kind == "TruncatedHeader"
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(CheckpointError) as error:
        read_header(path)
    assert error.value.kind == "TruncatedHeader"
    text = b'{"t":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"t":{"dtype":"F32","shape":[1],"data_offsets":[4,8]}}'
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(text)) + text + b"\0" * 8)
    with pytest.raises(CheckpointError) as error:
        read_header(path)
    assert error.value.kind == "DuplicateTensorName"


def test_random_folder_loads_by_name(tmp_path):
    for raw, seed in ((TINY_A, 0), (TINY_B, 1)):
        config = Qwen3Config.from_dict(raw)
        folder = write_model_folder(str(tmp_path / f"m{seed}"), config, seed)
        assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
        tensors = load_tensors(folder, config)
        assert set(tensors) == set(config.tensor_shapes())
        for name, shape in config.tensor_shapes().items():
            assert tuple(tensors[name].shape) == shape and tensors[name].dtype == torch.bfloat16
        assert ("lm_head.weight" in tensors) == (not config.tie_word_embeddings)
        # statistics of the two kinds of tensors
        matrix = tensors["model.layers.0.mlp.gate_proj.weight"].float()
        assert abs(float(matrix.std()) - 0.02) < 0.002 and abs(float(matrix.mean())) < 0.002
        norm = tensors["model.layers.0.self_attn.q_norm.weight"].float()
        assert float(norm.min()) >= 0.9 - 2 ** -8 and float(norm.max()) <= 1.1 + 2 ** -7  # one bfloat16 step
        # the same seed gives the same values, another seed other values
        again = random_tensors(config, seed)
        other = random_tensors(config, seed + 1)
        assert torch.equal(again["model.norm.weight"], tensors["model.norm.weight"])
        assert not torch.equal(other["model.embed_tokens.weight"], tensors["model.embed_tokens.weight"])


def test_random_values_come_from_a_counter():
    """Element i of a tensor depends on (seed, name, i) alone: a tensor made
    alone, as part of a larger one, or in another order has the same values,
    and the Philox words are those of the plain implementation."""
    import plain_qwen3 as plain
    from metallix_b200.weights import random_init
    key = random_init._tensor_key(4, "model.norm.weight")
    words = random_init.philox_words(key, (1 << 32) - 2, 4, "cpu")   # across the low word's carry
    for column in range(4):
        block = (1 << 32) - 2 + column
        want = plain.philox4x32_10((block & 0xFFFFFFFF, block >> 32, 0, random_init._DOMAIN), key)
        assert tuple(int(words[row, column]) for row in range(4)) == want
    small = random_init.random_tensor(9, "w", (7,), False)
    large = random_init.random_tensor(9, "w", (5, 1000), False)
    assert torch.equal(small, large.reshape(-1)[:7])
    assert not torch.equal(small, random_init.random_tensor(9, "v", (7,), False))
    # N(0, 0.02): moments of a million values, and tails beyond four sigma exist
    values = random_init.random_tensor(1, "moments", (1000, 1000), False).double() / 0.02
    assert abs(float(values.mean())) < 5e-3 and abs(float(values.std()) - 1.0) < 5e-3
    assert abs(float((values ** 4).mean()) - 3.0) < 0.05 and float(values.abs().max()) > 4.0
    # the series behind the transform against the library functions
    u = torch.rand(10000, dtype=torch.float64).clamp_min(2.0 ** -33)
    assert float((random_init._log_unit(u) - torch.log(u)).abs().max()) < 1e-14
    word = torch.randint(0, 1 << 32, (10000,), dtype=torch.int64)
    cos, sin = random_init._unit_circle(word)
    angle = word.double() * (2.0 * torch.pi / (1 << 32))
    assert float((cos - torch.cos(angle)).abs().max()) < 1e-14 and float((sin - torch.sin(angle)).abs().max()) < 1e-14


@pytest.mark.gpu
def test_random_values_are_the_same_on_cpu_and_gpu():
    from metallix_b200.weights import random_init
    for norm in (False, True):
        host = random_init.random_tensor(11, "model.layers.0.mlp.up_proj.weight", (257, 1031), norm, "cpu")
        device = random_init.random_tensor(11, "model.layers.0.mlp.up_proj.weight", (257, 1031), norm, "cuda")
        assert torch.equal(host, device.cpu())
    config = Qwen3Config.from_dict(TINY_B)
    host, device = random_tensors(config, 2), random_tensors(config, 2, device="cuda")
    assert all(torch.equal(host[name], device[name].cpu()) for name in host)


def test_stored_dtype_is_kept(tmp_path):
    config = Qwen3Config.from_dict(TINY_A)
    folder = write_model_folder(str(tmp_path / "mixed"), config, 3, dtype="bfloat16", norm_dtype="float32")
    tensors = load_tensors(folder, config)
    assert tensors["model.norm.weight"].dtype == torch.float32           # stored in 32 bits: stays
    assert tensors["model.embed_tokens.weight"].dtype == torch.bfloat16  # stored in bfloat16: stays
    tensors32 = load_tensors(write_model_folder(str(tmp_path / "f32"), config, 3, dtype="float32"), config)
    assert tensors32["model.embed_tokens.weight"].dtype == torch.float32


def test_integer_tables_become_int32(tmp_path):
    class WithTable:
        def tensor_shapes(self):
            return {"model.embed_tokens.weight": (2, 2), "model.table": (3,)}

        def ignored_tensors(self):
            return ()
    folder = tmp_path / "ints"
    folder.mkdir()
    write_file(str(folder / "model.safetensors"),
               {"model.embed_tokens.weight": torch.zeros(2, 2), "model.table": torch.tensor([1, 2, 3])})
    assert load_tensors(str(folder), WithTable())["model.table"].dtype == torch.int32


def test_one_error_lists_everything(tmp_path):
    config = Qwen3Config.from_dict(TINY_B)
    tensors = random_tensors(config, 5)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(8, 8, dtype=torch.bfloat16)
    tensors["model.layers.9.extra.weight"] = torch.zeros(2, dtype=torch.bfloat16)
    folder = tmp_path / "broken"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(config.to_dict()))
    write_file(str(folder / "model.safetensors"), tensors)
    with pytest.raises(CheckpointError) as error:
        inspect(str(folder), config)
    text = str(error.value)
    assert error.value.kind == "TensorMismatch"
    assert error.value.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.value.unexpected == ["model.layers.9.extra.weight"]
    assert "model.layers.0.self_attn.k_proj.weight: expected [64, 96], found [8, 8]" in text
    for name in error.value.missing + error.value.unexpected:
        assert name in text


def test_bare_names_tied_stray_head_and_ambiguity(tmp_path):
    config = Qwen3Config.from_dict(TINY_A)
    tensors = random_tensors(config, 6)
    bare = {name[len("model."):]: value for name, value in tensors.items()}
    bare["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()  # tied: dropped, metal.rs:778-784
    folder = tmp_path / "bare"
    folder.mkdir()
    write_file(str(folder / "model.safetensors"), bare)
    loaded = load_tensors(str(folder), config)
    assert set(loaded) == set(config.tensor_shapes())
    bare["model.embed_tokens.weight"] = tensors["model.embed_tokens.weight"]
    write_file(str(folder / "model.safetensors"), bare)
    with pytest.raises(CheckpointError) as error:
        load_tensors(str(folder), config)
    assert error.value.kind == "AmbiguousTensorNaming"


def test_sharded_folder_and_missing_files(tmp_path):
    config = Qwen3Config.from_dict(TINY_A)
    tensors = random_tensors(config, 7)
    names = sorted(tensors)
    folder = tmp_path / "shards"
    folder.mkdir()
    write_file(str(folder / "model-00001-of-00002.safetensors"), {n: tensors[n] for n in names[::2]})
    write_file(str(folder / "model-00002-of-00002.safetensors"), {n: tensors[n] for n in names[1::2]})
    loaded = load_tensors(str(folder), config)
    assert all(torch.equal(loaded[n], tensors[n]) for n in names)
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(CheckpointError) as error:
        load_tensors(str(empty), config)
    assert error.value.kind == "NoSafetensors"
    with pytest.raises(CheckpointError) as error:
        load_tensors(str(tmp_path / "nowhere"), config)
    assert error.value.kind == "NotDirectory"
