"""The plain implementation itself (no GPU): properties that pin how the
reference's formulas were read, and the reference's own sampler vectors."""
import json
import os
import struct

import numpy as np
import pytest

import plain_qwen3 as plain
from conftest import random_ids

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_sampler_vectors.json")))


def _int(value):
    return int(value, 16) if isinstance(value, str) else value


def test_philox_known_answers():
    for case in GOLDEN["philox4x32_10"]["cases"]:
        out = plain.philox4x32_10(tuple(_int(c) for c in case["counter"]), tuple(_int(k) for k in case["key"]))
        assert list(out) == [_int(o) for o in case["out"]]


def test_race_noise_and_tokens():
    noise = GOLDEN["race_noise"]
    for row in noise["rows"]:
        bits = plain.race_bits(noise["seed"], noise["choice"], noise["position"], row["row"])
        assert bits == _int(row["bits"])
        expected = struct.unpack("<d", struct.pack("<Q", _int(row["noise_f64_bits"])))[0]
        assert abs(plain.gumbel_from_bits(bits) - expected) < 1e-15
    golden = GOLDEN["race_v2_tokens"]
    tokens = [plain.sample_race(golden["logits"], golden["temperature"], golden["seed"], position,
                                golden["choice"], golden["legal"]) for position in range(24)]
    assert tokens == golden["tokens"]


def test_categorical_cases():
    for case in GOLDEN["categorical"]["cases"]:
        token = plain.sample_categorical(case["logits"], case["temperature"], case["uniform"], case["legal"])
        assert token == case["token"], case


def test_categorical_matches_enumeration():
    """The f64 enumeration oracle of sampling.rs:174-223."""
    rng = np.random.default_rng(3)
    for _ in range(200):
        logits = rng.normal(0, 2, size=9).astype(np.float32)
        temperature = float(rng.uniform(0.3, 2.0))
        uniform = float(rng.random())
        probabilities = np.exp(logits.astype(np.float64) / temperature)
        probabilities /= probabilities.sum()
        expected = int(np.searchsorted(np.cumsum(probabilities), uniform, side="right"))
        assert plain.sample_categorical(logits, temperature, uniform) == min(expected, 8)


def test_nucleus_mask():
    logits = [2.0, 1.0, 2.0, 0.0, -1.0, 1.0]
    assert plain.nucleus_mask(logits, 1.0, 1.0, None).all()
    assert plain.nucleus_mask(logits, 1.0, 1.0, 3).tolist() == [True, True, True, False, False, False]
    assert plain.nucleus_mask(logits, 1.0, 1.0, 6).all()          # top_k must be below the size
    # weights e^0, e^-1, e^0, ...: the first two cover 2 / 3.04 = 0.66 of the mass
    assert plain.nucleus_mask(logits, 1.0, 0.6, None).tolist() == [True, False, True, False, False, False]
    assert plain.nucleus_mask(logits, 1.0, 0.3, None).tolist() == [True, False, False, False, False, False]
    assert plain.nucleus_mask(logits, 1.0, 0.9, 3).tolist() == [True, True, True, False, False, False]


def test_greedy_takes_the_first_maximum():
    assert plain.greedy_pick([0.5, 2.0, 2.0, -1.0]) == 1
    with pytest.raises(ValueError):
        plain.greedy_pick([0.0, float("nan")])


def test_rope_is_a_rotation_by_relative_position():
    rng = np.random.default_rng(0)
    q, k = rng.normal(size=(1, 1, 32)), rng.normal(size=(1, 1, 32))
    dots = [float(np.sum(plain.rope_half(q, [p + 5], 1e4) * plain.rope_half(k, [p], 1e4))) for p in (0, 3, 40)]
    assert np.allclose(dots, dots[0], atol=1e-12)
    assert np.allclose(plain.rope_half(q, [0], 1e4), q)
    x = np.zeros((1, 1, 4)); x[0, 0, 0] = 1.0   # first pair (0, 2) has frequency 1
    out = plain.rope_half(x, [1], 1e4)[0, 0]
    assert np.allclose(out, [np.cos(1.0), 0.0, np.sin(1.0), 0.0])


def test_rms_norm_weight_multiplies_directly():
    x = np.array([[3.0, 4.0]])
    assert np.allclose(plain.rms_norm(x, np.array([1.0, 2.0]), 0.0), [[3 / np.sqrt(12.5), 8 / np.sqrt(12.5)]])


def test_attention_is_causal_and_groups_heads(model_folders):
    rng = np.random.default_rng(1)
    q, k, v = rng.normal(size=(6, 4, 8)), rng.normal(size=(6, 2, 8)), rng.normal(size=(6, 2, 8))
    out = plain.causal_gqa_attention(q, k, v, 8 ** -0.5)
    assert np.allclose(out[0, :2], v[0, 0]) and np.allclose(out[0, 2:], v[0, 1])  # one key: its value
    k2, v2 = k.copy(), v.copy()
    k2[4:], v2[4:] = rng.normal(size=(2, 2, 8)), rng.normal(size=(2, 2, 8))
    assert np.allclose(plain.causal_gqa_attention(q, k2, v2, 8 ** -0.5)[:4], out[:4])
    windowed = plain.causal_gqa_attention(q, k, v, 8 ** -0.5, window=1)
    assert np.allclose(windowed[:, 0], v[:, 0])


def test_logits_of_a_prefix_do_not_depend_on_what_follows(model_folders):
    for name in ("A", "B"):
        _, config, tensors, _ = model_folders[name]
        ids = random_ids(5, 24, config["vocab_size"])
        whole = plain.forward_logits(config, tensors, ids)
        prefix = plain.forward_logits(config, tensors, ids[:11])
        assert np.allclose(whole[:11], prefix, atol=1e-12)
        single = plain.forward_logits(config, tensors, ids, dtype=np.float32)
        assert np.abs(single - whole).max() < 1e-4
        assert whole.shape == (24, config["vocab_size"])


def test_tied_and_untied_heads(model_folders):
    _, config_a, tensors_a, _ = model_folders["A"]
    _, config_b, tensors_b, _ = model_folders["B"]
    assert "lm_head.weight" not in tensors_a and "lm_head.weight" in tensors_b
    assert config_a["tie_word_embeddings"] and not config_b["tie_word_embeddings"]


def test_bf16_rounding():
    values = np.array([1.0, 1.00390625, 1.001953125, 1.005859375, -2.5, 3.1415927], dtype=np.float64)
    rounded = plain.bf16_round(values)
    assert rounded[0] == 1.0 and rounded[1] == 1.0 and rounded[4] == -2.5   # 1 + 2^-8 ties to even
    assert rounded[2] == 1.0 and rounded[3] == 1.0078125 and rounded[5] == 3.140625


def test_two_plain_implementations_agree(model_folders):
    """The numpy implementation (whole sequences under a mask) and the torch
    one (one position at a time over growing keys and values, the rotation as
    a complex product, repeated key/value heads, its own file reader) were
    written apart from the same lines of the reference; they must give the
    same logits, also when layers run in another order or share a cache."""
    import plain_qwen3_torch as second
    worst = 0.0
    for name in ("A", "B", "C", "D"):
        folder, config, tensors, _ = model_folders[name]
        other_config, other_tensors = second.load_folder(folder)
        assert other_config == config and set(other_tensors) == set(tensors)
        ids = random_ids(len(name) + 40, 37, config["vocab_size"])
        layers = config["num_hidden_layers"]
        variants = [dict(), dict(order=list(range(layers)) + [0]),             # a layer run twice
                    dict(order=list(range(layers)) + [0], reads={layers: 0})]  # ... reading the first run's cache
        for variant in variants:
            first = plain.forward_logits(config, tensors, ids, **variant)
            again = second.all_logits(other_config, other_tensors, ids, **variant).numpy()
            scale = np.abs(first).max()
            worst = max(worst, float(np.abs(first - again).max() / scale))
            assert np.abs(first - again).max() <= 1e-9 * scale, (name, variant)
    print(f"largest relative difference between the two plain implementations: {worst:.2e}")
