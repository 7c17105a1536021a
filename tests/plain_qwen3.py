"""A plain, slow implementation of the Qwen3 dense decoder in numpy.

Whole sequences, no cache, one function for each part, float64 by default.
It shares no code with ``metallix_b200``: it has its own safetensors reader,
its own configuration reading and its own sampler. It rests on the formulas of
the reference's source (each function cites file:line); the reference's model
code is Rust on MLX/Metal and can be neither imported nor compiled on a Linux
box without a Rust toolchain, so there is no golden output of the reference
itself under ``tests/golden/``; the vectors kept there are the reference's own
published test vectors for its samplers, read from its test files as text.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# --------------------------------------------------------------------- files
def read_safetensors(path):
    """name -> float64 / int64 numpy array. Container layout as described at
    crates/core/checkpoint/src/safetensors.rs:1-9: u64 LE header length, JSON
    header, then the payload."""
    with open(path, "rb") as handle:
        data = handle.read()
    (length,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + length])
    payload = data[8 + length:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        begin, end = info["data_offsets"]
        raw = payload[begin:end]
        kind = info["dtype"]
        if kind == "F32":
            values = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif kind == "F64":
            values = np.frombuffer(raw, dtype="<f8").astype(np.float64)
        elif kind == "F16":
            values = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        elif kind == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            values = bits.view(np.float32).astype(np.float64)
        elif kind in ("I64", "I32"):
            values = np.frombuffer(raw, dtype="<i8" if kind == "I64" else "<i4").astype(np.int64)
        else:
            raise ValueError(f"dtype {kind} of {name}")
        out[name] = values.reshape(info["shape"])
    return out


def read_model(model_dir):
    """(config dict, tensors) of a folder with config.json and *.safetensors."""
    with open(os.path.join(model_dir, "config.json")) as handle:
        config = json.load(handle)
    tensors = {}
    for name in sorted(os.listdir(model_dir)):
        if name.endswith(".safetensors"):
            tensors.update(read_safetensors(os.path.join(model_dir, name)))
    if "embed_tokens.weight" in tensors:  # bare names, checkpoint.rs:193-233
        tensors = {(k if k.startswith("lm_head.") else "model." + k): v
                   for k, v in tensors.items()}
    return config, tensors


def f32(value):
    """The reference keeps eps and theta as f32 (forward.rs:388-389)."""
    return float(np.float32(value))


def bf16_round(x):
    """Round-to-nearest-even to bfloat16, kept in the array's own dtype."""
    as32 = np.asarray(x, dtype=np.float32)
    bits = as32.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).astype(np.asarray(x).dtype)


# --------------------------------------------------------------------- parts
def embed(table, ids):
    """x0[t] = E[id_t] (projection.rs:208-216); ids are checked first
    (forward.rs:2238-2249)."""
    ids = np.asarray(ids, dtype=np.int64)
    if ids.size == 0 or ids.min() < 0 or ids.max() >= table.shape[0]:
        raise ValueError("token id outside the vocabulary")
    return table[ids]


def rms_norm(x, weight, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w over the last axis; the weight
    multiplies directly (forward.rs:2442-2449)."""
    mean_square = np.mean(x * x, axis=-1, keepdims=True)
    return x / np.sqrt(mean_square + eps) * weight


def rope_half(x, positions, theta):
    """Rotate-half over the full head (forward.rs:2031-2054: dims = head_dim,
    traditional = false, base = rope_theta, scale 1). x: [T, heads, hd].
    For i < hd/2: f_i = theta^(-2i/hd),
    out[i] = x[i] cos(p f_i) - x[i+hd/2] sin(p f_i),
    out[i+hd/2] = x[i+hd/2] cos(p f_i) + x[i] sin(p f_i)
    (sign convention as restated on the CPU at
    crates/models/julia/src/encoder.rs:614-631)."""
    hd = x.shape[-1]
    half = hd // 2
    index = np.arange(half, dtype=np.float64)
    frequency = theta ** (-2.0 * index / hd)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * frequency[None, :]
    cos = np.cos(angle)[:, None, :].astype(x.dtype)
    sin = np.sin(angle)[:, None, :].astype(x.dtype)
    first, second = x[..., :half], x[..., half:]
    return np.concatenate([first * cos - second * sin, second * cos + first * sin], axis=-1)


def causal_gqa_attention(q, k, v, scale, window=None):
    """softmax(q k^T * scale) v with a causal mask; query head j uses key/value
    head j // (H / KV) (forward.rs:1967-1989; grouping by head-count ratio).
    q: [T, H, hd], k and v: [T, KV, hd]. ``window``: a query at position p sees
    keys p-window+1 .. p (not part of Qwen3, used by kernel tests)."""
    tokens, heads, _ = q.shape
    group = heads // k.shape[1]
    out = np.zeros_like(q)
    position = np.arange(tokens)
    allowed = position[None, :] <= position[:, None]
    if window is not None:
        allowed &= position[None, :] > position[:, None] - window
    for head in range(heads):
        scores = (q[:, head, :] @ k[:, head // group, :].T) * scale
        scores = np.where(allowed, scores, -np.inf)
        scores = scores - scores.max(axis=-1, keepdims=True)
        weights = np.exp(scores)
        weights = weights / weights.sum(axis=-1, keepdims=True)
        out[:, head, :] = weights @ v[:, head // group, :]
    return out


def swiglu(x, gate_w, up_w, down_w, rounding=None):
    """d = ((sigmoid(g) * g) * u) Wd^T with g = x Wg^T, u = x Wu^T
    (forward.rs:1904-1920)."""
    r = rounding or (lambda a: a)
    gate = r(x @ gate_w.T)
    up = r(x @ up_w.T)
    activated = gate / (1.0 + np.exp(-gate))
    return r(r(activated * up) @ down_w.T)


def attention_block(x, positions, w, base, config, rounding=None, window=None, shared_kv=None,
                    keep=None):
    """q/k/v projections, per-head q/k RMSNorm before RoPE, attention, output
    projection (forward.rs:2012-2065 and :2070-2093). ``shared_kv``: keys and
    values another layer produced, used instead of this layer's own (not part
    of Qwen3; for the tests of the layer order). ``keep``: a list that
    receives this layer's (k, v)."""
    r = rounding or (lambda a: a)
    tokens = x.shape[0]
    heads, kv_heads, hd = (config["num_attention_heads"], config["num_key_value_heads"],
                           config["head_dim"])
    eps = f32(config.get("rms_norm_eps", 1e-6))
    theta = f32(config.get("rope_theta", 1e6))
    q = r(x @ w[f"{base}.q_proj.weight"].T).reshape(tokens, heads, hd)
    k = r(x @ w[f"{base}.k_proj.weight"].T).reshape(tokens, kv_heads, hd)
    v = r(x @ w[f"{base}.v_proj.weight"].T).reshape(tokens, kv_heads, hd)
    q = rms_norm(q, w[f"{base}.q_norm.weight"], eps)
    k = rms_norm(k, w[f"{base}.k_norm.weight"], eps)
    q = r(rope_half(q, positions, theta))
    k = r(rope_half(k, positions, theta))
    if keep is not None:
        keep.append((k, v))
    if shared_kv is not None:
        k, v = shared_kv
    scale = float(np.float32(hd) ** np.float32(-0.5))  # forward.rs:2290-2295
    out = r(causal_gqa_attention(q, k, v, scale, window))
    return r(out.reshape(tokens, heads * hd) @ w[f"{base}.o_proj.weight"].T)


def decoder_layer(x, positions, w, layer, config, rounding=None, shared_kv=None, keep=None):
    """Pre-norm attention, residual, pre-norm SwiGLU, residual
    (forward.rs:1856-1885 and :1889-1922)."""
    r = rounding or (lambda a: a)
    base = f"model.layers.{layer}"
    eps = f32(config.get("rms_norm_eps", 1e-6))
    attention_in = r(rms_norm(x, w[f"{base}.input_layernorm.weight"], eps))
    residual = x + attention_block(attention_in, positions, w, f"{base}.self_attn", config,
                                   rounding, shared_kv=shared_kv, keep=keep)
    mlp_in = r(rms_norm(residual, w[f"{base}.post_attention_layernorm.weight"], eps))
    return residual + swiglu(mlp_in, w[f"{base}.mlp.gate_proj.weight"],
                             w[f"{base}.mlp.up_proj.weight"],
                             w[f"{base}.mlp.down_proj.weight"], rounding)


def forward_logits(config, tensors, ids, dtype=np.float64, bf16_activations=False,
                   order=None, reads=None, rows=None):
    """Logits [T, V] at every position of one whole sequence (forward.rs:741-773,
    :995-1020): embedding, the layers in order, final norm, output head through
    the embedding when tied, else lm_head (forward.rs:574-580; an absent
    tie_word_embeddings is false, :2606-2607). ``bf16_activations`` rounds
    activations to bfloat16 where a bfloat16 engine stores them, keeping the
    residual sum unrounded. ``order`` runs the layers in another order;
    ``reads[i] = j`` lets the i-th run use the keys and values the j-th run
    produced. ``rows``: only these positions go through the final norm and the
    head (forward.rs:1585-1597 norms the requested rows only); the result is
    then [len(rows), V]."""
    w = {name: value.astype(dtype, copy=False) for name, value in tensors.items()}
    rounding = bf16_round if bf16_activations else None
    r = rounding or (lambda a: a)
    positions = np.arange(len(ids))
    x = embed(w["model.embed_tokens.weight"], ids)
    layers = range(config["num_hidden_layers"]) if order is None else order
    produced = []
    for run, layer in enumerate(layers):
        keep = []
        shared = produced[reads[run]] if reads and run in reads else None
        x = decoder_layer(x, positions, w, layer, config, rounding, shared_kv=shared, keep=keep)
        produced.append(keep[0])
    eps = f32(config.get("rms_norm_eps", 1e-6))
    if rows is not None:
        x = x[np.asarray(rows, dtype=np.int64)]
    normed = r(rms_norm(x, w["model.norm.weight"], eps))
    head = (w["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False)
            else w["lm_head.weight"])
    return normed @ head.T


# ------------------------------------------------------------------ sampling
def greedy_pick(logits):
    """First maximum; a non-finite row is an error (qwen_forward.rs:1546-1557)."""
    row = np.asarray(logits, dtype=np.float64)
    if not np.all(np.isfinite(row)):
        raise ValueError("non-finite logits")
    return int(np.argmax(row))


def sample_categorical(logits, temperature, uniform, legal=None):
    """Inverse CDF in token-id order over exp((logit - max) / T) in float64:
    target = u * sum, the first id whose cumulative weight exceeds the target,
    else the last id of positive weight
    (crates/core/engine/src/sampling.rs:56-103)."""
    row = np.asarray(logits, dtype=np.float32).astype(np.float64)
    if not np.all(np.isfinite(row)):
        raise ValueError("non-finite logits")
    if not (math.isfinite(temperature) and temperature > 0.0):
        raise ValueError("temperature must be positive")
    if not 0.0 <= uniform < 1.0:
        raise ValueError("uniform outside [0, 1)")
    legal = np.ones(row.shape, dtype=bool) if legal is None else np.asarray(legal, dtype=bool)
    if not legal.any():
        raise ValueError("empty support")
    maximum = row[legal].max()
    total = 0.0
    for index in range(row.size):  # id order, as sampling.rs:142-147
        if legal[index]:
            total += math.exp((row[index] - maximum) / temperature)
    target = uniform * total
    cumulative = 0.0
    last_positive = None
    for index in range(row.size):
        if not legal[index]:
            continue
        weight = math.exp((row[index] - maximum) / temperature)
        cumulative += weight
        if weight > 0.0:
            last_positive = index
        if target < cumulative:
            return index
    return last_positive


def nucleus_mask(logits, temperature, top_p, top_k=None):
    """Legal set of top-k then top-p: descending logit, lower id first on ties,
    the first top_k, then the shortest prefix whose mass reaches top_p of the
    kept mass (qwen_forward.rs:474-549)."""
    row = np.asarray(logits, dtype=np.float32).astype(np.float64)
    size = row.size
    if top_k is not None and not 0 < top_k < size:
        top_k = None
    if top_p >= 1.0 and top_k is None:
        return np.ones(size, dtype=bool)
    weights = np.exp((row - row.max()) / temperature)
    # f32::total_cmp (qwen_forward.rs:498-502): -0.0 sorts below +0.0
    bits = np.asarray(logits, dtype=np.float32).view(np.uint32).astype(np.int64)
    total_order = np.where(bits & 0x80000000, 0xFFFFFFFF - bits, bits | 0x80000000)
    order = sorted(range(size), key=lambda i: (-total_order[i], i))
    if top_k is not None:
        order = order[:top_k]
    kept = sum(weights[i] for i in order)
    mask = np.zeros(size, dtype=bool)
    covered = 0.0
    for index in order:
        mask[index] = True
        covered += weights[index]
        if covered >= top_p * kept:
            break
    return mask


_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85


def philox4x32_10(counter, key):
    """Philox4x32 with ten rounds (crates/core/engine/src/sampling/race.rs:40-53)."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for round_index in range(10):
        if round_index:
            k0 = (k0 + _W0) & 0xFFFFFFFF
            k1 = (k1 + _W1) & 0xFFFFFFFF
        p0, p1 = _M0 * c0, _M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & 0xFFFFFFFF, p1 & 0xFFFFFFFF, \
            ((p0 >> 32) ^ c3 ^ k1) & 0xFFFFFFFF, p0 & 0xFFFFFFFF
    return c0, c1, c2, c3


def race_bits(seed, choice, position, row):
    """64 noise bits of one vocabulary row (race.rs:68-86): key = seed's low and
    high words, counter = (row >> 1, position, choice, "race"); an even row
    takes words 0 and 1, an odd row words 2 and 3, high word first."""
    words = philox4x32_10((row >> 1, position, choice, 0x72616365),
                          (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    high, low = (words[0], words[1]) if row % 2 == 0 else (words[2], words[3])
    return (high << 32) | low


def gumbel_from_bits(bits):
    """-ln E with E = -ln(1 - w), w = (bits + 1/2) 2^-64, each half of the
    range in the form that keeps relative precision (race.rs:88-105)."""
    two_to_minus_64 = 1.0 / 18446744073709551616.0
    if bits < 1 << 63:
        exponential = -math.log1p(-((float(bits) + 0.5) * two_to_minus_64))
    else:
        exponential = -math.log((float(bits ^ 0xFFFFFFFFFFFFFFFF) + 0.5) * two_to_minus_64)
    return -math.log(exponential)


def sample_race(logits, temperature, seed, position, choice=0, legal=None):
    """Gumbel-max: the legal row maximizing f64(logit) / T + noise, lowest row
    on ties (race.rs:107-160)."""
    row = np.asarray(logits, dtype=np.float32).astype(np.float64)
    if not np.all(np.isfinite(row)):
        raise ValueError("non-finite logits")
    best, best_score = None, None
    for index in range(row.size):
        if legal is not None and not legal[index]:
            continue
        score = row[index] / temperature + gumbel_from_bits(race_bits(seed, choice, position, index))
        if best is None or score > best_score:
            best, best_score = index, score
    return best


def unit_uniform(word):
    """Top 53 bits of a 64-bit word over 2^53 (qwen_forward.rs:551-559)."""
    return float(word >> 11) / 9007199254740992.0


def request_uniform(seed, stream, position):
    """The uniform of generated position ``position`` of a request: Philox
    words 0 (high) and 1 (low) with key = seed halves and counter
    (position, stream low, stream high, "icdf"), through ``unit_uniform``.
    The reference draws from a ChaCha8 stream (qwen_forward.rs:175-208); a
    counter keyed by position gives the same token whatever else is in the
    batch, which is what its race sampler is for (race.rs:3-10)."""
    words = philox4x32_10((position & 0xFFFFFFFF, stream & 0xFFFFFFFF,
                           (stream >> 32) & 0xFFFFFFFF, 0x69636466),
                          (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    return unit_uniform((words[0] << 32) | words[1])


def generate(config, tensors, prompt, max_new_tokens, pick, dtype=np.float64):
    """Greedy or sampled generation by recomputing the whole sequence for
    every token. ``pick(logits_row, generated_position) -> id``."""
    ids = list(prompt)
    out = []
    for position in range(max_new_tokens):
        logits = forward_logits(config, tensors, ids, dtype=dtype)[-1]
        token = pick(logits, position)
        out.append(token)
        ids.append(token)
    return out
