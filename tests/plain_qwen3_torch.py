"""A second plain implementation of the Qwen3 dense decoder, in torch on the
CPU, written on its own from the reference's formulas to check the reading
that ``plain_qwen3.py`` rests on (the reference itself cannot be run here: it
is Rust on MLX/Metal). It shares nothing with ``plain_qwen3.py`` nor with
``metallix_b200``, and it is decomposed another way on purpose:

* one position at a time with a growing list of keys and values per layer,
  as the reference's cached path does (``forward.rs:1856-1885``), instead of a
  whole sequence under a mask;
* the rotation as a complex product (x[i] + j x[i + hd/2]) e^{j p f_i}
  (rotate-half, ``forward.rs:2031-2054`` with ``traditional = false``);
* key/value heads repeated to the query heads (the library call the
  reference makes takes H query heads and KV key/value heads in contiguous
  groups, ``forward.rs:1967-1989``) instead of an index j // group;
* its own reader of the safetensors container.

float64 throughout. The two implementations must agree to about 1e-9.
"""
from __future__ import annotations

import json
import os
import struct

import torch

_KINDS = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
          "I64": torch.int64, "I32": torch.int32}


def load_folder(folder):
    """(config, {canonical name: float64 tensor})."""
    with open(os.path.join(folder, "config.json"), encoding="utf-8") as handle:
        config = json.load(handle)
    found = {}
    for file_name in sorted(os.listdir(folder)):
        if not file_name.endswith(".safetensors"):
            continue
        with open(os.path.join(folder, file_name), "rb") as handle:
            blob = handle.read()
        (header_bytes,) = struct.unpack_from("<Q", blob, 0)
        table = json.loads(blob[8:8 + header_bytes].decode("utf-8"))
        base = 8 + header_bytes
        for name, entry in table.items():
            if name == "__metadata__":
                continue
            lo, hi = entry["data_offsets"]
            flat = torch.frombuffer(bytearray(blob[base + lo:base + hi]), dtype=_KINDS[entry["dtype"]])
            found[name] = flat.reshape(entry["shape"]).to(torch.float64)
    if "embed_tokens.weight" in found and "model.embed_tokens.weight" not in found:
        # bare names become prefixed ones (checkpoint.rs:193-233)
        found = {(n if n.startswith("lm_head.") else "model." + n): t for n, t in found.items()}
    return config, found


class CachedDecoder:
    """Feeds tokens one by one; keeps per layer the keys and values so far."""

    def __init__(self, config, tensors):
        self.c, self.t = config, tensors
        self.layers = config["num_hidden_layers"]
        self.heads = config["num_attention_heads"]
        self.kv_heads = config["num_key_value_heads"]
        self.hd = config["head_dim"]
        # eps and theta are f32 fields of the reference's config (forward.rs:388-389)
        self.eps = float(torch.tensor(config.get("rms_norm_eps", 1e-6), dtype=torch.float32))
        self.theta = float(torch.tensor(config.get("rope_theta", 1e6), dtype=torch.float32))
        # scale = (head_dim as f32).powf(-0.5) (forward.rs:2290-2295)
        self.scale = float(torch.tensor(float(self.hd), dtype=torch.float32) ** -0.5)
        pair = torch.arange(self.hd // 2, dtype=torch.float64)
        self.frequency = torch.exp(-torch.log(torch.tensor(self.theta, dtype=torch.float64)) * 2.0 * pair / self.hd)
        self.reset()

    def reset(self):
        self.position = 0
        self.keys, self.values = {}, {}

    def _norm(self, x, name):
        # y = x * rsqrt(mean(x^2) + eps) * w, no "1 + w" (forward.rs:2442-2449)
        return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + self.eps) * self.t[name]

    def _rotate(self, heads_by_width):
        half = self.hd // 2
        as_complex = torch.complex(heads_by_width[:, :half], heads_by_width[:, half:])
        turned = as_complex * torch.polar(torch.ones(half, dtype=torch.float64), self.position * self.frequency)
        return torch.cat([turned.real, turned.imag], dim=-1)

    def _attention(self, normed, prefix, entry, write, read_from):
        # forward.rs:2012-2065: project, per-head norm of q and k, then the rotation
        q = (self.t[f"{prefix}.q_proj.weight"] @ normed).reshape(self.heads, self.hd)
        k = (self.t[f"{prefix}.k_proj.weight"] @ normed).reshape(self.kv_heads, self.hd)
        v = (self.t[f"{prefix}.v_proj.weight"] @ normed).reshape(self.kv_heads, self.hd)
        q = self._rotate(self._norm(q, f"{prefix}.q_norm.weight"))
        k = self._rotate(self._norm(k, f"{prefix}.k_norm.weight"))
        if write:
            self.keys.setdefault(entry, []).append(k)
            self.values.setdefault(entry, []).append(v)
        source = entry if read_from is None else read_from
        all_keys = torch.stack(self.keys[source]).repeat_interleave(self.heads // self.kv_heads, dim=1)
        all_values = torch.stack(self.values[source]).repeat_interleave(self.heads // self.kv_heads, dim=1)
        # a single decoded token sees every cached key, itself included (forward.rs:1967-1989)
        weights = torch.softmax(torch.einsum("hd,thd->ht", q, all_keys) * self.scale, dim=-1)
        mixed = torch.einsum("ht,thd->hd", weights, all_values).reshape(self.heads * self.hd)
        return self.t[f"{prefix}.o_proj.weight"] @ mixed    # head-major columns (forward.rs:2070-2093)

    def feed(self, token, order=None, reads=None):
        """Logits [V] after ``token`` at the next position. ``order`` and
        ``reads`` as in ``plain_qwen3.forward_logits``."""
        x = self.t["model.embed_tokens.weight"][int(token)]
        runs = list(range(self.layers)) if order is None else list(order)
        for run, layer in enumerate(runs):
            base = f"model.layers.{layer}"
            read_from = reads[run] if reads and run in reads else None
            x = x + self._attention(self._norm(x, f"{base}.input_layernorm.weight"),
                                    f"{base}.self_attn", run, True, read_from)
            m = self._norm(x, f"{base}.post_attention_layernorm.weight")
            gate = self.t[f"{base}.mlp.gate_proj.weight"] @ m
            up = self.t[f"{base}.mlp.up_proj.weight"] @ m
            x = x + self.t[f"{base}.mlp.down_proj.weight"] @ ((torch.sigmoid(gate) * gate) * up)   # forward.rs:1904-1921
        self.position += 1
        head = "model.embed_tokens.weight" if self.c.get("tie_word_embeddings", False) else "lm_head.weight"
        return self.t[head] @ self._norm(x, "model.norm.weight")


def all_logits(config, tensors, ids, order=None, reads=None):
    """float64 [T, V]: logits after every token of one sequence."""
    decoder = CachedDecoder(config, tensors)
    return torch.stack([decoder.feed(token, order, reads) for token in ids])
