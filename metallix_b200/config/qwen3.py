"""Typed configuration of the Qwen3 dense decoder, read from ``config.json``.

Follows the validation list of the reference's
``Qwen3ForwardConfig::parse`` (``crates/models/qwen/src/forward.rs:461-557``,
raw keys and defaults ``:2576-2661``, dimension checks ``:400-432``): every
size comes from the file, variants the decoder does not implement are refused
by name instead of being ignored.
"""
from __future__ import annotations

import json
import math
import struct
from dataclasses import dataclass
from typing import Any, Dict, Mapping

from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec


class ConfigError(ValueError):
    """A ``config.json`` this engine refuses. ``kind`` names the reason
    (the error kinds of ``forward.rs:2738-2830``)."""

    def __init__(self, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.kind = kind


def _as_count(raw: Mapping[str, Any], key: str) -> int:
    """A size key: absent counts as zero (serde default, ``forward.rs:2585-2600``)
    and zero is refused later by name."""
    value = raw.get(key, 0)
    if value is None:
        return 0
    if isinstance(value, bool) or not isinstance(value, int) or value < 0:
        raise ConfigError("Json", f"{key} must be a non-negative integer, got {value!r}")
    return value


def _as_bool(raw: Mapping[str, Any], key: str) -> bool:
    value = raw.get(key, False)
    if value is None:
        return False
    if not isinstance(value, bool):
        raise ConfigError("Json", f"{key} must be a boolean, got {value!r}")
    return value


def _as_f32(value: Any, key: str) -> float:
    """The reference holds eps and theta as f32 (``forward.rs:388-389``); the
    value used everywhere is the number rounded to 32 bits."""
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError("Json", f"{key} must be a number, got {value!r}")
    try:
        return struct.unpack("<f", struct.pack("<f", float(value)))[0]
    except OverflowError:
        return math.inf


@dataclass(frozen=True)
class Qwen3Config:
    """Sizes and constants of one Qwen3 dense checkpoint."""

    num_hidden_layers: int
    hidden_size: int
    intermediate_size: int
    vocab_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    eos_token_ids: tuple = ()

    ARCHITECTURE = "Qwen3ForCausalLM"
    MODEL_TYPE = "qwen3"

    # ------------------------------------------------------------------ parse
    @classmethod
    def parse(cls, text: str) -> "Qwen3Config":
        try:
            raw = json.loads(text)
        except json.JSONDecodeError as error:
            raise ConfigError("Json", str(error)) from None
        if not isinstance(raw, dict):
            raise ConfigError("Json", "config.json must hold one JSON object")
        return cls.from_dict(raw)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        model_type = raw.get("model_type", "")
        # forward.rs:463-468 with lib.rs:91-98,134-139: this engine builds the
        # causal qwen3 family only.
        if model_type != cls.MODEL_TYPE or _as_bool(raw, "use_bidirectional_attention"):
            raise ConfigError("UnsupportedModelType", f"model_type {model_type!r}")
        if _as_bool(raw, "attention_bias") or _as_bool(raw, "mlp_bias"):
            raise ConfigError("UnsupportedBiasLayout", "attention_bias / mlp_bias must be false")
        hidden_act = raw.get("hidden_act", "")
        if hidden_act != "silu":  # forward.rs:472-474: absent is refused too
            raise ConfigError("UnsupportedActivation", f"hidden_act {hidden_act!r}, only 'silu'")
        if raw.get("rope_scaling") is not None:  # forward.rs:475-477
            raise ConfigError("UnsupportedRopeScaling", "rope_scaling must be absent or null")

        rope_theta = raw.get("rope_theta")
        if rope_theta is not None:
            rope_theta = _as_f32(rope_theta, "rope_theta")
        parameters = raw.get("rope_parameters")
        if parameters is not None:  # forward.rs:482-498
            if not isinstance(parameters, dict):
                raise ConfigError("Json", "rope_parameters must be an object")
            other = {k: v for k, v in parameters.items() if k not in ("rope_type", "rope_theta")}
            if parameters.get("rope_type", "") != "default" or other:
                raise ConfigError("UnsupportedRopeScaling",
                                  "rope_parameters: only rope_type 'default' with rope_theta")
            nested = parameters.get("rope_theta")
            if nested is not None:
                nested = _as_f32(nested, "rope_parameters.rope_theta")
            if rope_theta is not None and nested is not None and \
                    struct.pack("<f", rope_theta) != struct.pack("<f", nested):
                raise ConfigError("ConflictingRopeTheta",
                                  f"rope_theta {rope_theta} but rope_parameters.rope_theta {nested}")
            if rope_theta is None:
                rope_theta = nested
        if rope_theta is None:
            rope_theta = 1_000_000.0  # forward.rs:502-508,2659-2661

        if _as_bool(raw, "use_sliding_window"):  # forward.rs:518-528
            raise ConfigError("UnsupportedSlidingWindow", "use_sliding_window must be false")
        for key in ("quantization", "quantization_config"):
            if raw.get(key) is not None:
                raise ConfigError("UnsupportedQuantization", f"{key} is set; only plain weights")

        sizes = {key: _as_count(raw, key) for key in (
            "num_hidden_layers", "hidden_size", "intermediate_size", "vocab_size",
            "num_attention_heads", "num_key_value_heads", "head_dim",
            "max_position_embeddings")}
        for key, value in sizes.items():  # forward.rs:400-415
            if value == 0:
                raise ConfigError("MissingDimension", key)
        if sizes["head_dim"] % 2:
            raise ConfigError("OddHeadDimension", str(sizes["head_dim"]))
        if sizes["head_dim"] > 0xFFFF:
            raise ConfigError("HeadDimensionTooLarge", str(sizes["head_dim"]))
        if sizes["num_attention_heads"] % sizes["num_key_value_heads"]:
            raise ConfigError(
                "InvalidGroupedQueryLayout",
                f"{sizes['num_attention_heads']} query heads over "
                f"{sizes['num_key_value_heads']} key/value heads")

        eps = _as_f32(raw.get("rms_norm_eps", 1e-6), "rms_norm_eps")
        if not math.isfinite(eps) or eps <= 0.0:
            raise ConfigError("InvalidRmsNormEpsilon", str(eps))
        if not math.isfinite(rope_theta) or rope_theta <= 0.0:
            raise ConfigError("InvalidRopeTheta", str(rope_theta))

        # Stop ids: eos_token_id of config.json, a number or a list
        # (crates/core/chat-format/src/lib.rs:207-253 unions it with
        # generation_config.json; the loader adds that file's ids).
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError("Json", f"eos_token_id must be an integer or a list, got {eos!r}")

        return cls(rms_norm_eps=eps, rope_theta=rope_theta,
                   tie_word_embeddings=_as_bool(raw, "tie_word_embeddings"),
                   eos_token_ids=eos_ids, **sizes)

    # ------------------------------------------------------------ derived facts
    def kv_bytes_per_token(self, bytes_per_value: int) -> int:
        """``L * 2 * KV * hd * bytes`` (``forward.rs:622-638``)."""
        return (self.num_hidden_layers * 2 * self.num_key_value_heads
                * self.head_dim * bytes_per_value)

    def parameter_count(self) -> int:
        h, i = self.hidden_size, self.intermediate_size
        q = self.num_attention_heads * self.head_dim
        kv = self.num_key_value_heads * self.head_dim
        per_layer = 2 * h + q * h + 2 * kv * h + h * q + 2 * self.head_dim + 3 * i * h
        head = 0 if self.tie_word_embeddings else self.vocab_size * h
        return self.vocab_size * h + self.num_hidden_layers * per_layer + h + head

    def to_dict(self) -> Dict[str, Any]:
        """The ``config.json`` this configuration is read back from."""
        out: Dict[str, Any] = {
            "architectures": [self.ARCHITECTURE],
            "model_type": self.MODEL_TYPE,
            "hidden_act": "silu",
            "attention_bias": False,
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    # ------------------------------------------------------------- model spec
    def to_model_spec(self) -> ModelSpec:
        """The decoder of ``forward.rs:1856-1922`` as data: every layer is
        pre-norm GQA attention with per-head q/k RMSNorm and rotate-half RoPE,
        then pre-norm SwiGLU, each followed by a residual sum."""
        h = self.hidden_size
        rope = PartSpec("rope_half", {  # forward.rs:2031-2054: dims = head_dim, scale 1
            "theta": self.rope_theta, "rotary_dim": self.head_dim, "head_dim": self.head_dim})
        layers = []
        for index in range(self.num_hidden_layers):
            base = f"model.layers.{index}"
            head_norm = lambda name: PartSpec("rmsnorm", {  # forward.rs:2425-2440
                "size": self.head_dim, "eps": self.rms_norm_eps,
                "weight": f"{base}.self_attn.{name}.weight"})
            mixer = PartSpec("gqa_attention", {
                "hidden_size": h,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "scale": float(self.head_dim) ** -0.5,  # forward.rs:2290-2295
                "window": None,
                "q_proj": f"{base}.self_attn.q_proj.weight",
                "k_proj": f"{base}.self_attn.k_proj.weight",
                "v_proj": f"{base}.self_attn.v_proj.weight",
                "o_proj": f"{base}.self_attn.o_proj.weight",
                "q_norm": head_norm("q_norm"),
                "k_norm": head_norm("k_norm"),
                "position": rope,
            })
            feed_forward = PartSpec("swiglu", {  # forward.rs:1889-1922
                "hidden_size": h, "intermediate_size": self.intermediate_size,
                "gate_proj": f"{base}.mlp.gate_proj.weight",
                "up_proj": f"{base}.mlp.up_proj.weight",
                "down_proj": f"{base}.mlp.down_proj.weight"})
            layers.append(LayerSpec(
                name=base,
                block=PartSpec("prenorm_residual", {}),
                mixer=mixer,
                feed_forward=feed_forward,
                mixer_norm=PartSpec("rmsnorm", {
                    "size": h, "eps": self.rms_norm_eps,
                    "weight": f"{base}.input_layernorm.weight"}),
                feed_forward_norm=PartSpec("rmsnorm", {
                    "size": h, "eps": self.rms_norm_eps,
                    "weight": f"{base}.post_attention_layernorm.weight"})))
        head_tensor = ("model.embed_tokens.weight" if self.tie_word_embeddings
                       else "lm_head.weight")  # forward.rs:574-580
        spec = ModelSpec(
            architecture=self.ARCHITECTURE,
            hidden_size=h,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {
                "vocab_size": self.vocab_size, "hidden_size": h,
                "weight": "model.embed_tokens.weight"}),
            layers=tuple(layers),
            order=tuple(LayerRun(layer=i) for i in range(self.num_hidden_layers)),
            final_norm=PartSpec("rmsnorm", {
                "size": h, "eps": self.rms_norm_eps, "weight": "model.norm.weight"}),
            head=PartSpec("linear_head", {
                "vocab_size": self.vocab_size, "hidden_size": h, "weight": head_tensor}),
        )
        spec.validate()
        return spec

    # --------------------------------------------------------- tensor contract
    def tensor_shapes(self) -> Dict[str, tuple]:
        """Every tensor the checkpoint must hold, by canonical name
        (``crates/models/qwen/src/checkpoint.rs:772-875``)."""
        h, hd, i = self.hidden_size, self.head_dim, self.intermediate_size
        q, kv = self.num_attention_heads * hd, self.num_key_value_heads * hd
        shapes: Dict[str, tuple] = {"model.embed_tokens.weight": (self.vocab_size, h)}
        for index in range(self.num_hidden_layers):
            base = f"model.layers.{index}"
            shapes.update({
                f"{base}.input_layernorm.weight": (h,),
                f"{base}.self_attn.q_proj.weight": (q, h),
                f"{base}.self_attn.k_proj.weight": (kv, h),
                f"{base}.self_attn.v_proj.weight": (kv, h),
                f"{base}.self_attn.o_proj.weight": (h, q),
                f"{base}.self_attn.q_norm.weight": (hd,),
                f"{base}.self_attn.k_norm.weight": (hd,),
                f"{base}.post_attention_layernorm.weight": (h,),
                f"{base}.mlp.gate_proj.weight": (i, h),
                f"{base}.mlp.up_proj.weight": (i, h),
                f"{base}.mlp.down_proj.weight": (h, i),
            })
        shapes["model.norm.weight"] = (h,)
        if not self.tie_word_embeddings:
            shapes["lm_head.weight"] = (self.vocab_size, h)
        return shapes

    def ignored_tensors(self) -> tuple:
        """Names a checkpoint may hold that are dropped, not loaded: a tied
        checkpoint's stray ``lm_head.weight`` (``metal.rs:778-784``)."""
        return ("lm_head.weight",) if self.tie_word_embeddings else ()

    def norm_tensor(self, name: str) -> bool:
        return name.endswith("norm.weight") or name.endswith("layernorm.weight")
