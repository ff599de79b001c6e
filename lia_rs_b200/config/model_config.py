"""Typed configuration of the Llama-family decoder, read from config.json's own keys.

The reference reads these keys as equality checks against one geometry
(src/models/minicpm5.rs:7-35); here each is a parameter.  MiniCPM's `scale_emb`,
`scale_depth` and `dim_model_base` are optional: when absent the model is the reference's
plain Llama.  No size or constant that config.json gives appears anywhere else in the code.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field, asdict
from typing import Optional


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value this engine refuses."""


def _need(raw: dict, key: str, kind):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: missing key {key!r}")
    value = raw[key]
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
            raise ConfigError(f"config.json: {key} must be a positive integer, got {value!r}")
        return value
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {key} must be a number, got {value!r}")
    value = float(value)
    if not math.isfinite(value) or value <= 0:
        raise ConfigError(f"config.json: {key} must be finite and positive, got {value!r}")
    return value


def _optional_number(raw: dict, key: str) -> Optional[float]:
    if raw.get(key) is None:
        return None
    return _need(raw, key, float)


LAYER_TYPES = ("full_attention", "sliding_attention")


@dataclass(frozen=True)
class LlamaConfig:
    """Every number the MiniCPM5 Llama decoder needs.

    Keys follow config.json: hidden_size, intermediate_size, num_hidden_layers,
    num_attention_heads, num_key_value_heads, head_dim, vocab_size,
    max_position_embeddings, rms_norm_eps, rope_theta, tie_word_embeddings, scale_emb,
    scale_depth, dim_model_base, sliding_window, layer_types, initializer_range.
    """

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    scale_emb: Optional[float] = None
    scale_depth: Optional[float] = None
    dim_model_base: Optional[float] = None
    sliding_window: Optional[int] = None
    layer_types: tuple = ()
    initializer_range: float = 0.02
    model_type: str = "llama"
    architectures: tuple = ("LlamaForCausalLM",)
    torch_dtype: str = "bfloat16"
    eos_token_id: tuple = ()
    extra: dict = field(default_factory=dict, compare=False)

    # ---- derived quantities (formulas, not constants) ----
    @property
    def embedding_scale(self) -> float:
        return 1.0 if self.scale_emb is None else float(self.scale_emb)

    @property
    def residual_scale(self) -> float:
        """scale_depth / sqrt(num_hidden_layers) on each residual branch; 1 when absent."""
        if self.scale_depth is None:
            return 1.0
        return float(self.scale_depth) / math.sqrt(self.num_hidden_layers)

    @property
    def logit_scale(self) -> float:
        """Logits are divided by hidden_size / dim_model_base; 1 when absent."""
        if self.dim_model_base is None:
            return 1.0
        return float(self.dim_model_base) / float(self.hidden_size)

    def window_of_layer(self, layer: int) -> Optional[int]:
        if self.layer_types and self.layer_types[layer] == "sliding_attention":
            return self.sliding_window
        return None

    # ---- construction ----
    @classmethod
    def from_dict(cls, raw: dict) -> "LlamaConfig":
        hidden = _need(raw, "hidden_size", int)
        heads = _need(raw, "num_attention_heads", int)
        kv_heads = raw.get("num_key_value_heads")
        kv_heads = heads if kv_heads is None else _need(raw, "num_key_value_heads", int)
        if raw.get("head_dim") is None:
            if hidden % heads:
                raise ConfigError("config.json: head_dim absent and hidden_size is not a multiple of num_attention_heads")
            head_dim = hidden // heads
        else:
            head_dim = _need(raw, "head_dim", int)
        layers = _need(raw, "num_hidden_layers", int)
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (only 'silu')")
        for key in ("attention_bias", "mlp_bias"):
            if raw.get(key):
                raise ConfigError(f"config.json: {key}=true is not supported")
        if raw.get("rope_scaling") is not None:
            raise ConfigError("config.json: rope_scaling must be null")
        if raw.get("quantization_config") is not None:
            raise ConfigError("config.json: quantized checkpoints are not supported")
        window = raw.get("sliding_window")
        if window is not None:
            window = _need(raw, "sliding_window", int)
        layer_types = raw.get("layer_types") or ()
        if layer_types:
            if len(layer_types) != layers:
                raise ConfigError("config.json: layer_types must have num_hidden_layers entries")
            for kind in layer_types:
                if kind not in LAYER_TYPES:
                    raise ConfigError(f"config.json: unknown layer type {kind!r}; known: {LAYER_TYPES}")
            if "sliding_attention" in layer_types and window is None:
                raise ConfigError("config.json: layer_types names sliding_attention but sliding_window is null")
        eos = raw.get("eos_token_id")
        if eos is None:
            eos = ()
        elif isinstance(eos, int):
            eos = (eos,)
        known = {f for f in cls.__dataclass_fields__} | {
            "hidden_act", "attention_bias", "mlp_bias", "rope_scaling", "quantization_config", "dtype"}
        cfg = cls(
            hidden_size=hidden,
            intermediate_size=_need(raw, "intermediate_size", int),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=_need(raw, "vocab_size", int),
            max_position_embeddings=_need(raw, "max_position_embeddings", int),
            rms_norm_eps=_need(raw, "rms_norm_eps", float),
            rope_theta=_need(raw, "rope_theta", float) if raw.get("rope_theta") is not None else 10000.0,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            scale_emb=_optional_number(raw, "scale_emb"),
            scale_depth=_optional_number(raw, "scale_depth"),
            dim_model_base=_optional_number(raw, "dim_model_base"),
            sliding_window=window,
            layer_types=tuple(layer_types),
            initializer_range=float(raw.get("initializer_range", 0.02)),
            model_type=str(raw.get("model_type", "llama")),
            architectures=tuple(raw.get("architectures") or ("LlamaForCausalLM",)),
            torch_dtype=str(raw.get("torch_dtype") or raw.get("dtype") or "bfloat16"),
            eos_token_id=tuple(int(t) for t in eos),
            extra={k: v for k, v in raw.items() if k not in known},
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_dim % 2:
            raise ConfigError("head_dim must be even (rotate-half rotary encoding)")
        for name in ("scale_emb", "scale_depth", "dim_model_base"):
            v = getattr(self, name)
            if v is not None and (not math.isfinite(v) or v <= 0):
                raise ConfigError(f"{name} must be finite and positive")

    def validate_capacity(self, capacity: int) -> None:
        """0 < capacity <= max_position_embeddings (src/models/mod.rs:96-102)."""
        if not (0 < capacity <= self.max_position_embeddings):
            raise ConfigError(
                f"context capacity {capacity} exceeds the model's max_position_embeddings "
                f"{self.max_position_embeddings}")

    def to_dict(self) -> dict:
        d = asdict(self)
        extra = d.pop("extra")
        d["architectures"] = list(self.architectures)
        d["layer_types"] = list(self.layer_types) or None
        d["eos_token_id"] = list(self.eos_token_id) or None
        d["hidden_act"] = "silu"
        d["rope_scaling"] = None
        d = {k: v for k, v in d.items() if v is not None or k in ("rope_scaling",)}
        d.update(extra)
        return d


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except OSError as error:
        raise ConfigError(f"opening {path}: {error}") from error
    except json.JSONDecodeError as error:
        raise ConfigError(f"reading {path}: {error}") from error
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: not a JSON object")
    return raw
