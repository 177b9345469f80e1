"""Typed configuration of the Llama 3 dense architecture, read from config.json.

Keys, defaults and validation follow tamnd/fastmlx compute/models/llama.go:23-137:
head_dim defaults to hidden_size / num_attention_heads, num_key_value_heads to
num_attention_heads, rope_theta to 10000 and tie_word_embeddings to true; unknown keys
are ignored.  Two things go beyond that file: rope_scaling is typed (and applied by the
rotary part; the Go forward parses it and never uses it, llama.go:36,61,87 against
411-412), and a `quantization` block is refused, since this engine holds dense weights
only (llama.go:111-115 parses it for the quantized linears).
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field, asdict
from typing import Any, Mapping

from .base import ConfigError, ModelConfig


@dataclass(frozen=True)
class RopeScaling:
    """The `rope_scaling` block.  Only the llama3 frequency-band rescaling is known."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_dict(d: Mapping[str, Any] | None) -> "RopeScaling | None":
        if d is None:
            return None
        if not isinstance(d, Mapping):
            raise ConfigError(f"llama: rope_scaling must be an object or null, got {d!r}")
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(f"llama: unsupported rope_scaling type {kind!r} (known: 'llama3', 'default')")
        try:
            rs = RopeScaling(
                rope_type="llama3",
                factor=float(d["factor"]),
                low_freq_factor=float(d["low_freq_factor"]),
                high_freq_factor=float(d["high_freq_factor"]),
                original_max_position_embeddings=int(d["original_max_position_embeddings"]),
            )
        except KeyError as e:
            raise ConfigError(f"llama: rope_scaling of type llama3 lacks {e.args[0]!r}") from None
        if rs.factor <= 0 or rs.original_max_position_embeddings <= 0:
            raise ConfigError("llama: rope_scaling factor and original_max_position_embeddings must be positive")
        if not rs.high_freq_factor > rs.low_freq_factor > 0:
            raise ConfigError("llama: rope_scaling needs high_freq_factor > low_freq_factor > 0")
        return rs


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    model_type: str = "llama"
    hidden_size: int = 0
    num_hidden_layers: int = 0
    intermediate_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    vocab_size: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 10000.0
    rope_traditional: bool = False
    rope_scaling: RopeScaling | None = None
    max_position_embeddings: int = 0
    attention_bias: bool = False
    mlp_bias: bool = False
    tie_word_embeddings: bool = True
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)

    # derived sizes (llama.go:139-149)
    @property
    def scale(self) -> float:
        return float(self.head_dim) ** -0.5

    @property
    def q_proj_out(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_proj_out(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def gqa_repeat(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def eos_token_id(self) -> int:
        """First of the ids, or -1 (compute/models/serve.go:49-65)."""
        return self.eos_token_ids[0] if self.eos_token_ids else -1

    @staticmethod
    def from_dict(c: Mapping[str, Any]) -> "LlamaConfig":
        def need_int(key: str, default=None) -> int:
            v = c.get(key, default)
            if v is None:
                v = 0
            if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
                raise ConfigError(f"llama: {key} must be an integer, got {v!r}")
            return int(v)

        if c.get("quantization") is not None or c.get("quantization_config") is not None:
            raise ConfigError("llama: quantized checkpoints are not supported (config has a quantization block)")
        nh = need_int("num_attention_heads")
        if nh <= 0:
            raise ConfigError(f"llama: num_attention_heads must be positive, got {nh}")
        hidden = need_int("hidden_size")
        head_dim = need_int("head_dim") if c.get("head_dim") is not None else hidden // nh
        nkv = need_int("num_key_value_heads") if c.get("num_key_value_heads") is not None else nh
        theta = c.get("rope_theta")
        theta = 10000.0 if theta is None else float(theta)
        tie = c.get("tie_word_embeddings")
        tie = True if tie is None else bool(tie)
        eos = c.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        cfg = LlamaConfig(
            model_type=str(c.get("model_type", "llama")),
            hidden_size=hidden,
            num_hidden_layers=need_int("num_hidden_layers"),
            intermediate_size=need_int("intermediate_size"),
            num_attention_heads=nh,
            num_key_value_heads=nkv,
            head_dim=head_dim,
            vocab_size=need_int("vocab_size"),
            rms_norm_eps=float(c.get("rms_norm_eps") or 0.0),
            rope_theta=theta,
            rope_traditional=bool(c.get("rope_traditional", False)),
            rope_scaling=RopeScaling.from_dict(c.get("rope_scaling")),
            max_position_embeddings=need_int("max_position_embeddings"),
            attention_bias=bool(c.get("attention_bias", False)),
            mlp_bias=bool(c.get("mlp_bias", False)),
            tie_word_embeddings=tie,
            eos_token_ids=eos_ids,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.hidden_size <= 0:
            raise ConfigError(f"llama: hidden_size must be positive, got {self.hidden_size}")
        if self.num_hidden_layers <= 0:
            raise ConfigError(f"llama: num_hidden_layers must be positive, got {self.num_hidden_layers}")
        if self.head_dim <= 0:
            raise ConfigError(f"llama: head_dim must be positive, got {self.head_dim}")
        if self.vocab_size <= 0:
            raise ConfigError(f"llama: vocab_size must be positive, got {self.vocab_size}")
        if self.num_key_value_heads <= 0 or self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"llama: num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        # Beyond the reference: what the kernels and the rotary table need.
        if self.intermediate_size <= 0:
            raise ConfigError(f"llama: intermediate_size must be positive, got {self.intermediate_size}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"llama: head_dim must be even for rotary pairs, got {self.head_dim}")
        if not (self.rms_norm_eps >= 0.0) or not math.isfinite(self.rms_norm_eps):
            raise ConfigError(f"llama: rms_norm_eps must be a finite number >= 0, got {self.rms_norm_eps}")
        if self.rope_theta <= 0:
            raise ConfigError(f"llama: rope_theta must be positive, got {self.rope_theta}")
        if self.max_position_embeddings < 0:
            raise ConfigError("llama: max_position_embeddings must not be negative")

    def to_dict(self) -> dict:
        """A config.json body that parses back to this configuration."""
        d = asdict(self)
        eos = d.pop("eos_token_ids")
        if len(eos) == 1:
            d["eos_token_id"] = eos[0]
        elif eos:
            d["eos_token_id"] = list(eos)
        d["architectures"] = ["LlamaForCausalLM"]
        return d

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), indent=2)
