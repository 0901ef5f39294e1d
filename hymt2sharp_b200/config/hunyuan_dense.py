"""Configuration of the Hunyuan dense architecture ("HunYuanDenseV1ForCausalLM").

The fields are the hyper-parameters that sdcb/HyMT2Sharp reads from GGUF
metadata (src/HyMT2Sharp/ModelConfig.cs:21-51), here under config.json's key
names, with the same defaults.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict

import numpy as np

from .base import ConfigError, ConfigReader

ARCHITECTURE = "HunYuanDenseV1ForCausalLM"


@dataclass(frozen=True)
class HunyuanDenseConfig:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rope_alpha: float
    rope_dim: int
    rms_norm_eps: float
    use_qk_norm: bool
    tie_word_embeddings: bool
    sliding_window: int | None = None

    architecture = ARCHITECTURE

    # -- derived sizes ------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def rope_base(self) -> float:
        """Dynamic-NTK base, computed once in float32:
        theta * alpha^(d/(d-2)) when alpha > 0 and d > 2, else theta
        (src/HyMT2Sharp/ModelConfig.cs:31-34; the exponent uses head_dim)."""
        base = np.float32(self.rope_theta)
        if self.rope_alpha > 0 and self.head_dim > 2:
            expo = np.float32(self.head_dim) / np.float32(self.head_dim - 2)
            base = np.float32(base * np.float32(math.pow(float(np.float32(self.rope_alpha)), float(expo))))
        return float(base)

    # -- construction -------------------------------------------------------
    @classmethod
    def from_dict(cls, data: dict, source: str = "config.json") -> "HunyuanDenseConfig":
        r = ConfigReader(data, source)
        heads = r.integer("num_attention_heads", minimum=1)
        hidden = r.integer("hidden_size", minimum=1)
        head_dim = r.integer("head_dim", "attention_head_dim", default=None, minimum=1)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"{source}: 'head_dim' is absent and hidden_size {hidden} "
                                  f"is not a multiple of num_attention_heads {heads}")
            head_dim = hidden // heads
        scaling_type = r.string("rope_scaling.type", "rope_scaling.rope_type", default=None)
        alpha = r.number("rope_scaling.alpha", default=0.0, minimum=0.0)
        if scaling_type not in (None, "dynamic"):
            raise ConfigError(f"{source}: rope_scaling.type '{scaling_type}' is not supported (only 'dynamic' with 'alpha')")
        cfg = cls(
            num_hidden_layers=r.integer("num_hidden_layers", minimum=1),
            hidden_size=hidden,
            num_attention_heads=heads,
            num_key_value_heads=r.integer("num_key_value_heads", default=heads, minimum=1),
            head_dim=head_dim,
            intermediate_size=r.integer("intermediate_size", minimum=1),
            vocab_size=r.integer("vocab_size", minimum=1),
            max_position_embeddings=r.integer("max_position_embeddings", default=4096, minimum=1),
            rope_theta=r.number("rope_theta", default=10000.0, exclusive_minimum=0.0),
            rope_alpha=alpha,
            rope_dim=r.integer("rope_dim", default=head_dim, minimum=0),
            rms_norm_eps=r.number("rms_norm_eps", default=1e-5, exclusive_minimum=0.0),
            use_qk_norm=r.boolean("use_qk_norm", default=True),
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=True),
            sliding_window=r.integer("sliding_window", default=None, minimum=1),
        )
        cfg.validate(source)
        return cfg

    def validate(self, source: str = "config") -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"{source}: num_attention_heads {self.num_attention_heads} is not a multiple "
                              f"of num_key_value_heads {self.num_key_value_heads}")
        if self.rope_dim % 2 or self.rope_dim > self.head_dim:
            raise ConfigError(f"{source}: rope_dim {self.rope_dim} must be even and at most head_dim {self.head_dim}")

    def to_dict(self) -> dict:
        """config.json form of this configuration."""
        d = {
            "architectures": [ARCHITECTURE],
            "model_type": "hunyuan_v1_dense",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rope_scaling": {"type": "dynamic", "alpha": self.rope_alpha} if self.rope_alpha > 0 else None,
            "rms_norm_eps": self.rms_norm_eps,
            "use_qk_norm": self.use_qk_norm,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": "bfloat16",
        }
        if self.rope_dim != self.head_dim:
            d["rope_dim"] = self.rope_dim
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        return d

    def describe(self) -> dict:
        return asdict(self)
