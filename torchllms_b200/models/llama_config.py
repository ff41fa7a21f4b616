"""Typed configuration of the Llama-3 dense decoder, read from its ``config.json`` keys.

The key map is the one the reference's converter applies offline
(torchllms/models/checkpoint_converter.py:359-397); a torchllms ``params.json`` is accepted as
a second source with the defaults of ``ModelParams`` (torchllms/models/networks.py:110-157).  No
size and no constant the file provides is repeated anywhere else in the code: every part
receives its numbers from this object through the model spec.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional

from ..config.model_config import ConfigError, ModelConfig, require_key, typed_value


@dataclass(frozen=True)
class RopeScaling:
    """Frequency rescaling of the rotary table.

    Field names and defaults follow the keyword arguments of the reference's
    ``RotaryPositionalEmbeddings`` (torchllms/models/networks.py:225-235), which
    receives the ``rope_scaling`` dictionary of the configuration verbatim.
    """

    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 1.0
    original_max_position_embeddings: int = 8192

    KNOWN_TYPES = ("default", "llama3")

    @classmethod
    def from_dict(cls, raw: Optional[Mapping[str, Any]], where: str) -> "RopeScaling":
        if not raw:
            return cls()
        if not isinstance(raw, Mapping):
            raise ConfigError(f"{where}: key 'rope_scaling' must be an object, got {raw!r}")
        raw = dict(raw)
        # Older Hugging Face files spell the key "type"; the reference would
        # fail on it with a TypeError.  It is accepted here as the same thing.
        if "rope_type" not in raw and "type" in raw:
            raw["rope_type"] = raw.pop("type")
        rope_type = typed_value(raw.get("rope_type", "default"), "rope_scaling.rope_type", str, where)
        if rope_type not in cls.KNOWN_TYPES:
            raise ConfigError(
                f"{where}: key 'rope_scaling.rope_type' is {rope_type!r}; known types: "
                + ", ".join(cls.KNOWN_TYPES)
            )
        out = cls(
            rope_type=rope_type,
            factor=typed_value(raw.get("factor", 1.0), "rope_scaling.factor", float, where),
            low_freq_factor=typed_value(raw.get("low_freq_factor", 1.0), "rope_scaling.low_freq_factor", float, where),
            high_freq_factor=typed_value(raw.get("high_freq_factor", 1.0), "rope_scaling.high_freq_factor", float, where),
            original_max_position_embeddings=typed_value(
                raw.get("original_max_position_embeddings", 8192),
                "rope_scaling.original_max_position_embeddings", int, where),
        )
        if out.rope_type == "llama3":
            if out.factor <= 0:
                raise ConfigError(f"{where}: key 'rope_scaling.factor' must be positive")
            if out.high_freq_factor == out.low_freq_factor:
                raise ConfigError(
                    f"{where}: 'rope_scaling.high_freq_factor' and 'low_freq_factor' must differ "
                    "for rope_type 'llama3'")
            if out.original_max_position_embeddings <= 0:
                raise ConfigError(
                    f"{where}: key 'rope_scaling.original_max_position_embeddings' must be positive")
        return out

    def to_dict(self) -> Optional[Dict[str, Any]]:
        if self.rope_type == "default":
            return None
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    """Sizes and constants of a Llama-3 style dense decoder.

    Mirrors the fields of the reference's ``ModelParams`` that its base
    ``Transformer`` reads (torchllms/models/networks.py:110-124), except that the
    feed-forward width is stored as a number (``ffn_hidden``) instead of the
    ``multiple_of`` / ``ffn_dim_multiplier`` pair, so a width that is no
    multiple of 256 can be expressed.
    """

    architecture: str
    n_layers: int
    dim: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn_hidden: int
    vocab_size: int
    norm_eps: float
    rope_theta: float
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    tie_word_embeddings: bool = False
    max_seq_len: int = 4096

    # ------------------------------------------------------------------ checks
    def validate(self, where: str = "config") -> "LlamaConfig":
        for key in ("n_layers", "dim", "n_heads", "n_kv_heads", "head_dim", "ffn_hidden",
                    "vocab_size", "max_seq_len"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{where}: '{key}' must be positive, got {getattr(self, key)}")
        if self.n_heads % self.n_kv_heads != 0:
            raise ConfigError(
                f"{where}: 'n_heads' ({self.n_heads}) must be a multiple of 'n_kv_heads' "
                f"({self.n_kv_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"{where}: 'head_dim' ({self.head_dim}) must be even for rotary pairs")
        if not (self.norm_eps > 0 and math.isfinite(self.norm_eps)):
            raise ConfigError(f"{where}: 'norm_eps' must be a positive number, got {self.norm_eps}")
        if not (self.rope_theta > 0 and math.isfinite(self.rope_theta)):
            raise ConfigError(f"{where}: 'rope_theta' must be a positive number, got {self.rope_theta}")
        return self

    # ------------------------------------------------------- config.json (HF)
    @classmethod
    def from_hf(cls, raw: Mapping[str, Any], where: str = "config.json") -> "LlamaConfig":
        """Key map of torchllms/models/checkpoint_converter.py:359-397, applied at load."""
        archs = raw.get("architectures") or []
        if not isinstance(archs, (list, tuple)) or not archs:
            raise ConfigError(f"{where}: missing required key 'architectures'")
        dim = require_key(raw, "hidden_size", int, where)
        n_heads = require_key(raw, "num_attention_heads", int, where)
        n_kv = raw.get("num_key_value_heads")
        n_kv = n_heads if n_kv is None else typed_value(n_kv, "num_key_value_heads", int, where)
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if n_heads <= 0 or dim % n_heads != 0:
                raise ConfigError(
                    f"{where}: 'hidden_size' ({dim}) is no multiple of 'num_attention_heads' "
                    f"({n_heads}) and no 'head_dim' is given")
            head_dim = dim // n_heads
        else:
            head_dim = typed_value(head_dim, "head_dim", int, where)
        if raw.get("attention_bias") or raw.get("mlp_bias"):
            raise ConfigError(f"{where}: projection biases ('attention_bias'/'mlp_bias') are not "
                              "part of this architecture")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"{where}: key 'hidden_act' is {act!r}; this architecture's feed-forward is "
                              "gated by 'silu' (torchllms/models/networks.py:604-605)")
        return cls(
            architecture=str(archs[0]),
            n_layers=require_key(raw, "num_hidden_layers", int, where),
            dim=dim,
            n_heads=n_heads,
            n_kv_heads=n_kv,
            head_dim=head_dim,
            ffn_hidden=require_key(raw, "intermediate_size", int, where),
            vocab_size=require_key(raw, "vocab_size", int, where),
            norm_eps=require_key(raw, "rms_norm_eps", float, where),
            rope_theta=require_key(raw, "rope_theta", float, where),
            rope_scaling=RopeScaling.from_dict(raw.get("rope_scaling"), where),
            tie_word_embeddings=typed_value(raw.get("tie_word_embeddings", False), "tie_word_embeddings", bool, where),
            max_seq_len=typed_value(raw.get("max_position_embeddings", 4096), "max_position_embeddings", int, where),
        ).validate(where)

    def to_hf(self) -> Dict[str, Any]:
        """The ``config.json`` that :meth:`from_hf` reads back to this object."""
        out: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_size": self.dim,
            "num_hidden_layers": self.n_layers,
            "num_attention_heads": self.n_heads,
            "num_key_value_heads": self.n_kv_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.ffn_hidden,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict(),
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_seq_len,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
        }
        return out

    # ------------------------------------------------ params.json (torchllms)
    @classmethod
    def from_params_json(cls, raw: Mapping[str, Any], where: str = "params.json") -> "LlamaConfig":
        """Defaults and derivations of torchllms/models/networks.py:110-157 and :595-598."""
        for flag in ("olmo2_arch", "gpt_oss_arch", "qk_norm_per_head", "use_role_embeddings",
                     "attn_proj_bias"):
            if raw.get(flag):
                raise ConfigError(f"{where}: '{flag}' selects another architecture than the "
                                  "Llama dense decoder")
        dim = typed_value(raw.get("dim", 4096), "dim", int, where)
        n_heads = typed_value(raw.get("n_heads", 32), "n_heads", int, where)
        n_kv = raw.get("n_kv_heads")
        n_kv = n_heads if n_kv is None else typed_value(n_kv, "n_kv_heads", int, where)
        head_dim = raw.get("head_dim")
        head_dim = dim // n_heads if head_dim is None else typed_value(head_dim, "head_dim", int, where)
        multiple_of = typed_value(raw.get("multiple_of", 256), "multiple_of", int, where)
        mult = typed_value(raw.get("ffn_dim_multiplier", 8 / 3), "ffn_dim_multiplier", float, where)
        hidden = int(mult * dim)
        hidden = multiple_of * ((hidden + multiple_of - 1) // multiple_of)
        return cls(
            architecture="LlamaForCausalLM",
            n_layers=typed_value(raw.get("n_layers", 32), "n_layers", int, where),
            dim=dim,
            n_heads=n_heads,
            n_kv_heads=n_kv,
            head_dim=head_dim,
            ffn_hidden=hidden,
            vocab_size=require_key(raw, "vocab_size", int, where),
            norm_eps=typed_value(raw.get("norm_eps", 1e-5), "norm_eps", float, where),
            rope_theta=typed_value(raw.get("rope_theta", 10000.0), "rope_theta", float, where),
            rope_scaling=RopeScaling.from_dict(raw.get("rope_scaling"), where),
            tie_word_embeddings=typed_value(raw.get("tie_word_embeddings", False), "tie_word_embeddings", bool, where),
            max_seq_len=typed_value(raw.get("max_seq_len", 4096), "max_seq_len", int, where),
        ).validate(where)

    # ---------------------------------------------------------------- helpers
    def coerce_override(self, key: str, value: Any) -> Any:
        if key == "rope_scaling" and not isinstance(value, RopeScaling):
            return RopeScaling.from_dict(value, "model_kwargs")
        return value

    def parameter_count(self) -> int:
        per_layer = (self.dim * self.head_dim * (2 * self.n_heads + 2 * self.n_kv_heads)
                     + 3 * self.dim * self.ffn_hidden + 2 * self.dim)
        head = 0 if self.tie_word_embeddings else self.vocab_size * self.dim
        return self.n_layers * per_layer + self.vocab_size * self.dim + head + self.dim
