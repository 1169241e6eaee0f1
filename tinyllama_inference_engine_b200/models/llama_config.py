"""Typed configuration of the Llama dense decoder, read from its own config.json keys.

The reference reads fifteen keys with ``json.at()`` and then pins them to one
checkpoint (src/model_config.cpp:16-76).  Here the same keys are read, every size
is free, and the few options the architecture does not have (biases, rope scaling,
another activation) are refused instead of being ignored.
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from pathlib import Path

from ..config.model_config import as_float as _as_float
from ..config.model_config import as_int as _as_int
from ..config.model_config import read_config_json
from ..errors import ConfigError

_REQUIRED = (
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "max_position_embeddings",
    "vocab_size",
    "rms_norm_eps",
)


@dataclass(frozen=True)
class LlamaConfig:
    """Sizes and constants of one Llama checkpoint (include/tlie/model_config.hpp:17-43)."""

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    bos_token_id: int | None = None
    eos_token_id: int | None = None
    torch_dtype: str = "bfloat16"
    model_type: str = "llama"
    architectures: tuple[str, ...] = ("LlamaForCausalLM",)
    extra: dict = field(default_factory=dict, compare=False)

    # --- derived sizes (include/tlie/model_config.hpp:34-38) ---------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def query_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # --- reading -----------------------------------------------------------------------
    @classmethod
    def from_dict(cls, data: dict) -> "LlamaConfig":
        if not isinstance(data, dict):
            raise ConfigError("config.json must hold a JSON object")
        missing = [key for key in _REQUIRED if key not in data]
        if missing:
            raise ConfigError("config.json lacks required keys: " + ", ".join(missing))
        model_type = data.get("model_type", "llama")
        if model_type != "llama":
            raise ConfigError(f"model_type must be llama, got {model_type!r}")
        hidden = _as_int("hidden_size", data["hidden_size"])
        heads = _as_int("num_attention_heads", data["num_attention_heads"])
        kv_heads = _as_int(
            "num_key_value_heads", data.get("num_key_value_heads") or heads
        )
        if data.get("head_dim") is not None:
            head_dim = _as_int("head_dim", data["head_dim"])
        else:
            if hidden % heads != 0:
                raise ConfigError(
                    f"hidden_size {hidden} is not a multiple of num_attention_heads {heads} "
                    "and no head_dim is given"
                )
            head_dim = hidden // heads
        rope_scaling = data.get("rope_scaling")
        if rope_scaling is not None:
            raise ConfigError("rope_scaling is not part of this architecture; it must be null")
        architectures = data.get("architectures") or ["LlamaForCausalLM"]
        known = {f.name for f in fields(cls)} | {"rope_scaling"}
        config = cls(
            hidden_size=hidden,
            intermediate_size=_as_int("intermediate_size", data["intermediate_size"]),
            num_hidden_layers=_as_int("num_hidden_layers", data["num_hidden_layers"]),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=_as_int(
                "max_position_embeddings", data["max_position_embeddings"]
            ),
            vocab_size=_as_int("vocab_size", data["vocab_size"]),
            rms_norm_eps=_as_float("rms_norm_eps", data["rms_norm_eps"]),
            rope_theta=_as_float("rope_theta", data.get("rope_theta", 10000.0)),
            tie_word_embeddings=bool(data.get("tie_word_embeddings", False)),
            hidden_act=str(data.get("hidden_act", "silu")),
            attention_bias=bool(data.get("attention_bias", False)),
            mlp_bias=bool(data.get("mlp_bias", False)),
            bos_token_id=data.get("bos_token_id"),
            eos_token_id=data.get("eos_token_id"),
            torch_dtype=str(data.get("torch_dtype") or data.get("dtype") or "bfloat16"),
            model_type=model_type,
            architectures=tuple(architectures),
            extra={k: v for k, v in data.items() if k not in known},
        )
        config.validate()
        return config

    @classmethod
    def from_json_file(cls, path: str | Path) -> "LlamaConfig":
        return cls.from_dict(read_config_json(path))

    def validate(self) -> None:
        """Consistency only; no size is pinned (contrast src/model_config.cpp:54-76)."""
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}"
            )
        if self.head_dim % 16 != 0 or self.head_dim > 256:
            # what the attention kernels take (a multiple of 16 up to 256); refused here, not at the first step
            raise ConfigError(f"head_dim must be a multiple of 16 up to 256, got {self.head_dim}")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act must be silu, got {self.hidden_act!r}")
        if self.attention_bias or self.mlp_bias:
            raise ConfigError("attention_bias and mlp_bias must be false: the architecture has no biases")
        for name in ("bos_token_id", "eos_token_id"):
            value = getattr(self, name)
            if value is not None and (isinstance(value, bool) or not isinstance(value, int)):
                raise ConfigError(f"{name} must be an integer or null, got {value!r}")

    def to_dict(self) -> dict:
        data = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": self.eos_token_id,
            "torch_dtype": self.torch_dtype,
        }
        data.update(self.extra)
        return data
