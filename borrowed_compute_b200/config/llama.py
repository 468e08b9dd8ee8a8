"""Typed configuration of the Llama dense decoder, read from config.json's own keys.

The reference reads the same quantities from GGUF metadata
(crates/bc-infer/src/model.rs:26-80) and applies the same defaults: kv heads default to
the head count (model.rs:60), the head size to hidden / heads (51), the rope base to 10000
(63), eps to 1e-5 (65), the context to 4096 (67).  Here the keys are config.json's.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError


def _get(d: Mapping[str, Any], key: str, kind, default=None, required: bool = False):
    if key not in d or d[key] is None:
        if required:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
        return float(v)
    if kind is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: '{key}' must be true or false, got {v!r}")
        return v
    if kind is str:
        if not isinstance(v, str):
            raise ConfigError(f"config.json: '{key}' must be a string, got {v!r}")
        return v
    raise AssertionError(kind)


@dataclass(frozen=True)
class Llama3RopeScaling:
    """The four numbers of config.json's ``rope_scaling`` object for the llama3 rule (low
    frequencies are slowed by ``factor``).  The rule itself belongs to the rotary part,
    which takes these numbers as plain parameters.
    """

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "Llama3RopeScaling":
        if not isinstance(d, Mapping):
            raise ConfigError(f"config.json: 'rope_scaling' must be an object, got {d!r}")
        kind = d.get("rope_type", d.get("type"))
        if kind != "llama3":
            raise ConfigError(f"config.json: rope_scaling.rope_type {kind!r} is not supported (only 'llama3')")
        s = Llama3RopeScaling(
            factor=_get(d, "factor", float, required=True),
            low_freq_factor=_get(d, "low_freq_factor", float, required=True),
            high_freq_factor=_get(d, "high_freq_factor", float, required=True),
            original_max_position_embeddings=_get(d, "original_max_position_embeddings", int, required=True),
        )
        if s.factor <= 0 or s.high_freq_factor <= s.low_freq_factor or s.original_max_position_embeddings <= 0:
            raise ConfigError(f"config.json: rope_scaling values are inconsistent: {dict(d)!r}")
        return s

    def to_dict(self) -> dict:
        return {
            "rope_type": "llama3",
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


@dataclass(frozen=True)
class LlamaConfig:
    """Every size and constant of one Llama model.  Nothing here has a default in code
    that config.json could give; the defaults below are the ones the format defines."""

    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float = 10000.0
    rope_scaling: Optional[Llama3RopeScaling] = None
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 4096
    # Which two dimensions of a head rotate together: "half" pairs i with i + d/2 (the
    # order of q_proj / k_proj rows in published safetensors checkpoints), "adjacent" pairs
    # 2i with 2i + 1 (the order of GGUF Llama files; model.rs:36-37,64).  Not a key of
    # published config.json files; absent means "half".
    rope_pairing: str = "half"
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "LlamaForCausalLM"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "LlamaConfig":
        heads = _get(d, "num_attention_heads", int, required=True)
        hidden = _get(d, "hidden_size", int, required=True)
        if heads <= 0 or hidden <= 0:
            raise ConfigError("config.json: 'num_attention_heads' and 'hidden_size' must be positive")
        kv_heads = _get(d, "num_key_value_heads", int, default=heads)
        head_dim = _get(d, "head_dim", int, default=None)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads {heads} and no 'head_dim' is given")
            head_dim = hidden // heads
        scaling = d.get("rope_scaling")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"config.json: 'eos_token_id' must be an integer or a list of integers, got {eos!r}")
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        cfg = LlamaConfig(
            num_hidden_layers=_get(d, "num_hidden_layers", int, required=True),
            hidden_size=hidden,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=_get(d, "intermediate_size", int, required=True),
            vocab_size=_get(d, "vocab_size", int, required=True),
            rope_theta=_get(d, "rope_theta", float, default=10000.0),
            rope_scaling=None if scaling is None else Llama3RopeScaling.from_dict(scaling),
            rms_norm_eps=_get(d, "rms_norm_eps", float, default=1e-5),
            tie_word_embeddings=_get(d, "tie_word_embeddings", bool, default=False),
            max_position_embeddings=_get(d, "max_position_embeddings", int, default=4096),
            rope_pairing=_get(d, "rope_pairing", str, default="half"),
            eos_token_ids=eos_ids,
            architecture=str(archs[0]),
            extra={k: v for k, v in d.items()},
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for key in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                    "intermediate_size", "vocab_size", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"config.json: '{key}' must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} is odd; rotary pairs need an even size")
        if self.rope_pairing not in ("half", "adjacent"):
            raise ConfigError(f"config.json: rope_pairing {self.rope_pairing!r} is neither 'half' nor 'adjacent'")
        if not (self.rms_norm_eps > 0.0) or not (self.rope_theta > 0.0):
            raise ConfigError("config.json: 'rms_norm_eps' and 'rope_theta' must be positive")
        for e in self.eos_token_ids:
            if not 0 <= e < self.vocab_size:
                raise ConfigError(f"config.json: eos_token_id {e} is outside the vocabulary of {self.vocab_size}")

    # Derived sizes (model.rs:72-79 has the same two for its f32 cache).
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def kv_bytes_per_token_layer(self, itemsize: int) -> int:
        return 2 * self.kv_dim * itemsize

    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rope_theta": self.rope_theta,
            "rope_scaling": None if self.rope_scaling is None else self.rope_scaling.to_dict(),
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
        }
        if self.rope_pairing != "half":
            d["rope_pairing"] = self.rope_pairing
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d
