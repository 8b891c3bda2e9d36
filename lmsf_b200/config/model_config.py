"""Typed model configurations read from config.json.

`LlamaConfig` plays the role of the reference's serde struct
(core/src/model_executor/models/llama/config.rs:7-54) with the differences that every
optional key has a default, `rope_theta`, `rope_scaling`, `head_dim` and
`tie_word_embeddings` are honoured, `eos_token_id` may be a list and `bfloat16` is a
valid `torch_dtype`.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model."""


@dataclass(frozen=True)
class RopeScaling:
    """Frequency rescaling of rotary embeddings.  `rope_type` is one of
    "default" (none), "linear" (all frequencies / factor) or "llama3"
    (wavelength-dependent interpolation between f and f / factor)."""
    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    KNOWN = ("default", "linear", "llama3")

    @staticmethod
    def from_dict(d: Optional[Dict[str, Any]]) -> "RopeScaling":
        if not d:
            return RopeScaling()
        kind = d.get("rope_type", d.get("type", "default"))
        if kind not in RopeScaling.KNOWN:
            raise ConfigError(f"rope_scaling type {kind!r} is not supported (known: {', '.join(RopeScaling.KNOWN)})")
        if kind == "default":
            return RopeScaling()
        if "factor" not in d:
            raise ConfigError(f"rope_scaling of type {kind!r} needs a 'factor'")
        if kind == "linear":
            return RopeScaling(rope_type=kind, factor=float(d["factor"]))
        missing = [k for k in ("low_freq_factor", "high_freq_factor", "original_max_position_embeddings") if k not in d]
        if missing:
            raise ConfigError(f"rope_scaling of type 'llama3' lacks {missing}")
        rs = RopeScaling(kind, float(d["factor"]), float(d["low_freq_factor"]), float(d["high_freq_factor"]),
                         int(d["original_max_position_embeddings"]))
        if rs.high_freq_factor <= rs.low_freq_factor:
            raise ConfigError("rope_scaling: high_freq_factor must exceed low_freq_factor")
        return rs


@dataclass
class LlamaConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    intermediate_size: int = 11008
    vocab_size: int = 32000
    num_key_value_heads: Optional[int] = None      # default: num_attention_heads (MHA)
    head_dim: Optional[int] = None                 # default: hidden_size / num_attention_heads
    hidden_act: str = "silu"
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    tie_word_embeddings: bool = False
    sliding_window: Optional[int] = None
    attention_bias: bool = False
    mlp_bias: bool = False
    bos_token_id: Optional[int] = 1
    eos_token_ids: List[int] = field(default_factory=lambda: [2])
    torch_dtype: str = "bfloat16"
    model_type: str = "llama"
    architectures: List[str] = field(default_factory=lambda: ["LlamaForCausalLM"])

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        for name in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                     "intermediate_size", "vocab_size", "max_position_embeddings"):
            v = getattr(self, name)
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"{name} must be a positive integer, got {v!r}")
        if self.head_dim is None:
            if self.hidden_size % self.num_attention_heads:
                raise ConfigError(f"hidden_size {self.hidden_size} is not a multiple of num_attention_heads "
                                  f"{self.num_attention_heads} and no head_dim is given")
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.head_dim <= 0 or self.head_dim % 2:
            raise ConfigError(f"head_dim must be a positive even number, got {self.head_dim}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.hidden_act not in ("silu", "swish", "gelu_tanh", "gelu_pytorch_tanh"):
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported by the gated feed-forward "
                              f"(silu, gelu_pytorch_tanh)")
        self.attention_bias, self.mlp_bias = bool(self.attention_bias), bool(self.mlp_bias)
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if self.sliding_window is not None and self.sliding_window <= 0:
            raise ConfigError(f"sliding_window must be positive or null, got {self.sliding_window}")
        if self.torch_dtype not in ("bfloat16", "float32", "float16", "half", "float"):
            raise ConfigError(f"invalid torch_dtype {self.torch_dtype!r}")

    # generic getters (the role of the reference's `trait ModelConfig`,
    # core/src/model_executor/models/model.rs:8-37)
    @property
    def max_model_len(self) -> int:
        return self.max_position_embeddings

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "LlamaConfig":
        for k in ("hidden_size", "num_hidden_layers", "num_attention_heads"):
            if k not in d:
                raise ConfigError(f"config.json lacks the mandatory key {k!r}")
        kw: Dict[str, Any] = {}
        for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size", "vocab_size",
                  "num_key_value_heads", "head_dim", "hidden_act", "max_position_embeddings", "rms_norm_eps",
                  "rope_theta", "tie_word_embeddings", "sliding_window", "attention_bias", "mlp_bias",
                  "bos_token_id", "model_type", "architectures"):
            if k in d and d[k] is not None:
                kw[k] = d[k]
        scaling = d.get("rope_scaling")
        params = d.get("rope_parameters")          # newer spelling: theta and scaling in one object
        if params:
            if "rope_theta" in params and "rope_theta" not in kw:
                kw["rope_theta"] = params["rope_theta"]
            if scaling is None and params.get("rope_type", "default") != "default":
                scaling = params
        kw["rope_scaling"] = RopeScaling.from_dict(scaling)
        if "rope_theta" in kw:
            kw["rope_theta"] = float(kw["rope_theta"])
        if "rms_norm_eps" in kw:
            kw["rms_norm_eps"] = float(kw["rms_norm_eps"])
        eos = d.get("eos_token_id")
        if eos is not None:
            kw["eos_token_ids"] = [int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos])]
        dt = d.get("torch_dtype", d.get("dtype"))
        if dt is not None:
            kw["torch_dtype"] = str(dt).replace("torch.", "")
        return LlamaConfig(**kw)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": list(self.architectures), "model_type": self.model_type,
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
            "hidden_act": self.hidden_act, "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings, "attention_bias": self.attention_bias, "mlp_bias": self.mlp_bias,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids),
            "torch_dtype": self.torch_dtype,
        }
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        rs = self.rope_scaling
        if rs.rope_type == "linear":
            d["rope_scaling"] = {"rope_type": "linear", "factor": rs.factor}
        elif rs.rope_type == "llama3":
            d["rope_scaling"] = {"rope_type": "llama3", "factor": rs.factor, "low_freq_factor": rs.low_freq_factor,
                                 "high_freq_factor": rs.high_freq_factor,
                                 "original_max_position_embeddings": rs.original_max_position_embeddings}
        else:
            d["rope_scaling"] = None
        return d


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir!r}")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return d
