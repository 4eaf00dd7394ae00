"""Typed model configuration read from an architecture's own ``config.json`` keys.

``read_model_dir`` loads the raw json (plus ``generation_config.json`` when present);
an architecture's config class then picks its own keys out of it.  Every size and
constant a model needs comes from here: nothing in the parts or kernels assumes one.

Keys, defaults and precedence follow CodeMan62/lily's
lily/models/model_config.py:85-170.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a model of the requested architecture."""


def read_model_dir(model_dir: str) -> Tuple[Dict[str, Any], Dict[str, Any]]:
    """Returns (config.json, generation_config.json or {})."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{model_dir!r} has no config.json")
    with open(path) as f:
        cfg = json.load(f)
    gen: Dict[str, Any] = {}
    gpath = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gpath):
        with open(gpath) as f:
            gen = json.load(f)
    return cfg, gen


def _require(d: Dict[str, Any], key: str, kind=int):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks the required key {key!r}")
    try:
        return kind(d[key])
    except (TypeError, ValueError):
        raise ConfigError(f"config.json key {key!r} = {d[key]!r} is not {kind.__name__}") from None


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of the rotary table (lily/layers/rotary.py:90-119,196-207)."""

    rope_type: str = "default"          # "default" | "llama3"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 1.0
    original_max_position_embeddings: int = 0

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> "RopeScaling":
        if not d:
            return cls()
        rtype = d.get("rope_type", d.get("type", "default"))   # model_config.py:108-109
        if rtype == "default":
            return cls()
        if rtype != "llama3":
            raise ConfigError(f"rope scaling type {rtype!r} is not supported (have: default, llama3)")
        try:
            return cls("llama3", float(d["factor"]), float(d["low_freq_factor"]), float(d["high_freq_factor"]),
                       int(d["original_max_position_embeddings"]))
        except KeyError as e:
            raise ConfigError(f"llama3 rope scaling lacks {e.args[0]!r}") from None

    def to_dict(self) -> Optional[Dict[str, Any]]:
        if self.rope_type == "default":
            return None
        return {"rope_type": self.rope_type, "factor": self.factor, "low_freq_factor": self.low_freq_factor,
                "high_freq_factor": self.high_freq_factor,
                "original_max_position_embeddings": self.original_max_position_embeddings}


@dataclass
class DenseDecoderConfig:
    """Llama / Qwen3 dense decoder (lily/models/llama.py, lily/models/qwen3.py)."""

    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    partial_rotary_factor: float = 1.0
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 4096
    hidden_act: str = "silu"
    attention_bias: bool = False
    qk_norm: bool = False
    torch_dtype: str = "bfloat16"
    model_type: str = ""
    eos_token_ids: List[int] = field(default_factory=list)
    bos_token_id: Optional[int] = None

    # architectures whose attention normalises each q and k head before the rotation
    # (a property of the class in the reference, not a config key: lily/models/qwen3.py:17-37)
    QK_NORM_ARCHITECTURES = ("Qwen3ForCausalLM",)

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any], generation: Optional[Dict[str, Any]] = None,
                  architecture: Optional[str] = None) -> "DenseDecoderConfig":
        text = cfg.get("text_config", cfg)
        arch = architecture or (cfg.get("architectures") or [""])[0]
        heads = _require(text, "num_attention_heads")
        hidden = _require(text, "hidden_size")
        rope_scaling = text.get("rope_scaling")
        rope_params = text.get("rope_parameters")
        theta = text.get("rope_theta", 10000.0)
        if rope_params:
            theta = rope_params.get("rope_theta", theta)
            if rope_params.get("rope_type", "default") != "default":
                rope_scaling = dict(rope_params)
        # options of other decoders that this architecture's code does not have (lily/models/llama.py:36-38 has no
        # MLP bias; its attention sees every earlier key): a file that turns one on would get other results
        if text.get("mlp_bias"):
            raise ConfigError("mlp_bias is set: this architecture's feed-forward has no bias")
        if text.get("use_sliding_window") and text.get("sliding_window"):
            raise ConfigError(f"use_sliding_window is set (window {text.get('sliding_window')}): this architecture "
                              "attends to every earlier key")
        eos = (generation or {}).get("eos_token_id", text.get("eos_token_id"))
        eos_ids = [] if eos is None else [int(eos)] if isinstance(eos, int) else [int(e) for e in eos]
        out = cls(
            architecture=arch,
            hidden_size=hidden,
            num_hidden_layers=_require(text, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=int(text.get("num_key_value_heads") or heads),
            head_dim=int(text.get("head_dim") or hidden // heads),
            intermediate_size=_require(text, "intermediate_size"),
            vocab_size=_require(text, "vocab_size"),
            rms_norm_eps=float(text.get("rms_norm_eps", 1e-6)),
            rope_theta=float(theta),
            rope_scaling=RopeScaling.from_dict(rope_scaling),
            partial_rotary_factor=float(text.get("partial_rotary_factor",
                                                 (rope_params or {}).get("partial_rotary_factor", 1.0))),
            tie_word_embeddings=bool(text.get("tie_word_embeddings", cfg.get("tie_word_embeddings", False))),
            max_position_embeddings=int(text.get("max_position_embeddings", 4096)),
            hidden_act=str(text.get("hidden_act", "silu")),
            attention_bias=bool(text.get("attention_bias", False)),
            qk_norm=arch in cls.QK_NORM_ARCHITECTURES,
            torch_dtype=str(text.get("torch_dtype") or text.get("dtype") or cfg.get("torch_dtype") or "bfloat16"),
            model_type=str(cfg.get("model_type", "")),
            eos_token_ids=eos_ids,
            bos_token_id=text.get("bos_token_id"),
        )
        out.validate()
        return out

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)   # model_config.py:174-176

    def validate(self) -> None:
        pos = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
               "intermediate_size", "vocab_size", "max_position_embeddings")
        for k in pos:
            if getattr(self, k) <= 0:
                raise ConfigError(f"{k} must be positive, got {getattr(self, k)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.hidden_act != "silu":
            raise ConfigError(f"Unsupported activation {self.hidden_act!r}")    # lily/models/llama.py:39-40
        if self.rotary_dim <= 0 or self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ConfigError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be positive")

    def to_hf_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        d: Dict[str, Any] = {
            "architectures": [self.architecture], "model_type": self.model_type,
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings, "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias, "torch_dtype": self.torch_dtype,
        }
        if self.partial_rotary_factor != 1.0:
            d["partial_rotary_factor"] = self.partial_rotary_factor
        if self.rope_scaling.to_dict() is not None:
            d["rope_scaling"] = self.rope_scaling.to_dict()
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    def summary(self) -> str:
        return (f"{self.architecture} layers={self.num_hidden_layers} hidden={self.hidden_size} "
                f"heads={self.num_attention_heads}/{self.num_key_value_heads} head_dim={self.head_dim} "
                f"inter={self.intermediate_size} vocab={self.vocab_size} tied={self.tie_word_embeddings} "
                f"qk_norm={self.qk_norm} rope_theta={self.rope_theta} scaling={self.rope_scaling.rope_type} "
                f"eps={self.rms_norm_eps} ctx={self.max_position_embeddings}")
