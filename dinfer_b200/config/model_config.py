"""Typed model configurations, read from an architecture's own ``config.json`` keys.

Every size and constant of a model comes from here; nothing in the parts or the kernels
stands in for a value that ``config.json`` gives.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, Dict, Optional, Tuple


class ConfigError(ValueError):
    """A ``config.json`` that is incomplete, of the wrong type, or outside what the engine runs."""


_MISSING = object()


def _take(d: Dict[str, Any], key: str, kind, default=_MISSING):
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: missing key '{key}'")
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
    return v


@dataclass(frozen=True)
class Qwen3Config:
    """``config.json`` of ``Qwen3ForCausalLM``.

    Same keys, defaults and refusals as the reference's ``Qwen3Config``
    (models/qwen3/src/config.rs:6-56): the first ten keys have no default; ``head_dim`` is
    explicit and may differ from ``hidden_size / num_attention_heads``; attention bias, a
    sliding window and activations other than silu are refused.
    """

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    sliding_window: Optional[int] = None
    use_sliding_window: bool = False
    hidden_act: str = "silu"
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Qwen3ForCausalLM"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen3Config":
        eos = d.get("eos_token_id")
        if isinstance(eos, bool):
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(x) for x in eos if isinstance(x, int) and not isinstance(x, bool))
        else:
            eos_ids = ()
        if d.get("rope_scaling") not in (None, {}):
            rs = d["rope_scaling"]
            kind = rs.get("rope_type", rs.get("type")) if isinstance(rs, dict) else rs
            if kind not in (None, "default"):
                raise ConfigError(f"config.json: rope_scaling {kind!r} is not supported")
        archs = d.get("architectures") or ["Qwen3ForCausalLM"]
        cfg = cls(
            vocab_size=_take(d, "vocab_size", int),
            hidden_size=_take(d, "hidden_size", int),
            intermediate_size=_take(d, "intermediate_size", int),
            num_hidden_layers=_take(d, "num_hidden_layers", int),
            num_attention_heads=_take(d, "num_attention_heads", int),
            num_key_value_heads=_take(d, "num_key_value_heads", int),
            head_dim=_take(d, "head_dim", int),
            rms_norm_eps=_take(d, "rms_norm_eps", float),
            rope_theta=_take(d, "rope_theta", float),
            max_position_embeddings=_take(d, "max_position_embeddings", int),
            tie_word_embeddings=_take(d, "tie_word_embeddings", bool, False),
            attention_bias=_take(d, "attention_bias", bool, False),
            sliding_window=_take(d, "sliding_window", int, None),
            use_sliding_window=_take(d, "use_sliding_window", bool, False),
            hidden_act=_take(d, "hidden_act", str, "silu"),
            eos_token_ids=eos_ids,
            architecture=str(archs[0]),
        )
        cfg.check()
        return cfg

    def check(self) -> None:
        for f in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "num_attention_heads", "num_key_value_heads", "head_dim",
                  "max_position_embeddings"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"config.json: '{f}' must be positive, got {getattr(self, f)}")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: unsupported hidden_act {self.hidden_act!r}")
        if self.attention_bias:
            raise ConfigError("config.json: attention_bias is not supported")
        if self.use_sliding_window:
            raise ConfigError("config.json: sliding window is not supported")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config.json: heads {self.num_attention_heads} not divisible by kv heads "
                f"{self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even (rotary pairs)")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"config.json: rope_theta must be positive, got {self.rope_theta}")

    # derived sizes (models/qwen3/src/config.rs:66-77)
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def to_dict(self) -> Dict[str, Any]:
        """The ``config.json`` dictionary that reads back as this configuration."""
        d: Dict[str, Any] = {"architectures": [self.architecture], "model_type": "qwen3"}
        for f in fields(self):
            if f.name in ("eos_token_ids", "architecture"):
                continue
            d[f.name] = getattr(self, f.name)
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        return d


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    _merge_generation_eos(model_dir, d)
    return d


def _merge_generation_eos(model_dir: str, d: Dict[str, Any]) -> None:
    """End-of-sequence ids that only ``generation_config.json`` names join those of config.json
    (the reference takes its stop ids from the generation config too: crates/server/src/service.rs:407)."""
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.isfile(path):
        return
    with open(path, "r", encoding="utf-8") as f:
        try:
            g = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
    extra = g.get("eos_token_id") if isinstance(g, dict) else None
    if extra is None:
        return
    def as_list(v):
        return [] if v is None else (list(v) if isinstance(v, (list, tuple)) else [v])
    have = as_list(d.get("eos_token_id"))
    merged = have + [t for t in as_list(extra) if t not in have]
    if not all(isinstance(t, int) and not isinstance(t, bool) for t in merged):
        raise ConfigError(f"{path}: eos_token_id must be an integer or a list of integers")
    d["eos_token_id"] = merged if len(merged) != 1 else merged[0]
