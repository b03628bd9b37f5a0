"""Typed model configuration read from an architecture's own `config.json` keys.

Role of the reference's `Config` struct and `config_from_gguf` (src/model.br:28-76, 380-513):
every hyper-parameter is a field read from the file, "never hardcoded to one architecture's
values" (src/model.br:6-8); required keys raise, optional keys have the reference's defaults.
"""
from __future__ import annotations

import json
import os
import warnings
from dataclasses import dataclass, field
from typing import Any, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model: missing key, bad value, unsupported option."""


_MISSING = object()


def _get(d: dict, key: str, kind, default=_MISSING):
    """Reads `key` with a type check; a missing required key raises like src/model.br:381-391."""
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: missing required key '{key}'")
        return default
    v = d[key]
    if kind is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if kind is int and isinstance(v, bool):
        raise ConfigError(f"config.json: key '{key}' must be an integer, got {v!r}")
    if not isinstance(v, kind):
        raise ConfigError(f"config.json: key '{key}' must be {kind.__name__}, got {v!r}")
    return v


def _positive(name: str, v: int) -> int:
    if v <= 0:
        raise ConfigError(f"config.json: '{name}' must be positive, got {v}")
    return v


# Keys that exist in published config.json files of this family and do not change inference math.
_INERT_KEYS = {
    "architectures", "model_type", "attention_dropout", "initializer_range", "use_cache",
    "torch_dtype", "dtype", "transformers_version", "bos_token_id", "eos_token_id", "pad_token_id",
    "_name_or_path", "use_mrope", "output_attentions", "output_hidden_states",
}


@dataclass(frozen=True)
class Qwen2Config:
    """Dense Qwen2 decoder: GQA attention with Q/K/V bias, NEOX rotary positions, RMSNorm, SwiGLU.

    Field ↔ reference `Config` field (src/model.br:28-76) ↔ config.json key:
    vocab_size ↔ vocab_size, hidden_size ↔ d_model, num_hidden_layers ↔ n_layer,
    num_attention_heads ↔ n_head, num_key_value_heads ↔ n_kv_head (default n_head, :385),
    head_dim ↔ d_head (default d_model / n_head, :410), intermediate_size ↔ ffn_dim,
    rope_theta ↔ rope_freq_base (default 10000, :393), rms_norm_eps ↔ rms_eps (default 1e-6, :398),
    tie_word_embeddings ↔ tied_embeddings (:402-405), layer_windows ↔ layer_window (:948-970).
    """
    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    hidden_act: str = "silu"
    attention_bias: bool = True
    # one entry per layer: 0 = every earlier key, n > 0 = the last n positions, itself included
    layer_windows: Tuple[int, ...] = ()
    eos_token_ids: Tuple[int, ...] = ()
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    ARCHITECTURES = ("Qwen2ForCausalLM",)
    MODEL_TYPES = ("qwen2",)

    @classmethod
    def from_dict(cls, d: dict) -> "Qwen2Config":
        arch = architecture_name(d)
        n_layer = _positive("num_hidden_layers", _get(d, "num_hidden_layers", int))
        hidden = _positive("hidden_size", _get(d, "hidden_size", int))
        n_head = _positive("num_attention_heads", _get(d, "num_attention_heads", int))
        n_kv = _positive("num_key_value_heads", _get(d, "num_key_value_heads", int, n_head))
        if n_head % n_kv != 0:
            raise ConfigError(
                f"config.json: num_attention_heads ({n_head}) must be a multiple of "
                f"num_key_value_heads ({n_kv})")
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _positive("head_dim", _get(d, "head_dim", int))
        else:
            if hidden % n_head != 0:
                raise ConfigError(
                    f"config.json: hidden_size ({hidden}) is not a multiple of num_attention_heads "
                    f"({n_head}) and no head_dim is given")
            head_dim = hidden // n_head
        if head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim ({head_dim}) must be even for rotary pairs")
        ffn = _positive("intermediate_size", _get(d, "intermediate_size", int))
        vocab = _positive("vocab_size", _get(d, "vocab_size", int))
        rope_params = d.get("rope_parameters") or {}
        if "rope_theta" in d and d["rope_theta"] is not None:
            theta = _get(d, "rope_theta", float)
        else:
            theta = _get(rope_params, "rope_theta", float, 10000.0)
        if theta <= 0:
            raise ConfigError(f"config.json: rope_theta must be positive, got {theta}")
        scaling = d.get("rope_scaling")
        if scaling is None and rope_params.get("rope_type") not in (None, "default"):
            scaling = rope_params
        if scaling:
            kind = scaling.get("rope_type", scaling.get("type"))
            if kind not in (None, "default"):
                raise ConfigError(
                    f"config.json: rope_scaling of type {kind!r} is not supported "
                    f"(only plain rotary positions)")
        eps = _get(d, "rms_norm_eps", float, 1e-6)
        if not eps > 0:
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {eps}")
        act = _get(d, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (only 'silu')")
        max_pos = _positive("max_position_embeddings", _get(d, "max_position_embeddings", int, 32768))
        tied = _get(d, "tie_word_embeddings", bool, False)
        bias = _get(d, "attention_bias", bool, True)
        windows = cls._layer_windows(d, n_layer)
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"config.json: eos_token_id must be an integer or a list of them, got {eos!r}")
        known = set(_INERT_KEYS) | {
            "num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
            "intermediate_size", "vocab_size", "rope_theta", "rope_parameters", "rope_scaling",
            "rms_norm_eps", "hidden_act", "max_position_embeddings", "tie_word_embeddings",
            "attention_bias", "use_sliding_window", "sliding_window", "max_window_layers", "layer_types"}
        unknown = sorted(k for k in d if k not in known and not k.startswith("_"))
        if unknown:
            warnings.warn(f"config.json: keys not used by {arch}: {', '.join(unknown)}")
        return cls(architecture=arch, vocab_size=vocab, hidden_size=hidden, num_hidden_layers=n_layer,
                   num_attention_heads=n_head, num_key_value_heads=n_kv, head_dim=head_dim,
                   intermediate_size=ffn, rope_theta=float(theta), rms_norm_eps=float(eps),
                   tie_word_embeddings=tied, max_position_embeddings=max_pos, hidden_act=act,
                   attention_bias=bias, layer_windows=windows, eos_token_ids=eos_ids, raw=dict(d))

    @staticmethod
    def _layer_windows(d: dict, n_layer: int) -> Tuple[int, ...]:
        """Per-layer window. `layer_types` wins when present; else layers from `max_window_layers`
        on use `sliding_window` when `use_sliding_window` is true. A window of n means a query sees
        the last n positions, itself included (src/math.br:296-298, 327-328)."""
        use = _get(d, "use_sliding_window", bool, False)
        types = d.get("layer_types")
        if types is not None:
            if not isinstance(types, list) or len(types) != n_layer:
                raise ConfigError(f"config.json: layer_types must list {n_layer} layers, got {types!r}")
            for t in types:
                if t not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"config.json: unknown layer type {t!r} in layer_types")
            sliding = [t == "sliding_attention" for t in types]
        elif use:
            first = _get(d, "max_window_layers", int, n_layer)
            sliding = [i >= first for i in range(n_layer)]
        else:
            sliding = [False] * n_layer
        if not any(sliding):
            return tuple(0 for _ in range(n_layer))
        win = _positive("sliding_window", _get(d, "sliding_window", int))
        return tuple(win if s else 0 for s in sliding)

    def to_dict(self) -> dict:
        """A config.json that reads back to the same configuration."""
        d = {
            "architectures": [self.architecture], "model_type": "qwen2",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers, "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size, "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps, "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings, "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
        }
        if any(self.layer_windows):
            d["use_sliding_window"] = True
            d["sliding_window"] = max(self.layer_windows)
            d["layer_types"] = ["sliding_attention" if w else "full_attention" for w in self.layer_windows]
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d


def architecture_name(d: dict) -> str:
    """The name the registry dispatches on: `architectures[0]`, else `model_type`
    (role of `general.architecture`, src/model.br:381)."""
    archs = d.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    mt = d.get("model_type")
    if isinstance(mt, str):
        return mt
    raise ConfigError("config.json: missing required key 'architectures' (or 'model_type')")


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json in the model folder")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return d
