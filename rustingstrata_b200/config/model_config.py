"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference keeps one struct of hyper-parameters per model (``ModelConfig``,
src/config.rs:196-262) filled from file metadata, with a per-architecture table of
flags (src/config.rs:56-87).  Here every architecture owns a small frozen dataclass
whose fields are exactly the ``config.json`` keys it reads; the key names and the
defaults of the optional ones follow the reference's two ``config.json`` readers
(src/gguf.rs:397-412 and src/gguf.rs:496-532).

No size or constant that ``config.json`` gives is written anywhere else in the
package: parts receive them as constructor parameters.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A ``config.json`` that cannot be turned into a typed configuration."""


def _require(d: Mapping[str, Any], key: str, typ, where: str):
    if key not in d or d[key] is None:
        raise ConfigError(f"{where}: missing required key '{key}'")
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{where}: key '{key}' must be an integer, got {v!r}")
        if v <= 0:
            raise ConfigError(f"{where}: key '{key}' must be positive, got {v}")
    elif typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{where}: key '{key}' must be a number, got {v!r}")
        v = float(v)
    return v


FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclass(frozen=True)
class Qwen3Config:
    """Hyper-parameters of the Qwen3 dense decoder.

    Reference keys (GGUF metadata → ``config.json``): block_count →
    num_hidden_layers, embedding_length → hidden_size, attention.head_count →
    num_attention_heads, attention.head_count_kv → num_key_value_heads,
    attention.key_length → head_dim (default hidden/heads, src/config.rs:299),
    rope.freq_base → rope_theta, attention.layer_norm_rms_epsilon → rms_norm_eps
    (required, src/config.rs:370), feed_forward_length → intermediate_size,
    attention.sliding_window(+pattern) → sliding_window + layer_types
    (src/config.rs:350-353, src/gguf.rs:511,529).
    """

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    # one entry per layer: FULL_ATTENTION or SLIDING_ATTENTION
    layer_types: Tuple[str, ...]
    # number of most recent keys (the current one included) a sliding layer sees; None if no layer slides
    sliding_window: Optional[int] = None
    hidden_act: str = "silu"
    architecture: str = "Qwen3ForCausalLM"
    model_type: str = "qwen3"
    torch_dtype: str = "bfloat16"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str = "config.json") -> "Qwen3Config":
        n_layer = _require(d, "num_hidden_layers", int, where)
        hidden = _require(d, "hidden_size", int, where)
        n_head = _require(d, "num_attention_heads", int, where)
        n_kv = _require(d, "num_key_value_heads", int, where)
        inter = _require(d, "intermediate_size", int, where)
        vocab = _require(d, "vocab_size", int, where)
        eps = _require(d, "rms_norm_eps", float, where)
        max_pos = _require(d, "max_position_embeddings", int, where)
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % n_head:
                raise ConfigError(f"{where}: no 'head_dim' and hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {n_head}")
            head_dim = hidden // n_head
        elif isinstance(head_dim, bool) or not isinstance(head_dim, int) or head_dim <= 0:
            raise ConfigError(f"{where}: key 'head_dim' must be a positive integer, got {head_dim!r}")
        theta = None
        rp = d.get("rope_parameters")
        if isinstance(rp, Mapping) and rp.get("rope_theta") is not None:
            theta = rp["rope_theta"]
            kind = rp.get("rope_type", rp.get("type", "default"))
            if kind not in (None, "default"):
                raise ConfigError(f"{where}: rope_parameters.rope_type '{kind}' is not supported "
                                  f"(only the default rotary encoding)")
        elif d.get("rope_theta") is not None:
            theta = d["rope_theta"]
        if theta is None:
            raise ConfigError(f"{where}: missing required key 'rope_theta'")
        if isinstance(theta, bool) or not isinstance(theta, (int, float)) or theta <= 0:
            raise ConfigError(f"{where}: 'rope_theta' must be a positive number, got {theta!r}")
        scaling = d.get("rope_scaling")
        if scaling not in (None, {}):
            kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, Mapping) else scaling
            if kind not in (None, "default"):
                raise ConfigError(f"{where}: rope_scaling {scaling!r} is not supported")
        if d.get("attention_bias", False):
            raise ConfigError(f"{where}: attention_bias=true is not supported (this architecture has no biases)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"{where}: hidden_act '{act}' is not supported (only 'silu')")
        if n_head % n_kv:
            raise ConfigError(f"{where}: num_attention_heads {n_head} is not a multiple of "
                              f"num_key_value_heads {n_kv}")
        if head_dim % 2:
            raise ConfigError(f"{where}: head_dim {head_dim} must be even for rotary pairs")

        use_window = bool(d.get("use_sliding_window", False))
        window = d.get("sliding_window")
        lt = d.get("layer_types")
        if use_window:
            if isinstance(window, bool) or not isinstance(window, int) or window <= 0:
                raise ConfigError(f"{where}: use_sliding_window=true needs a positive integer 'sliding_window', "
                                  f"got {window!r}")
            if lt is not None:
                if not isinstance(lt, (list, tuple)) or len(lt) != n_layer:
                    raise ConfigError(f"{where}: 'layer_types' must list {n_layer} layers, got {lt!r}")
                for t in lt:
                    if t not in (FULL_ATTENTION, SLIDING_ATTENTION):
                        raise ConfigError(f"{where}: unknown layer type {t!r} in 'layer_types'")
                layer_types = tuple(lt)
            else:
                first = d.get("max_window_layers", 0)
                if isinstance(first, bool) or not isinstance(first, int) or first < 0:
                    raise ConfigError(f"{where}: 'max_window_layers' must be a non-negative integer, got {first!r}")
                layer_types = tuple(SLIDING_ATTENTION if i >= first else FULL_ATTENTION for i in range(n_layer))
        else:
            layer_types = tuple(FULL_ATTENTION for _ in range(n_layer))
        if SLIDING_ATTENTION not in layer_types:
            window = None
        archs = d.get("architectures") or ["Qwen3ForCausalLM"]
        return cls(
            vocab_size=vocab, hidden_size=hidden, num_hidden_layers=n_layer, num_attention_heads=n_head,
            num_key_value_heads=n_kv, head_dim=int(head_dim), intermediate_size=inter, rms_norm_eps=float(eps),
            rope_theta=float(theta), max_position_embeddings=max_pos,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)), layer_types=layer_types,
            sliding_window=window, hidden_act=act, architecture=str(archs[0]),
            model_type=str(d.get("model_type", "qwen3")), torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        slides = SLIDING_ATTENTION in self.layer_types
        out = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "hidden_act": self.hidden_act,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "attention_bias": False,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": slides,
            "sliding_window": self.sliding_window if slides else None,
            "torch_dtype": self.torch_dtype,
        }
        if slides:
            out["layer_types"] = list(self.layer_types)
        return out


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file (a model folder holds config.json and model.safetensors)")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d
