"""Descriptions of parts, layers and whole models as plain data.

The reference describes a layer as a record of two norms, a mixer enum and a
feed-forward enum (``Layer``/``Mixer``/``Ffn``, src/gpu_model.rs:64-116) chosen per
layer from the configuration (``layers: Vec<LayerKind>``, src/config.rs:255-256).
Here the same idea is pure data: an architecture's builder turns its typed
configuration into a :class:`ModelSpec`; the generic model in ``models/causal_lm.py``
instantiates the named part classes from the part registry.  Nothing in a part refers
to the architecture that uses it: sizes and constants arrive in ``params`` and the
checkpoint's tensor names arrive in ``tensors``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered ``kind``, its numbers, and where its tensors live."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    # logical slot of the part (e.g. "q_proj") → tensor name in the checkpoint
    tensors: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class TensorNeed:
    """A tensor a part wants from the checkpoint.

    role: "matrix" (projection, drawn N(0, std) in random mode), "embedding"
    (token table, same distribution), "norm" (scale vector, ones or 1+N(0, s)),
    "int_table" (integer table kept as int32).
    """
    shape: Tuple[int, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement ("block") and the parts it arranges."""
    block: PartSpec
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec
    feed_forward_norm: PartSpec
    position: Optional[PartSpec] = None


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` and may occur more than once.  ``cache``
    is None when the call owns a cache of its own, or the index (into the order) of
    an earlier call whose cache this call reads without writing.
    """
    layer: int
    cache: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    name: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec


@dataclass(frozen=True)
class CacheNeed:
    """What one mixer call keeps per token: keys and values in pages.

    ``window`` None keeps every key; an integer keeps the most recent ``window`` keys
    (the current one included), so pages wholly older than that are given back.
    Calls with equal needs share a page pool ("cache group").
    """
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-request state of one mixer call (``numel`` float32 values, zeroed at admission)."""
    numel: int
