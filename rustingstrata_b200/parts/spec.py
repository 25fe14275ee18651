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
from typing import Any, Dict, Mapping, Optional, Tuple, Union


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
    """One layer: the arrangement ("block") and the parts it arranges, by role.

    Which roles exist, and which category of part fills each, is the block kind's business (its class attribute
    ``roles``): the pre-norm block wants ``mixer_norm``, ``mixer``, ``feed_forward_norm`` and ``feed_forward``; a
    block with post-norms, with one norm before a parallel mixer and feed-forward, or with two mixers names other
    roles.  A role whose category is "position" is handed to the mixers of the layer: ``<mixer role>_position`` to
    that mixer, plain ``position`` to every mixer that has none of its own.
    """
    block: PartSpec
    parts: Mapping[str, PartSpec] = field(default_factory=dict)

    @classmethod
    def pre_norm(cls, block: PartSpec, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: PartSpec,
                 feed_forward_norm: PartSpec, position: Optional[PartSpec] = None) -> "LayerSpec":
        """The usual decoder layer: x += mixer(norm(x)); x += feed_forward(norm(x))."""
        parts = {"mixer_norm": mixer_norm, "mixer": mixer, "feed_forward_norm": feed_forward_norm,
                 "feed_forward": feed_forward}
        if position is not None:
            parts["position"] = position
        return cls(block, parts)


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` and may occur more than once.  ``cache``
    is None when the call owns a cache of its own, or the index (into the order) of
    an earlier call whose cache this call reads without writing; in a layer with
    several mixers it may be a mapping mixer role → index for the mixers that borrow.
    """
    layer: int
    cache: Union[None, int, Mapping[str, int]] = None


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
    """Fixed-size per-request state of one mixer call: ``numel`` values of element type ``dtype`` (a name of the
    element-type table: "float32", "bfloat16", "int32"), zeroed at admission."""
    numel: int
    dtype: str = "float32"
