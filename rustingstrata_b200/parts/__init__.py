from .spec import PartSpec, TensorNeed, LayerSpec, LayerCall, ModelSpec, CacheNeed, StateNeed
from .registry import register_part, unregister_part, part_class, registered_parts, CATEGORIES
from .base import (Runtime, HostBatch, CallInfo, LayerCallInfo, StepContext, Part, Mixer, FeedForward, Norm, PositionEncoding, Block)
# importing the modules registers the built-in parts
from . import norm, position, attention, feed_forward, block, embedding  # noqa: E402,F401
