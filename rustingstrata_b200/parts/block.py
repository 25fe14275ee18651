"""Arrangement of a layer's parts around the residual stream.

Reference ``block`` (src/model.rs:587-599): x += mixer(norm(x)); x += ffn(norm(x)).
The residual stream is float32 in both engines; the norm writes the activation type.
"""
from __future__ import annotations

from .base import Block
from .registry import register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """params: hidden.  Made of: mixer_norm, mixer, feed_forward_norm, feed_forward (and a position encoding for
    the mixer, if the layer lists one)."""
    chain_safe = True
    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, spec, runtime, parts):
        super().__init__(spec, runtime, parts)
        self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
        self.ff_norm, self.feed_forward = parts["feed_forward_norm"], parts["feed_forward"]
        self.hidden = int(spec.params["hidden"])
        runtime.scratch("normed", runtime.max_batch_tokens, self.hidden)

    @property
    def first_reader_takes_owed(self):
        return getattr(self.mixer_norm, "takes_owed", False)

    def forward(self, residual, ctx, call):
        h = self.runtime.get_scratch("normed")[:, : self.hidden]
        self.norm_of_stream(self.mixer_norm, residual, h, ctx)
        ctx.may_owe = getattr(self.ff_norm, "takes_owed", False)
        self.mixer.forward(h, residual, ctx, call.mixers["mixer"])
        ctx.may_owe = False
        self.norm_of_stream(self.ff_norm, residual, h, ctx)
        ctx.may_owe = ctx.next_block_takes_owed
        self.feed_forward.forward(h, residual, ctx)
        ctx.may_owe = False
