"""Token embedding (row lookup without scale, src/model.rs:334-339) and the output head
(final norm is a norm part; the head is one matrix, the token table itself when tied,
src/model.rs:602-607)."""
from __future__ import annotations

from ..kernels import ops
from .base import Part
from .registry import register_part
from .spec import TensorNeed


@register_part("embedding", "token_table")
class TokenEmbedding(Part):
    """params: vocab, width.  tensors: weight."""
    chain_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab"])
        self.width = int(spec.params["width"])
        self.weight = None

    def tensor_needs(self):
        return {self.spec.tensors["weight"]: TensorNeed((self.vocab, self.width), "embedding")}

    def load(self, tensors):
        self.weight = tensors[self.spec.tensors["weight"]]

    def forward(self, ctx, residual):
        ops.embed(self.weight, ctx.token_ids, residual[: ctx.n_tokens], ctx.status)


@register_part("head", "linear")
class LinearHead(Part):
    """params: vocab, width.  tensors: weight (names the token table when the head is tied, in
    which case both parts hold the same device tensor)."""
    chain_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab"])
        self.width = int(spec.params["width"])
        self.weight = None

    def tensor_needs(self):
        return {self.spec.tensors["weight"]: TensorNeed((self.vocab, self.width), "embedding")}

    def load(self, tensors):
        self.weight = tensors[self.spec.tensors["weight"]]

    def forward(self, h, logits, n_rows, status=None):
        ops.linear(h, self.weight, logits, n_rows, status=status)
