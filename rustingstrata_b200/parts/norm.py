"""RMSNorm: out = x * rsqrt(mean(x^2) + eps) * w   (reference src/ops.rs:3-7; device
src/cuda/kernels.cu:1504-1552).  ``eps`` and the width are parameters."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm
from .registry import register_part
from .spec import TensorNeed


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """params: width, eps.  tensors: weight."""
    chain_safe = True
    takes_owed = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    def tensor_needs(self):
        return {self.spec.tensors["weight"]: TensorNeed((self.width,), "norm")}

    def load(self, tensors):
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()

    def forward(self, x, out, n_rows, rows=None, owed=None):
        ops.rmsnorm(x, self.weight, self.eps, out, rows=rows, n_rows=n_rows, pending=owed)
