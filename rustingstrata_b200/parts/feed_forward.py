"""Gated feed-forward (SwiGLU): down(act(gate h) * (up h)), no biases.

Reference: src/model.rs:803-811,818-820 with silu(z) = z / (1 + exp(-z)) (src/ops.rs:14);
device: gate and up as one launch, then ``swiglu``, then down returned as a pending
residual (src/gpu_model.rs:3307-3328).  Here gate and up are one [2I, hidden] matrix,
and the down projection adds straight into the residual stream.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward
from .registry import register_part
from .spec import TensorNeed


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    """params: hidden, intermediate, activation ("silu").  tensors: gate_proj, up_proj, down_proj."""
    chain_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec.params["hidden"])
        self.inter = int(spec.params["intermediate"])
        act = spec.params.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"gated_mlp: activation '{act}' has no kernel (only 'silu')")
        runtime.scratch("gate_up", runtime.max_batch_tokens, 2 * self.inter)
        runtime.scratch("ff_act", runtime.max_batch_tokens, self.inter)
        self.w_gate_up = self.w_down = None

    def tensor_needs(self):
        t = self.spec.tensors
        return {t["gate_proj"]: TensorNeed((self.inter, self.hidden)),
                t["up_proj"]: TensorNeed((self.inter, self.hidden)),
                t["down_proj"]: TensorNeed((self.hidden, self.inter))}

    def load(self, tensors):
        t = self.spec.tensors
        g, u = tensors[t["gate_proj"]], tensors[t["up_proj"]]
        if g.dtype != u.dtype:
            raise ValueError("gated_mlp: gate and up projections must share an element type")
        # bfloat16 engine with 16-byte aligned rows: gate and up rows alternate, so the product's epilogue
        # applies SiLU(gate)*up to neighbouring accumulator columns and the [T, 2I] intermediate never
        # reaches memory.  Otherwise [gate; up] stacked, followed by the separate activation kernel.
        self.fused = (g.dtype == torch.bfloat16 and self.runtime.dtype == torch.bfloat16 and self.hidden % 8 == 0)
        if self.fused:
            self.w_gate_up = torch.stack([g, u], dim=1).reshape(2 * self.inter, self.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors[t["down_proj"]].contiguous()

    def forward(self, h, residual, ctx):
        rt = self.runtime
        T = ctx.n_tokens
        gate_up = rt.get_scratch("gate_up")[:, : 2 * self.inter]
        act = rt.get_scratch("ff_act")[:, : self.inter]
        if self.fused:
            ops.linear_swiglu(h, self.w_gate_up, act, T, status=ctx.status)
        else:
            ops.linear(h, self.w_gate_up, gate_up, T)
            ops.silu_mul(gate_up, act, T)
        ctx.owed = ops.linear(act, self.w_down, residual, T, accumulate=True, status=ctx.status, may_defer=ctx.may_owe)
