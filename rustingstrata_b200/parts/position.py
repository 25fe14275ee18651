"""Rotary position encoding, NEOX pairing (i, i + n_rot/2).

Reference: theta = pos * base^(-2i/n_rot) in float64, sin/cos rounded to float32
(src/ops.rs:36-45; device src/cuda/kernels.cu:2192-2194,2212-2220).  Here the table
[position, cos(n_rot/2) | sin(n_rot/2)] is computed once on the host in float64 for all
positions the engine can reach and shared by every layer with the same parameters.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding
from .registry import register_part


@register_part("position", "rope_neox")
class RotaryNeox(PositionEncoding):
    """params: n_rot (rotated dims of a head), base."""
    chain_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.n_rot = int(spec.params["n_rot"])
        self.base = float(spec.params["base"])
        if self.n_rot % 2:
            raise ValueError(f"rope_neox: n_rot {self.n_rot} must be even")
        self._key = ("rope_neox", self.n_rot, self.base, runtime.max_positions)

    @property
    def cos_sin(self) -> torch.Tensor:
        """[positions, cos(n_rot/2) | sin(n_rot/2)] float32, built at first use, one per parameter set."""
        return self.runtime.shared(self._key, self._table)

    def _table(self) -> torch.Tensor:
        half = self.n_rot // 2
        i = np.arange(half, dtype=np.float64)
        # the reference holds the base as float32 and widens it (src/ops.rs:39)
        inv = np.power(np.float64(np.float32(self.base)), -2.0 * i / self.n_rot)
        theta = np.arange(self.runtime.max_positions, dtype=np.float64)[:, None] * inv[None, :]
        tab = np.concatenate([np.cos(theta), np.sin(theta)], axis=1).astype(np.float32)
        return torch.from_numpy(tab).to(self.runtime.device)


@register_part("position", "none")
class NoPosition(PositionEncoding):
    chain_safe = True
    n_rot = 0
    cos_sin = None
