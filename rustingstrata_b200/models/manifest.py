"""The tensor manifest of a configuration without touching a GPU (for the random-weights writer)."""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..config.registry import resolve_architecture
from ..parts import Runtime, TensorNeed
from .causal_lm import CausalLM


def manifest_for(config_dict: Mapping) -> Dict[str, TensorNeed]:
    """Tensor name → (shape, role) for the model a config.json describes."""
    arch = resolve_architecture(config_dict)
    cfg = arch.config_class.from_dict(config_dict)
    spec = arch.build_spec(cfg)
    rt = Runtime(torch.bfloat16, torch.device("cpu"), 1, 1, 1, 16, spec.max_positions, 16)
    return CausalLM(spec, rt).tensor_needs()
