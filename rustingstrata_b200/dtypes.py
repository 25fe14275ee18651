"""The one table of element types: name, torch type, the code the kernels take, the safetensors tag.

Everything that names an element type - the engine option ``dtype``, the kernel launchers, the cache and state
allocation, the command line's spellings - looks it up here.  The kernel codes are those of ``RsDtype`` in
csrc/common.cuh (2 is the integer code ``rs_fill_random`` takes).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Union

import torch


@dataclass(frozen=True)
class ElementType:
    name: str
    torch: torch.dtype
    code: int              # what the kernels are told
    tag: str               # safetensors dtype tag
    itemsize: int
    aliases: tuple = ()


_TYPES = (
    ElementType("float32", torch.float32, 0, "F32", 4, ("fp32", "f32")),
    ElementType("bfloat16", torch.bfloat16, 1, "BF16", 2, ("bf16",)),
    ElementType("int32", torch.int32, 2, "I32", 4, ("i32",)),
)
_BY_KEY: Dict[object, ElementType] = {}
for _t in _TYPES:
    for _k in (_t.name, _t.torch, _t.tag, *_t.aliases):
        _BY_KEY[_k] = _t

# what an engine can compute in: "bfloat16" = the serving kernels, "float32" = true 32-bit everywhere
ENGINE_DTYPES = ("bfloat16", "float32")


def element_type(key: Union[str, torch.dtype, ElementType]) -> ElementType:
    """The table's row for a name ("bfloat16"), an alias ("bf16"), a safetensors tag ("BF16") or a torch type."""
    if isinstance(key, ElementType):
        return key
    try:
        return _BY_KEY[key]
    except KeyError:
        known = ", ".join(t.name for t in _TYPES)
        raise ValueError(f"unknown element type {key!r} (known: {known})") from None


def engine_dtype_name(key: str) -> str:
    """Canonical name of an engine compute type, accepting the command line's short spellings."""
    t = element_type(key)
    if t.name not in ENGINE_DTYPES:
        raise ValueError(f"dtype must be one of {ENGINE_DTYPES}, got {key!r}")
    return t.name
