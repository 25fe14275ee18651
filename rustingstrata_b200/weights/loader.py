"""Loading a checkpoint against a model's tensor manifest.

The reference looks tensors up by name in a memory-mapped file and fails on the first
missing one (``Weights::get``, src/weights.rs:166-187; shape/type validation
src/weights.rs:243-255).  Here the model states every tensor it wants (name → shape),
the loader compares that manifest with the file once, and a single
:class:`WeightsError` lists every missing tensor, every unexpected tensor and every
wrong shape.

Element types: a tensor stored as BF16 stays bfloat16; one stored as F32 stays float32
(in the 32-bit engine everything floating is widened to float32; F16 is widened to
float32 as the reference does on upload, src/backend.rs:156-164); integer tables
become int32.
"""
from __future__ import annotations

from typing import Dict, Mapping

import numpy as np
import torch

from ..parts.spec import TensorNeed
from .safetensors_io import SafetensorsError, TensorEntry, TensorFileReader, index_model_dir


class WeightsError(ValueError):
    def __init__(self, where: str, missing, unexpected, wrong_shape, wrong_type=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.wrong_type = sorted(wrong_type)
        lines = [f"{where}: the checkpoint does not match the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " +
                         "; ".join(f"{n}: file {list(got)} vs model {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_type:
            lines.append(f"  wrong element types ({len(self.wrong_type)}): " +
                         "; ".join(f"{n}: {t}" for n, t in self.wrong_type))
        super().__init__("\n".join(lines))


_FLOAT_TAGS = ("BF16", "F16", "F32", "F64")
_INT_TAGS = ("I64", "I32", "I16", "I8", "U8")


def _strip(name: str) -> str:
    return name[len("model."):] if name.startswith("model.") else name


def match_names(manifest: Mapping[str, TensorNeed], entries: Mapping[str, TensorEntry]):
    """Pairs manifest names with file names; a leading ``model.`` may be present or absent on either side."""
    by_stripped = {}
    for n in entries:
        by_stripped.setdefault(_strip(n), n)
    pairs, missing = {}, []
    used = set()
    for want in manifest:
        if want in entries:
            pairs[want] = want
            used.add(want)
        elif _strip(want) in by_stripped and by_stripped[_strip(want)] not in used:
            pairs[want] = by_stripped[_strip(want)]
            used.add(by_stripped[_strip(want)])
        else:
            missing.append(want)
    unexpected = [n for n in entries if n not in used]
    return pairs, missing, unexpected


def to_torch(arr: np.ndarray, tag: str, engine_dtype: torch.dtype, role: str) -> torch.Tensor:
    """One file tensor as a CPU torch tensor of the type the engine keeps it in."""
    if role == "int_table":
        return torch.from_numpy(arr.astype(np.int32))
    if tag == "BF16":
        t = torch.from_numpy(arr.copy() if not arr.flags.writeable else arr).view(torch.bfloat16)
        return t.to(torch.float32) if engine_dtype == torch.float32 else t
    if tag == "F32":
        return torch.from_numpy(arr.copy() if not arr.flags.writeable else arr)
    if tag in ("F16", "F64"):
        return torch.from_numpy(arr.astype(np.float32))
    raise AssertionError(tag)


def load_checkpoint(model_dir: str, manifest: Mapping[str, TensorNeed], engine_dtype: torch.dtype
                    ) -> Dict[str, torch.Tensor]:
    try:
        entries = index_model_dir(model_dir)
    except SafetensorsError as e:
        raise WeightsError(str(e), [], [], []) from None
    pairs, missing, unexpected = match_names(manifest, entries)
    wrong_shape, wrong_type = [], []
    for want, have in pairs.items():
        need, ent = manifest[want], entries[have]
        if tuple(need.shape) != tuple(ent.shape):
            wrong_shape.append((want, ent.shape, need.shape))
        if need.role == "int_table":
            if ent.dtype not in _INT_TAGS:
                wrong_type.append((want, f"file {ent.dtype}, model wants an integer table"))
        elif ent.dtype not in _FLOAT_TAGS:
            wrong_type.append((want, f"file {ent.dtype}, model wants floating point"))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightsError(model_dir, missing, unexpected, wrong_shape, wrong_type)
    reader = TensorFileReader()
    out = {}
    for want, have in pairs.items():
        ent = entries[have]
        out[want] = to_torch(reader.array(ent), ent.dtype, engine_dtype, manifest[want].role)
    reader.close()
    return out
