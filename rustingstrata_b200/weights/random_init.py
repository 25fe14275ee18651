"""Random-weights mode: a model folder drawn from a configuration and a seed.

The reference only has test helpers that fill tiny models from an integer hash with
norm weights 1.0 (src/model.rs:1448-1461).  Here every tensor of the model's manifest
is drawn from a counter-based generator keyed by (seed, tensor name), so a tensor's
values do not depend on which other tensors exist or in which order they are written:
projections and the token table N(0, std), norm scales 1.0 or 1 + N(0, norm_std).
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Mapping

import numpy as np

from ..parts.spec import TensorNeed
from .safetensors_io import SafetensorsWriter, f32_to_bf16_bits

_CHUNK = 1 << 24


def _generator(seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed & 0xFFFFFFFFFFFFFFFF, zlib.crc32(name.encode("utf-8"))]))


def draw_tensor(seed: int, name: str, need: TensorNeed, std: float, norm_std: float):
    """Yields the tensor's values as flat float32 chunks (int32 for integer tables)."""
    n = 1
    for s in need.shape:
        n *= s
    g = _generator(seed, name)
    done = 0
    while done < n:
        m = min(_CHUNK, n - done)
        if need.role == "norm":
            a = np.ones(m, dtype=np.float32)
            if norm_std > 0:
                a += g.standard_normal(m, dtype=np.float32) * np.float32(norm_std)
        elif need.role == "int_table":
            a = g.integers(0, 2, size=m, dtype=np.int32)
        else:
            a = g.standard_normal(m, dtype=np.float32) * np.float32(std)
        yield a
        done += m


def write_random_model(model_dir: str, config_dict: Mapping, manifest: Mapping[str, TensorNeed], seed: int,
                       std: float = 0.02, norm_std: float = 0.0, store_dtype: str = "bfloat16",
                       progress=None) -> None:
    """Writes ``config.json`` and ``model.safetensors`` under ``model_dir``.

    ``store_dtype`` "bfloat16" stores floating tensors as BF16 (values rounded to
    nearest even, so a 32-bit run of the same folder sees exactly the same numbers);
    "float32" stores them as F32.
    """
    if store_dtype not in ("bfloat16", "float32"):
        raise ValueError(f"store_dtype must be 'bfloat16' or 'float32', got {store_dtype!r}")
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(config_dict), f, indent=2)
        f.write("\n")
    tag = "BF16" if store_dtype == "bfloat16" else "F32"
    layout = [(name, "I32" if need.role == "int_table" else tag, tuple(need.shape)) for name, need in manifest.items()]
    w = SafetensorsWriter(os.path.join(model_dir, "model.safetensors"), layout,
                          metadata={"format": "pt", "seed": str(seed)})
    for i, (name, need) in enumerate(manifest.items()):
        parts = []
        for chunk in draw_tensor(seed, name, need, std, norm_std):
            if need.role == "int_table":
                parts.append(chunk)
            elif tag == "BF16":
                parts.append(f32_to_bf16_bits(chunk))
            else:
                parts.append(chunk)
        w.write(name, parts[0] if len(parts) == 1 else np.concatenate(parts))
        if progress is not None:
            progress(i + 1, len(manifest), name)
    w.close()
