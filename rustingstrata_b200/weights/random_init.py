"""Random-weights mode: one generator, on the host and on the device, for a model drawn from a seed.

The reference only has test helpers that fill tiny models from an integer hash of the
element index with norm weights 1.0 (src/model.rs:1448-1461).  Here every element of
every tensor of the model's manifest is a pure function of (seed, tensor name, element
index), so a tensor's values do not depend on which other tensors exist, in which
order they are drawn, how the work is cut, or where it is computed:

    key   = mix64(seed ^ mix64(fnv1a64(name)))
    z     = mix64(key + (index + 1) * 0x9E3779B97F4A7C15)        (a counter run through a 64-bit finaliser)
    value = shift + scale * NORMAL[z >> 48]                      (two float32 operations)

``NORMAL`` is a table of the 65,536 mid-point quantiles of the standard normal
distribution, rounded to float32; the draw is a look-up, so the host (numpy, this
file) and the device (``rs_fill_random`` in csrc/elementwise.cu, given the same table)
produce the same bits.  Projections and the token table are N(0, std) (scale = std,
shift = 0), norm scales 1 + N(0, norm_std) (shift = 1), integer tables the low bit of
z.  ``write_random_model`` writes a model folder with these values; the engine's
``from_random`` draws the same values straight into device memory.
"""
from __future__ import annotations

import json
import os
import statistics
from typing import Iterator, Mapping, Tuple

import numpy as np

from ..parts.spec import TensorNeed
from .safetensors_io import SafetensorsWriter, f32_to_bf16_bits

_CHUNK = 1 << 22
_M64 = 0xFFFFFFFFFFFFFFFF
GOLDEN = 0x9E3779B97F4A7C15
_C1, _C2 = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
TABLE_BITS = 16


def mix64(x: int) -> int:
    """The 64-bit finaliser both sides use (xor-shift, multiply, twice, xor-shift)."""
    x &= _M64
    x = ((x ^ (x >> 30)) * _C1) & _M64
    x = ((x ^ (x >> 27)) * _C2) & _M64
    return x ^ (x >> 31)


def fnv1a64(text: str) -> int:
    h = 0xCBF29CE484222325
    for b in text.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & _M64
    return h


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of one tensor's stream."""
    return mix64((seed & _M64) ^ mix64(fnv1a64(name)))


_TABLE = None


def normal_table() -> np.ndarray:
    """float32[65536]: the standard normal quantile at (k + 0.5) / 65536 (largest |value| about 4.2)."""
    global _TABLE
    if _TABLE is None:
        inv = statistics.NormalDist().inv_cdf
        n = 1 << TABLE_BITS
        half = [inv((k + 0.5) / n) for k in range(n // 2)]                  # the lower half; the upper mirrors it exactly
        t = np.array(half + [-v for v in reversed(half)], dtype=np.float64).astype(np.float32)
        t.setflags(write=False)
        _TABLE = t
    return _TABLE


def scale_shift(need: TensorNeed, std: float, norm_std: float) -> Tuple[float, float]:
    """(scale, shift) of value = shift + scale * normal for a tensor of this role."""
    if need.role == "norm":
        return float(norm_std), 1.0
    return float(std), 0.0


def draw_bits(key: int, start: int, count: int) -> np.ndarray:
    """z of elements start .. start + count - 1 as uint64."""
    x = np.arange(start + 1, start + count + 1, dtype=np.uint64)
    t = np.empty_like(x)
    with np.errstate(over="ignore"):                       # arithmetic modulo 2^64, in place
        x *= np.uint64(GOLDEN)
        x += np.uint64(key)
        for shift, mul in ((30, _C1), (27, _C2)):
            np.right_shift(x, np.uint64(shift), out=t)
            x ^= t
            x *= np.uint64(mul)
        np.right_shift(x, np.uint64(31), out=t)
        x ^= t
    return x


def draw_values(seed: int, name: str, need: TensorNeed, std: float, norm_std: float, start: int = 0,
                count: int = -1) -> np.ndarray:
    """Elements start .. start + count - 1 of the flattened tensor: float32, or int32 for an integer table."""
    n = int(np.prod(need.shape, dtype=np.int64)) if len(need.shape) else 1
    count = n - start if count < 0 else count
    z = draw_bits(tensor_key(seed, name), start, count)
    if need.role == "int_table":
        return (z & np.uint64(1)).astype(np.int32)
    scale, shift = scale_shift(need, std, norm_std)
    z >>= np.uint64(64 - TABLE_BITS)
    v = normal_table()[z.view(np.int64)]
    v *= np.float32(scale)                                      # float32 multiply, then float32 add
    v += np.float32(shift)
    return v


def draw_tensor(seed: int, name: str, need: TensorNeed, std: float, norm_std: float) -> Iterator[np.ndarray]:
    """Yields the tensor's values as flat chunks."""
    n = int(np.prod(need.shape, dtype=np.int64)) if len(need.shape) else 1
    for done in range(0, n, _CHUNK):
        yield draw_values(seed, name, need, std, norm_std, done, min(_CHUNK, n - done))


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
