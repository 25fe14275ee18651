"""Reading and writing the safetensors container, nothing else.

Layout (as the reference's private helper parses it, src/gguf.rs:207-229): an 8-byte
little-endian header length N, N bytes of JSON mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the first
byte after the header; ``__metadata__`` is skipped), then the raw little-endian data.
A sharded model has ``model.safetensors.index.json`` whose ``weight_map`` names the
file of each tensor.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import numpy as np

# safetensors dtype tag → (numpy dtype used to view the bytes, bytes per element)
_DTYPES = {
    "F32": (np.dtype("<f4"), 4),
    "F16": (np.dtype("<f2"), 2),
    "BF16": (np.dtype("<u2"), 2),   # viewed as raw 16-bit patterns
    "F64": (np.dtype("<f8"), 8),
    "I64": (np.dtype("<i8"), 8),
    "I32": (np.dtype("<i4"), 4),
    "I16": (np.dtype("<i2"), 2),
    "I8": (np.dtype("i1"), 1),
    "U8": (np.dtype("u1"), 1),
    "BOOL": (np.dtype("u1"), 1),
}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str               # safetensors tag, e.g. "BF16"
    shape: Tuple[int, ...]
    file: str
    begin: int               # absolute byte offset in ``file``
    end: int

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


def read_header(path: str) -> Dict[str, TensorEntry]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: file is shorter than the 8-byte header length")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        raw = f.read(n)
    try:
        hdr = json.loads(raw.decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
    if not isinstance(hdr, dict):
        raise SafetensorsError(f"{path}: header must be a JSON object")
    base = 8 + n
    out: Dict[str, TensorEntry] = {}
    for name, info in hdr.items():
        if name == "__metadata__":
            continue
        try:
            tag = info["dtype"]
            shape = tuple(int(s) for s in info["shape"])
            b, e = (int(x) for x in info["data_offsets"])
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: malformed header entry for tensor '{name}'") from None
        if tag not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {tag}")
        ent = TensorEntry(name, tag, shape, path, base + b, base + e)
        if b > e or base + e > size:
            raise SafetensorsError(f"{path}: tensor '{name}' data [{b}, {e}) lies outside the file")
        if e - b != ent.numel * _DTYPES[tag][1]:
            raise SafetensorsError(f"{path}: tensor '{name}' has {e - b} bytes but shape {list(shape)} of {tag} "
                                   f"needs {ent.numel * _DTYPES[tag][1]}")
        out[name] = ent
    return out


def index_model_dir(model_dir: str) -> Dict[str, TensorEntry]:
    """All tensors of a model folder (single file or shards named by the index file)."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return read_header(single)
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            try:
                wm = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise SafetensorsError(f"{index}: no readable 'weight_map'") from None
        entries: Dict[str, TensorEntry] = {}
        for shard in sorted(set(wm.values())):
            sp = os.path.join(model_dir, shard)
            if not os.path.isfile(sp):
                raise SafetensorsError(f"{index}: names shard '{shard}', which is missing")
            entries.update(read_header(sp))
        return entries
    raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")


class TensorFileReader:
    """Memory-maps the files of a set of entries and hands out numpy views."""

    def __init__(self):
        self._maps: Dict[str, mmap.mmap] = {}
        self._files = {}

    def array(self, e: TensorEntry) -> np.ndarray:
        m = self._maps.get(e.file)
        if m is None:
            f = open(e.file, "rb")
            m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._files[e.file] = f
            self._maps[e.file] = m
        npdt, _ = _DTYPES[e.dtype]
        return np.frombuffer(m, dtype=npdt, count=e.numel, offset=e.begin).reshape(e.shape)

    def close(self):
        # numpy views keep the maps alive; dropping our references is enough
        self._maps.clear()
        for f in self._files.values():
            f.close()
        self._files.clear()


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 → bfloat16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (r >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


class SafetensorsWriter:
    """Streams tensors into one safetensors file: declare all, then write each in order."""

    def __init__(self, path: str, layout: List[Tuple[str, str, Tuple[int, ...]]], metadata: Mapping[str, str] = None):
        self.path = path
        hdr = {}
        off = 0
        self._order = []
        for name, tag, shape in layout:
            n = 1
            for s in shape:
                n *= s
            nbytes = n * _DTYPES[tag][1]
            hdr[name] = {"dtype": tag, "shape": list(shape), "data_offsets": [off, off + nbytes]}
            self._order.append((name, tag, tuple(shape), nbytes))
            off += nbytes
        if metadata:
            hdr["__metadata__"] = dict(metadata)
        raw = json.dumps(hdr, separators=(",", ":")).encode("utf-8")
        raw += b" " * ((8 - len(raw) % 8) % 8)
        self._f = open(path, "wb")
        self._f.write(struct.pack("<Q", len(raw)))
        self._f.write(raw)
        self._next = 0

    def write(self, name: str, data: np.ndarray) -> None:
        want, tag, shape, nbytes = self._order[self._next]
        if name != want:
            raise SafetensorsError(f"writer expects tensor '{want}' next, got '{name}'")
        buf = np.ascontiguousarray(data)
        if buf.nbytes != nbytes:
            raise SafetensorsError(f"tensor '{name}': {buf.nbytes} bytes given, {nbytes} declared")
        self._f.write(buf.tobytes() if buf.nbytes < (1 << 20) else memoryview(buf).cast("B"))
        self._next += 1

    def close(self):
        if self._next != len(self._order):
            raise SafetensorsError(f"{self.path}: {len(self._order) - self._next} declared tensors were not written")
        self._f.close()
