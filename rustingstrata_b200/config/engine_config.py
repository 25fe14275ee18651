"""Engine options: everything about the run that is not the model.

The reference spreads these over command-line flags (``--ctx``, ``--chunk``,
``--parallel``: src/main.rs:28-35,216) and environment knobs.  Here they are one typed
record; nothing in the hot path reads the environment.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..dtypes import ENGINE_DTYPES, engine_dtype_name

DTYPES = ENGINE_DTYPES


@dataclass(frozen=True)
class EngineConfig:
    dtype: str = "bfloat16"          # "bfloat16": serving kernels; "float32": true 32-bit everywhere
    page_size: int = 16              # tokens per cache page
    num_pages: int = 0               # pages per cache group pool; 0 = derive from max_tokens
    max_tokens: int = 4096           # tokens the pool must hold when num_pages is 0 (rounded up to pages)
    max_seqs: int = 64               # live requests (also the number of state slots)
    max_batch_tokens: int = 2048     # tokens in one step
    max_logit_rows: int = 256        # rows of logits one step may return
    device: str = "cuda:0"

    def __post_init__(self):
        object.__setattr__(self, "dtype", engine_dtype_name(self.dtype))      # "bf16" and "fp32" are accepted
        if self.page_size <= 0:
            raise ValueError("page_size must be positive")
        for k in ("max_seqs", "max_batch_tokens", "max_logit_rows"):
            if getattr(self, k) <= 0:
                raise ValueError(f"{k} must be positive")

    def pool_pages(self) -> int:
        if self.num_pages > 0:
            return self.num_pages
        return (self.max_tokens + self.page_size - 1) // self.page_size
