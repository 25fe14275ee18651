"""Device storage behind the cache manager's page numbers and state slots.

One tensor per cache group, [calls in the group, pages, 2 (K, V), kv heads, page_size,
head_dim] in the engine's element type, so a (page, K|V, kv head) tile is one
contiguous [page_size, head_dim] block; one [max_seqs, numel] array per mixer call
that keeps per-request state, in the element type the mixer asked for.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..dtypes import element_type
from ..parts.spec import CacheNeed, StateNeed


def allocate_caches(groups: Sequence[CacheNeed], group_calls: Sequence[Sequence[int]], num_pages: int, page_size: int,
                    dtype: torch.dtype, device) -> List[torch.Tensor]:
    out = []
    for need, calls in zip(groups, group_calls):
        out.append(torch.zeros((len(calls), num_pages, 2, need.n_kv_heads, page_size, need.head_dim), dtype=dtype,
                               device=device))
    return out


def allocate_states(needs: Dict, max_seqs: int, device) -> Dict:
    """needs: key (call index, mixer role) → StateNeed; returns the same keys → [max_seqs, numel] zeros."""
    return {k: torch.zeros((max_seqs, n.numel), dtype=element_type(n.dtype).torch, device=device)
            for k, n in needs.items()}


def cache_bytes_per_token(groups: Sequence[CacheNeed], group_calls: Sequence[Sequence[int]], dtype: torch.dtype) -> int:
    es = element_type(dtype).itemsize
    return sum(2 * n.n_kv_heads * n.head_dim * es * len(c) for n, c in zip(groups, group_calls))
