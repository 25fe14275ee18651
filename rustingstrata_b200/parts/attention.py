"""Attention mixer over a paged key/value cache.

Reference (src/model.rs:747-801; device decode path src/gpu_model.rs:3181-3277, batch
path src/gpu_model/prefill.rs:811-828): q/k/v projections without biases, optional
per-head RMSNorm on q and k with one weight shared by all heads, rotation, the new k
and v stored at the token's position before any query of the step reads the cache,
query head i reading kv head i // (n_heads / n_kv_heads), score scale 1/sqrt(head_dim),
causal over all keys or over the most recent ``window`` keys, output projection added
to the residual stream.

Everything that distinguishes one architecture's attention from another's is a
parameter: head counts, head size, whether q/k are normed and with which eps, the
window, the score scale, which position encoding is applied, and whether this call
projects keys and values at all (a call that reads another call's cache does not).
A position encoding reaches the attention in one of two ways, or both: a rotation of
q and k (its ``cos_sin`` table, ``n_rot`` and ``stream``) applied before the cache
write, and a bias on the scores that is linear in the distance between query and key
(its ``score_slopes``, one per head), which the CUDA-core attention kernels add.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..kernels import ops
from .base import CallInfo, HostBatch, Mixer, StepContext
from .registry import register_part
from .spec import CacheNeed, TensorNeed

SPLIT_KEYS = 128     # keys per split of the decode form; fixed so a position's reduction order never changes
SPLIT_BUCKET = 8     # captured steps round the number of splits launched up to a multiple of this


def decode_splits(kv_len: np.ndarray, window: int) -> np.ndarray:
    """How many SPLIT_KEYS-aligned splits hold the visible keys of a single query at position kv_len-1."""
    lo = np.maximum(0, kv_len - window) if window > 0 else np.zeros_like(kv_len)
    return (kv_len + SPLIT_KEYS - 1) // SPLIT_KEYS - lo // SPLIT_KEYS


@register_part("mixer", "paged_attention")
class PagedAttention(Mixer):
    """params: hidden, n_heads, n_kv_heads, head_dim, qk_norm (bool), eps, window (int or None),
    scale (float or None = 1/sqrt(head_dim)), kv_projection (bool, default True).
    tensors: q_proj, k_proj, v_proj, o_proj, and q_norm, k_norm when qk_norm."""
    chain_safe = True

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.hd = int(p["head_dim"])
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("eps", 0.0))
        self.window = int(p["window"]) if p.get("window") else 0
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.kv_projection = bool(p.get("kv_projection", True))
        self.position = position
        if self.n_heads % self.n_kv:
            raise ValueError(f"paged_attention: {self.n_heads} heads are not a multiple of {self.n_kv} kv heads")
        if self.hd % 16 or not 16 <= self.hd <= 256:
            raise ValueError(f"paged_attention: head size {self.hd} is not supported by the attention kernels "
                             f"(multiples of 16 from 16 to 256)")
        self.q_width = self.n_heads * self.hd
        self.kv_width = self.n_kv * self.hd
        self.qkv_width = self.q_width + (2 * self.kv_width if self.kv_projection else 0)
        self.q_per_cta = None
        rt = runtime
        rt.scratch("qkv", rt.max_batch_tokens, self.q_width + 2 * self.kv_width)
        rt.scratch("attn_out", rt.max_batch_tokens, self.q_width)
        # Partial results of the split form: one slot per (sequence, split).  The keys a step can see lie in the
        # pool, so whole splits number at most pool_tokens / SPLIT_KEYS in all; beside them every sequence may have
        # a partly filled split at either end of what it sees (the newest keys; the oldest ones inside a window).
        self.partial_slots = rt.pool_tokens // SPLIT_KEYS + 2 * rt.max_seqs + 1
        rt.scratch("attn_partial", 1, self.partial_slots * self.n_heads * (self.hd + 2), torch.float32)
        # The step's list of (sequence, kv head, split) items of the tensor-core decode kernel.  The first layer of a
        # step that needs it writes it and the later ones read it, so it has a name that only layers with the same
        # plan (the plan's key follows from window and head shape) share: nobody else may write it in between.
        self.items_name = f"attn_items_w{self.window}_h{self.n_heads}x{self.n_kv}x{self.hd}"
        rt.scratch(self.items_name, 1, self.partial_slots * self.n_kv, torch.int32)
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    # ---------------------------------------------------------------- weights
    def tensor_needs(self):
        t = self.spec.tensors
        needs = {t["q_proj"]: TensorNeed((self.q_width, self.hidden)),
                 t["o_proj"]: TensorNeed((self.hidden, self.q_width))}
        if self.kv_projection:
            needs[t["k_proj"]] = TensorNeed((self.kv_width, self.hidden))
            needs[t["v_proj"]] = TensorNeed((self.kv_width, self.hidden))
        if self.qk_norm:
            needs[t["q_norm"]] = TensorNeed((self.hd,), "norm")
            if self.kv_projection:
                needs[t["k_norm"]] = TensorNeed((self.hd,), "norm")
        return needs

    def load(self, tensors):
        t = self.spec.tensors
        mats = [tensors[t["q_proj"]]]
        if self.kv_projection:
            mats += [tensors[t["k_proj"]], tensors[t["v_proj"]]]
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("paged_attention: q, k and v projections must share an element type")
        # one [q | k | v] matrix so the three projections are one product (the reference runs
        # q+k as one launch and v beside it, src/gpu_model.rs:3190)
        self.w_qkv = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0].contiguous()
        self.w_o = tensors[t["o_proj"]].contiguous()
        if self.qk_norm:
            self.q_norm_w = tensors[t["q_norm"]].contiguous()
            self.k_norm_w = tensors[t["k_norm"]].contiguous() if self.kv_projection else None

    # ---------------------------------------------------------------- state
    def cache_need(self):
        return CacheNeed(self.n_kv, self.hd, self.window or None)

    def mixing_flops(self, q_lens, kv_lens) -> float:
        """Flops of scores and weighted sums for sequences that add q_lens[i] queries and then hold kv_lens[i] keys:
        4 * heads * head size per (query, visible key) pair."""
        pairs = 0.0
        for q, kv in zip(np.asarray(q_lens, dtype=np.int64), np.asarray(kv_lens, dtype=np.int64)):
            pos = np.arange(kv - q, kv, dtype=np.float64)                  # query positions; each sees pos + 1 keys
            seen = pos + 1 if not self.window else np.minimum(pos + 1, self.window)
            pairs += float(seen.sum())
        return 4.0 * self.n_heads * self.hd * pairs

    # ---------------------------------------------------------------- planning
    def _score_slopes(self):
        """The position encoding's bias on the scores, if it has one: float32 [n_heads], slope of head h times (key
        position - query position) added to every scaled score.  The CUDA-core attention kernels take it."""
        return getattr(self.position, "score_slopes", None) if self.position is not None else None

    def plan_key(self):
        if self.q_per_cta is None:
            force = "simt" if self._score_slopes() is not None else ""
            self.q_per_cta = ops.attention_prefill_q_per_cta(self.runtime.dtype, self.n_heads, self.n_kv, self.hd,
                                                              self.runtime.page_size, force)
        return ("paged_attention", self.q_per_cta, self.window)

    def build_plan(self, batch: HostBatch):
        """Work lists: sequences with one query take the split (decode) form, the rest are cut into query tiles."""
        qpc = self.q_per_cta
        single = batch.q_lens == 1
        dec = np.nonzero(single)[0].astype(np.int32)
        splits = decode_splits(batch.kv_lens[dec], self.window).astype(np.int32) if len(dec) else np.zeros(0, np.int32)
        split_start = np.zeros(len(dec) + 1, np.int32)
        np.cumsum(splits, out=split_start[1:])
        tiles = []
        for s in np.nonzero(~single)[0]:
            offs = np.arange(0, batch.q_lens[s], qpc, dtype=np.int32)
            tiles.append(np.stack([np.full_like(offs, s), offs], axis=1))
        pre = np.concatenate(tiles, axis=0).astype(np.int32) if tiles else np.zeros((0, 2), np.int32)
        if len(pre) > 1:
            # tiles with the most keys to walk first: the last wave of CTAs then holds the short ones
            last_pos = batch.kv_lens[pre[:, 0]] - batch.q_lens[pre[:, 0]] + pre[:, 1]
            pre = pre[np.argsort(-last_pos, kind="stable")]
        max_splits = int(splits.max()) if len(dec) else 0
        total_splits = int(split_start[-1])
        if total_splits > self.partial_slots:
            raise ValueError(f"paged_attention: the step's single-token sequences span {total_splits} splits of "
                             f"{SPLIT_KEYS} keys, the workspace was sized for {self.partial_slots} (more keys than "
                             f"the cache pool holds?)")
        if batch.bucketed and len(dec):
            # A captured step: the number of splits launched per sequence is a launch shape, so it is rounded up (a
            # split beyond a sequence's own count exits at once).  The slots really used change from replay to
            # replay and always fit (checked above, every step); the launcher is told nothing about them (0), so
            # that the captured layout does not depend on the lengths.
            max_splits = (max_splits + SPLIT_BUCKET - 1) // SPLIT_BUCKET * SPLIT_BUCKET
            total_splits = 0
        return {"decode_work": dec, "split_start": split_start, "prefill_work": pre.reshape(-1),
                "n_decode": int(len(dec)), "n_prefill": int(pre.shape[0]),
                "max_splits": max_splits, "total_splits": total_splits}

    # ---------------------------------------------------------------- the step
    def forward(self, h, residual, ctx: StepContext, call: CallInfo):
        rt = self.runtime
        T = ctx.n_tokens
        write_kv = call.writes_cache
        if write_kv and not self.kv_projection:
            raise RuntimeError("paged_attention: a call without key/value projections must read another call's cache")
        width = self.qkv_width if write_kv else self.q_width
        qkv = rt.get_scratch("qkv")[:, :width]
        w = self.w_qkv if write_kv else self.w_qkv[: self.q_width]
        ops.linear(h, w, qkv, T, status=ctx.status)
        table = ctx.block_tables[call.cache_group]
        pos = self.position
        rot = getattr(pos, "cos_sin", None) if pos is not None else None
        ops.qk_norm_rope_kv(qkv, T, self.n_heads, self.n_kv, self.hd, self.q_norm_w, self.k_norm_w, self.eps,
                            rot, pos.n_rot if rot is not None else 0,
                            ctx.positions, ctx.seq_of_token, table, rt.page_size, call.cache, write_kv, ctx.status,
                            stream=pos.stream if pos is not None else 0)
        out = rt.get_scratch("attn_out")[:, : self.q_width]
        plan = ctx.plans[self.plan_key()]
        common = dict(q=qkv, out=out, cache=call.cache, block_table=table, q_start=ctx.q_start, kv_len=ctx.kv_len,
                      n_q=self.n_heads, n_kv=self.n_kv, head_dim=self.hd, page_size=rt.page_size, window=self.window,
                      scale=self.scale, status=ctx.status)
        slopes = self._score_slopes()
        if plan["n_prefill"]:
            ops.attention_prefill(work=plan["prefill_work"], n_work=plan["n_prefill"], slopes=slopes,
                                  force="simt" if slopes is not None else "", **common)
        if plan["n_decode"]:
            items = None
            if slopes is None and ops.attention_decode_fast_ok(rt.dtype, self.n_heads, self.n_kv, self.hd, rt.page_size):
                # built by the first layer of the step that needs it; the plan (and the list) is the step's, not the layer's
                items = rt.get_scratch(self.items_name, torch.int32).view(-1)
                if ("items", self.n_kv) not in plan:
                    ops.attention_decode_items(plan["split_start"], plan["n_decode"], self.n_kv, plan["max_splits"], items)
                    plan[("items", self.n_kv)] = True
            ops.attention_decode(work=plan["decode_work"], n_work=plan["n_decode"], split_keys=SPLIT_KEYS,
                                 max_splits=plan["max_splits"], split_start=plan["split_start"],
                                 total_splits=plan["total_splits"], slopes=slopes, items=items,
                                 partial=rt.get_scratch("attn_partial", torch.float32), **common)
        ctx.owed = ops.linear(out, self.w_o, residual, T, accumulate=True, status=ctx.status, may_defer=ctx.may_owe)
