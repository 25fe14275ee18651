"""The generic decoder: embedding → layers in the run order → final norm → head.

Built from a :class:`~rustingstrata_b200.parts.spec.ModelSpec` by instantiating the
registered part classes; it contains no architecture-specific code.  The reference's
counterpart is ``GpuModel`` with its per-architecture branches (load
src/gpu_model.rs:656-1133, layer loop :1950-2016, batch step
src/gpu_model/prefill.rs:781-845).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from ..parts import (CallInfo, CacheNeed, HostBatch, LayerCall, ModelSpec, Runtime, StateNeed, StepContext, TensorNeed,
                     part_class)


class CausalLM:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        mk = lambda cat, ps, *a, **k: part_class(cat, ps.kind)(ps, runtime, *a, **k)  # noqa: E731
        self.embedding = mk("embedding", spec.embedding)
        self.blocks = []
        for ls in spec.layers:
            pos = mk("position", ls.position) if ls.position is not None else None
            mixer = mk("mixer", ls.mixer, position=pos) if pos is not None else mk("mixer", ls.mixer)
            block = mk("block", ls.block, mk("norm", ls.mixer_norm), mixer, mk("norm", ls.feed_forward_norm),
                       mk("feed_forward", ls.feed_forward))
            self.blocks.append(block)
        self.final_norm = mk("norm", spec.final_norm)
        self.head = mk("head", spec.head)
        runtime.scratch("residual", runtime.max_batch_tokens, spec.hidden_size, torch.float32)
        runtime.scratch("head_in", runtime.max_logit_rows, spec.hidden_size)
        runtime.scratch("logits", runtime.max_logit_rows, spec.vocab_size, torch.float32)

        # ---- the run order: which cache and state each call uses
        if not spec.order:
            raise ValueError("model spec has an empty run order")
        self.calls: List[CallInfo] = []
        self.cache_groups: List[CacheNeed] = []        # distinct needs, in order of first use
        self.group_calls: List[List[int]] = []         # per group: the calls that own a cache in it
        self.state_needs: Dict[int, StateNeed] = {}    # call index → state need
        self._cache_slot: Dict[int, Tuple[int, int]] = {}   # owning call → (group, index within group)
        for i, lc in enumerate(spec.order):
            if not 0 <= lc.layer < len(self.blocks):
                raise ValueError(f"run order entry {i} names layer {lc.layer}, but the model has {len(self.blocks)}")
            mixer = self.blocks[lc.layer].mixer
            need = mixer.cache_need()
            info = CallInfo(index=i, layer=lc.layer)
            if need is not None:
                if lc.cache is None:
                    if need not in self.cache_groups:
                        self.cache_groups.append(need)
                        self.group_calls.append([])
                    g = self.cache_groups.index(need)
                    self._cache_slot[i] = (g, len(self.group_calls[g]))
                    self.group_calls[g].append(i)
                    info.cache_group, info.writes_cache = g, True
                else:
                    if not 0 <= lc.cache < i or lc.cache not in self._cache_slot:
                        raise ValueError(f"run order entry {i} reads the cache of entry {lc.cache}, which is not an "
                                         f"earlier entry that owns a cache")
                    owner_need = self.cache_groups[self._cache_slot[lc.cache][0]]
                    if (owner_need.n_kv_heads, owner_need.head_dim) != (need.n_kv_heads, need.head_dim):
                        raise ValueError(f"run order entry {i} cannot read the cache of entry {lc.cache}: "
                                         f"key/value shapes differ")
                    self._cache_slot[i] = self._cache_slot[lc.cache]
                    info.cache_group, info.writes_cache = self._cache_slot[lc.cache][0], False
            elif lc.cache is not None:
                raise ValueError(f"run order entry {i} names a cache but its mixer keeps none")
            sn = mixer.state_need()
            if sn is not None:
                self.state_needs[i] = sn
            self.calls.append(info)

    # ---------------------------------------------------------------- weights
    def parts(self):
        yield self.embedding
        for b in self.blocks:
            yield from (b, b.mixer_norm, b.mixer, b.ff_norm, b.feed_forward)
            if getattr(b.mixer, "position", None) is not None:
                yield b.mixer.position
        yield self.final_norm
        yield self.head

    @property
    def capturable(self) -> bool:
        """Whether a step of this model may be replayed from a CUDA graph (every part allows it)."""
        return all(p.capturable for p in self.parts())

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        needs: Dict[str, TensorNeed] = {}
        for p in self.parts():
            for name, need in p.tensor_needs().items():
                if name in needs and tuple(needs[name].shape) != tuple(need.shape):
                    raise ValueError(f"tensor '{name}' is wanted with shapes {needs[name].shape} and {need.shape}")
                needs.setdefault(name, need)
        return needs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.load(tensors)

    # ---------------------------------------------------------------- storage binding
    def bind_storage(self, caches: List[torch.Tensor], states: Dict[int, torch.Tensor]) -> None:
        """caches[g]: [calls in group g, pages, 2, n_kv, page_size, head_dim]; states[call]: [max_seqs, numel]."""
        for i, info in enumerate(self.calls):
            if i in self._cache_slot:
                g, j = self._cache_slot[i]
                info.cache = caches[g][j]
            info.state = states.get(i)

    # ---------------------------------------------------------------- one step
    def plan(self, batch: HostBatch) -> Dict:
        plans = {}
        for p in self.parts():
            key = p.plan_key()
            if key is not None and key not in plans:
                plans[key] = p.build_plan(batch)
        return plans

    def forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """Runs the step's tokens and returns float32 logits [n_logit_rows, vocab] (None if none are wanted)."""
        rt = self.runtime
        residual = rt.get_scratch("residual", torch.float32)[:, : self.spec.hidden_size]
        self.embedding.forward(ctx, residual)
        for k, info in enumerate(self.calls):
            # a block's last product may leave its final sum to the next block's first norm, if that norm can take it
            ctx.next_block_takes_owed = (k + 1 < len(self.calls)
                                         and self.blocks[self.calls[k + 1].layer].first_reader_takes_owed)
            self.blocks[info.layer].forward(residual, ctx, info)
        if ctx.owed is not None:
            ctx.owed.finish()
            ctx.owed = None
        if ctx.n_logit_rows == 0:
            return None
        R = ctx.n_logit_rows
        head_in = rt.get_scratch("head_in")[:, : self.spec.hidden_size]
        logits = rt.get_scratch("logits", torch.float32)[:, : self.spec.vocab_size]
        self.final_norm.forward(residual, head_in, R, rows=ctx.logit_rows)
        self.head.forward(head_in, logits, R, status=ctx.status)
        return logits[:R]
