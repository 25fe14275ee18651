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

from ..parts import (CallInfo, CacheNeed, HostBatch, LayerCall, LayerCallInfo, ModelSpec, Runtime, StateNeed, StepContext,
                     TensorNeed, part_class)


class CausalLM:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        mk = lambda cat, ps, *a, **k: part_class(cat, ps.kind)(ps, runtime, *a, **k)  # noqa: E731
        self.embedding = mk("embedding", spec.embedding)
        self.blocks = []
        for li, ls in enumerate(spec.layers):
            block_cls = part_class("block", ls.block.kind)
            try:
                block_cls.check_roles(ls.parts)
            except ValueError as e:
                raise ValueError(f"layer {li}: {e}") from None
            cat = {role: block_cls.category_of(role) for role in ls.parts}
            # position encodings first: a mixer is built with the one that belongs to it
            built = {role: mk("position", ps) for role, ps in ls.parts.items() if cat[role] == "position"}
            for role, ps in ls.parts.items():
                if cat[role] == "mixer":
                    pos = built.get(role + "_position", built.get("position"))
                    built[role] = mk("mixer", ps, position=pos) if pos is not None else mk("mixer", ps)
                elif cat[role] != "position":
                    built[role] = mk(cat[role], ps)
            self.blocks.append(block_cls(ls.block, runtime, built))
        self.final_norm = mk("norm", spec.final_norm)
        self.head = mk("head", spec.head)
        runtime.scratch("residual", runtime.max_batch_tokens, spec.hidden_size, torch.float32)
        runtime.scratch("head_in", runtime.max_logit_rows, spec.hidden_size)
        runtime.scratch("logits", runtime.max_logit_rows, spec.vocab_size, torch.float32)
        # position values a step carries per token: the most any position encoding of the model asks for
        self.n_position_streams = max([1] + [int(getattr(p, "n_streams", 1)) for p in self.parts()
                                             if p.category == "position"])

        # ---- the run order: which cache and state each mixer of each call uses
        if not spec.order:
            raise ValueError("model spec has an empty run order")
        self.calls: List[LayerCallInfo] = []
        self.cache_groups: List[CacheNeed] = []        # distinct needs, in order of first use
        self.group_calls: List[List[Tuple[int, str]]] = []     # per group: the (call, mixer role) that own a cache in it
        self.state_needs: Dict[Tuple[int, str], StateNeed] = {}     # (call index, mixer role) → state need
        self._cache_slot: Dict[Tuple[int, str], Tuple[int, int]] = {}   # (call, role) → (group, index within group)
        for i, lc in enumerate(spec.order):
            if not 0 <= lc.layer < len(self.blocks):
                raise ValueError(f"run order entry {i} names layer {lc.layer}, but the model has {len(self.blocks)}")
            mixers = self.blocks[lc.layer].mixers()
            if isinstance(lc.cache, Mapping):
                borrow = dict(lc.cache)
                unknown = [r for r in borrow if r not in mixers]
                if unknown:
                    raise ValueError(f"run order entry {i} names a cache for {unknown}, which are no mixers of its layer")
            else:
                borrow = {r: lc.cache for r in mixers} if lc.cache is not None else {}
            entry = LayerCallInfo(index=i, layer=lc.layer)
            any_cache = False
            for role, mixer in mixers.items():
                need = mixer.cache_need()
                info = CallInfo(index=i, layer=lc.layer, role=role)
                src = borrow.get(role)
                if need is not None:
                    any_cache = True
                    if src is None:
                        if need not in self.cache_groups:
                            self.cache_groups.append(need)
                            self.group_calls.append([])
                        g = self.cache_groups.index(need)
                        self._cache_slot[(i, role)] = (g, len(self.group_calls[g]))
                        self.group_calls[g].append((i, role))
                        info.cache_group, info.writes_cache = g, True
                    else:
                        if not 0 <= src < i or (src, role) not in self._cache_slot:
                            raise ValueError(f"run order entry {i} reads the cache of entry {src}, which is not an "
                                             f"earlier entry that owns a cache")
                        owner_need = self.cache_groups[self._cache_slot[(src, role)][0]]
                        if (owner_need.n_kv_heads, owner_need.head_dim) != (need.n_kv_heads, need.head_dim):
                            raise ValueError(f"run order entry {i} cannot read the cache of entry {src}: "
                                             f"key/value shapes differ")
                        self._cache_slot[(i, role)] = self._cache_slot[(src, role)]
                        info.cache_group, info.writes_cache = self._cache_slot[(src, role)][0], False
                sn = mixer.state_need()
                if sn is not None:
                    self.state_needs[(i, role)] = sn
                entry.mixers[role] = info
            if lc.cache is not None and not any_cache:
                raise ValueError(f"run order entry {i} names a cache but its mixer keeps none")
            self.calls.append(entry)

    # ---------------------------------------------------------------- weights
    def parts(self):
        """Every part of the model, each object once."""
        seen = set()

        def once(p):
            if p is not None and id(p) not in seen:
                seen.add(id(p))
                yield p
        yield from once(self.embedding)
        for b in self.blocks:
            yield from once(b)
            for p in b.parts.values():
                yield from once(p)
                yield from once(getattr(p, "position", None))
        yield from once(self.final_norm)
        yield from once(self.head)

    @property
    def capturable(self) -> bool:
        """Whether a step of this model may be replayed from a CUDA graph (every part allows it)."""
        return all(p.capturable for p in self.parts())

    @property
    def chain_safe(self) -> bool:
        """Whether the launchers may chain the products of a small decode step (every part goes through them alone)."""
        return all(p.chain_safe for p in self.parts())

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
    def bind_storage(self, caches: List[torch.Tensor], states: Dict[Tuple[int, str], torch.Tensor]) -> None:
        """caches[g]: [owners in group g, pages, 2, n_kv, page_size, head_dim]; states[(call, role)]: [max_seqs, numel]."""
        for entry in self.calls:
            for role, info in entry.mixers.items():
                key = (entry.index, role)
                if key in self._cache_slot:
                    g, j = self._cache_slot[key]
                    info.cache = caches[g][j]
                info.state = states.get(key)

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
