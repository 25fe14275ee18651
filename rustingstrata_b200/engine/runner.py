"""The model runner: owns the model, its weights, the cache and the one step function.

``step`` is the engine's only way to run the model.  It takes a batch of
(request, its next tokens, the places whose logits are wanted) - portions of prompts
beside single decoded tokens, cut anywhere - runs exactly those tokens as one batch
against the cache earlier steps left, and returns the logits at the wanted places.
Generation, the scheduler, the benchmark and trace replay all go through it.

Reference: ``GpuModel::batch_rows`` (src/gpu_model/prefill.rs:781-845): rows of
(slot, token, want_logits), consecutive rows of a slot at consecutive positions, K/V of
every row stored before attention reads it, the head run on the wanted rows only.
"""
from __future__ import annotations

import gc
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Mapping, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, GroupNeed, OutOfPages, allocate_caches, allocate_states, cache_bytes_per_token
from ..config import EngineConfig, load_model_config, resolve_architecture
from ..dtypes import element_type
from ..kernels import ops
from ..models import CausalLM
from ..parts import HostBatch, Runtime, StepContext
from ..weights import load_checkpoint


class StepError(RuntimeError):
    pass


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the indices among them whose logits are wanted.

    ``stream_positions``: only for models whose position encodings follow more than the token count (their parts
    say ``n_streams`` > 1): per token, the values of position streams 1, 2, ... (stream 0 is always the token's place
    in its sequence, which the engine counts itself).  Left out, every stream equals stream 0."""
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    stream_positions: Optional[Sequence[Sequence[int]]] = None


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class ModelRunner:
    def __init__(self, arch, config, engine: EngineConfig, tensors_loader):
        """Use :meth:`from_dir` or :meth:`from_random`; ``tensors_loader(needs, dtype, device)`` returns
        name → device tensor for the model's manifest."""
        if not torch.cuda.is_available():
            raise RuntimeError("rustingstrata_b200 runs on a CUDA device only; no GPU is visible")
        self.arch, self.config, self.engine = arch, config, engine
        self.device = torch.device(engine.device)
        torch.cuda.set_device(self.device)
        self.dtype = element_type(engine.dtype).torch
        self.spec = arch.build_spec(config)
        self.page_size = engine.page_size
        self.num_pages = engine.pool_pages()
        self.runtime = Runtime(self.dtype, self.device, engine.max_batch_tokens, engine.max_seqs,
                               engine.max_logit_rows, engine.page_size, self.spec.max_positions,
                               self.num_pages * engine.page_size)
        self.model = CausalLM(self.spec, self.runtime)
        tensors = tensors_loader(self.model.tensor_needs(), self.dtype, self.device)
        self.model.load(tensors)
        del tensors
        self.vocab_size = self.spec.vocab_size
        self.max_positions = self.spec.max_positions
        # ---- cache and state
        m = self.model
        self.cache = CacheManager([GroupNeed(n.window) for n in m.cache_groups], self.page_size, self.num_pages,
                                  engine.max_seqs)
        self.caches = allocate_caches(m.cache_groups, m.group_calls, self.num_pages, self.page_size, self.dtype,
                                      self.device)
        self.states = allocate_states(m.state_needs, engine.max_seqs, self.device)
        m.bind_storage(self.caches, self.states)
        self.kv_bytes_per_token = cache_bytes_per_token(m.cache_groups, m.group_calls, self.dtype)
        # ---- step metadata buffers (pinned host mirror + device), grown on demand
        self._meta_host = None
        self._meta_dev = None
        self._meta_event = None
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.steps_run = 0
        self.h2d_bytes_last_step = 0
        # pure-decode steps (one token per request) are captured once per shape and replayed
        self.use_graphs = True
        self._graphs: Dict = {}
        self.graph_replays = 0
        self.kernels_replayed = 0           # kernels this runner launched through graph replays
        self.chain_kernels = 0              # chained-product kernels launched outside graph replays

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dir(cls, model_dir: str, engine: EngineConfig) -> "ModelRunner":
        arch, config = load_model_config(model_dir)

        def loader(needs, dtype, device):
            cpu = load_checkpoint(model_dir, needs, dtype)
            out = {}
            for k in list(cpu):
                out[k] = cpu.pop(k).to(device, non_blocking=False)
            return out
        return cls(arch, config, engine, loader)

    @classmethod
    def from_random(cls, config_dict: Mapping, engine: EngineConfig, seed: int = 0, std: float = 0.02,
                    norm_std: float = 0.0) -> "ModelRunner":
        """Weights drawn on the device (no file) by the generator of ``weights/random_init.py``: the same values,
        bit for bit, that ``write_random_model`` writes for this configuration, seed, std and norm_std (stored as
        bfloat16), so a folder made by ``init-random`` and this mode describe the same model.  For sizes too large
        to write to disk first."""
        from ..weights.random_init import normal_table, scale_shift, tensor_key
        arch = resolve_architecture(config_dict)
        config = arch.config_class.from_dict(config_dict)

        def loader(needs, dtype, device):
            table = torch.from_numpy(normal_table().copy()).to(device)
            out = {}
            for name, need in needs.items():
                if need.role == "int_table":
                    t = torch.empty(need.shape, dtype=torch.int32, device=device)
                    ops.fill_random(t, tensor_key(seed, name), None, 0.0, 0.0)
                else:
                    scale, shift = scale_shift(need, std, norm_std)
                    t = torch.empty(need.shape, dtype=torch.bfloat16, device=device)
                    ops.fill_random(t, tensor_key(seed, name), table, scale, shift)
                    if dtype == torch.float32:
                        t = t.to(torch.float32)
                out[name] = t
            torch.cuda.synchronize(device)
            return out
        return cls(arch, config, engine, loader)

    # ------------------------------------------------------------------ requests
    def admit(self, rid: Hashable) -> int:
        slot = self.cache.admit(rid)
        for st in self.states.values():
            st[slot].zero_()
        return slot

    def release(self, rid: Hashable) -> None:
        self.cache.release(rid)

    def length(self, rid: Hashable) -> int:
        return self.cache.length(rid)

    # ------------------------------------------------------------------ the step function
    def _meta_buffers(self, n_ints: int):
        if self._meta_host is None or self._meta_host.numel() < n_ints:
            cap = max(n_ints, 1 << 18)
            self._graphs.clear()                    # captured steps point into the old buffer
            cap = 1 << (cap - 1).bit_length()
            self._meta_host = torch.empty(cap, dtype=torch.int32).pin_memory()
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._meta_event = None
        if self._meta_event is not None:
            self._meta_event.synchronize()      # the previous upload has left the pinned buffer
        return self._meta_host, self._meta_dev

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None, post=None
             ) -> Optional[torch.Tensor]:
        """Runs one batch.  Returns float32 logits [wanted, vocab] on the device, in the order of the
        entries and of each entry's ``want`` (None when nothing is wanted).  Unknown requests are admitted.
        On an error nothing advances: pages taken for the step are given back.

        ``device_tokens`` (int32 on the device, one id per token of the step) replaces the entries' token
        values, which then only give the counts: a decode loop feeds the ids the device chose in the last
        step without the host waiting for them.  ``post(logits, n_rows)`` is called after the forward pass
        (the engine's sampling kernel); in a captured step it becomes part of the graph, so it must only
        launch kernels on buffers that stay where they are.

        A step of single tokens only is captured in a CUDA graph the first time its shape occurs (number of
        requests and logit rows, block-table width and attention splits rounded up to buckets) and replayed
        afterwards: the per-step index arrays live at fixed places of one device buffer that is refreshed
        before every replay."""
        eng = self.engine
        if not entries:
            raise StepError("a step needs at least one entry")
        ids = [e.rid for e in entries]
        if len(set(ids)) != len(ids):
            raise StepError("a request may appear once in a step")
        if len(entries) > eng.max_seqs:
            raise StepError(f"{len(entries)} requests in one step, the engine is built for {eng.max_seqs}")
        q_lens = np.array([len(e.tokens) for e in entries], dtype=np.int32)
        if (q_lens <= 0).any():
            raise StepError("every entry needs at least one token")
        T = int(q_lens.sum())
        if T > eng.max_batch_tokens:
            raise StepError(f"{T} tokens in one step, the engine is built for {eng.max_batch_tokens}")
        R = sum(len(e.want) for e in entries)
        if R > eng.max_logit_rows:
            raise StepError(f"{R} logit rows wanted in one step, the engine is built for {eng.max_logit_rows}")
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if (tokens < 0).any() or (tokens >= self.vocab_size).any():
            bad = int(tokens[(tokens < 0) | (tokens >= self.vocab_size)][0])
            raise StepError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
        for e, n in zip(entries, q_lens):
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.rid!r}: wanted place {w} is not among its {n} tokens")
        n_streams = self.model.n_position_streams
        for e, n in zip(entries, q_lens):
            if e.stream_positions is None:
                continue
            sp = np.asarray(e.stream_positions, dtype=np.int64)
            if n_streams == 1:
                raise StepError(f"request {e.rid!r} gives position streams, the model's position encodings use none")
            if sp.shape != (n, n_streams - 1):
                raise StepError(f"request {e.rid!r}: stream_positions must be [{n} tokens][{n_streams - 1} streams], got "
                                f"shape {sp.shape}")
            if (sp < 0).any() or (sp >= self.max_positions).any():
                raise StepError(f"request {e.rid!r}: a stream position lies outside 0..{self.max_positions - 1}")

        admitted, reserved = [], []
        try:
            for e in entries:
                if not self.cache.is_live(e.rid):
                    self.admit(e.rid)
                    admitted.append(e.rid)
            old = np.array([self.cache.length(e.rid) for e in entries], dtype=np.int32)
            kv_lens = old + q_lens
            if (kv_lens > self.max_positions).any():
                i = int(np.argmax(kv_lens > self.max_positions))
                raise StepError(f"request {entries[i].rid!r} would reach {int(kv_lens[i])} positions, the model "
                                f"has {self.max_positions}")
            for e, n in zip(entries, q_lens):
                self.cache.reserve(e.rid, int(n))
                reserved.append(e.rid)
        except Exception:
            for rid in reserved:
                self.cache.rollback(rid)
            for rid in admitted:
                self.cache.release(rid)
            raise

        if device_tokens is not None and (device_tokens.dtype != torch.int32 or device_tokens.numel() < T
                                          or not device_tokens.is_cuda):
            raise StepError("device_tokens must be int32 on the device with one id per token")
        graphable = self.use_graphs and self.model.capturable and bool((q_lens == 1).all())
        try:
            ctx, layout = self._build_context(entries, tokens, q_lens, old, kv_lens, T, R, graphable)

            chain = (ops.CHAIN_DECODE and self.dtype == torch.bfloat16 and T <= ops.chain_max_rows()
                     and self.model.chain_safe)

            def run():
                if device_tokens is not None:
                    ctx.token_ids[:T].copy_(device_tokens[:T], non_blocking=True)
                if chain:
                    # a small decode step: the products between two attention calls leave as one persistent kernel
                    ops.begin_chain(self.status)
                    try:
                        out = self.model.forward(ctx)
                    finally:
                        self.chain_kernels += ops.end_chain()
                else:
                    out = self.model.forward(ctx)
                if post is not None:
                    post(out, R)
                return out
            if not graphable:
                logits = run()
            else:
                key = (layout, None if device_tokens is None else device_tokens.data_ptr(), post)
                entry = self._graphs.get(key)
                if entry is None:
                    logits = run()                        # first time: eagerly (allocates every scratch buffer) ...
                    self._graphs[key] = "warm"
                elif entry == "warm":                     # ... second time: capture (the capture also runs nothing)
                    graph = torch.cuda.CUDAGraph()
                    # Python's cyclic collector must not run while the stream is capturing: freeing another
                    # engine's pinned buffers or graphs there is "not permitted" and invalidates the capture
                    gc_was_on = gc.isenabled()
                    gc.disable()
                    n0 = ops.launch_count()
                    try:
                        with torch.cuda.graph(graph):
                            logits = run()
                    finally:
                        if gc_was_on:
                            gc.enable()
                    kernels = ops.launch_count() - n0          # kernel nodes of this graph
                    self._graphs[key] = (graph, logits, kernels)
                    graph.replay()
                else:
                    graph, logits, kernels = entry
                    graph.replay()
                    self.graph_replays += 1
                    self.kernels_replayed += kernels
        except Exception:
            for rid in reserved:
                self.cache.rollback(rid)
            for rid in admitted:
                self.cache.release(rid)
            raise
        for e, n in zip(entries, q_lens):
            self.cache.commit(e.rid, int(n))
        self.steps_run += 1
        return logits

    def _build_context(self, entries, tokens, q_lens, old, kv_lens, T, R, bucketed=False):
        """The step's index arrays in one pinned buffer, uploaded with one copy.  Returns the context and a
        hashable description of the layout (sizes and host scalars): equal layouts put every array at the
        same device address, which is what lets a captured step be replayed."""
        S = len(entries)
        q_start = np.zeros(S + 1, dtype=np.int32)
        np.cumsum(q_lens, out=q_start[1:])
        seq_of_token = np.repeat(np.arange(S, dtype=np.int32), q_lens)
        place = (np.arange(T, dtype=np.int32) - np.repeat(q_start[:-1], q_lens) + np.repeat(old, q_lens)
                 ).astype(np.int32)
        n_streams = self.model.n_position_streams
        positions = np.repeat(place[:, None], n_streams, axis=1)           # [T, streams]; stream 0 = place in the cache
        if n_streams > 1:
            for i, e in enumerate(entries):
                if e.stream_positions is not None:
                    positions[q_start[i]:q_start[i + 1], 1:] = np.asarray(e.stream_positions, dtype=np.int32)
        slots = np.array([self.cache.slot(e.rid) for e in entries], dtype=np.int32)
        logit_rows = np.array([q_start[i] + w for i, e in enumerate(entries) for w in e.want], dtype=np.int32)
        n_groups = len(self.cache.groups)
        tables = []
        for g in range(n_groups):
            rows = [self.cache.table(e.rid, g) for e in entries]
            width = max(1, max(len(r) for r in rows))
            if bucketed:
                width = (width + 63) // 64 * 64
            tab = np.full((S, width), -1, dtype=np.int32)
            for i, r in enumerate(rows):
                tab[i, :len(r)] = r
            tables.append(tab)
        batch = HostBatch(n_tokens=T, n_seqs=S, q_lens=q_lens, kv_lens=kv_lens.astype(np.int32), q_start=q_start,
                          state_slots=slots, first_step=(old == 0).astype(np.int32), page_size=self.page_size,
                          max_blocks=[t.shape[1] for t in tables], bucketed=bucketed)
        plans = self.model.plan(batch)

        arrays = [("token_ids", tokens.astype(np.int32)), ("positions", positions.reshape(-1)), ("seq_of_token", seq_of_token),
                  ("q_start", q_start), ("kv_len", batch.kv_lens), ("state_slots", slots), ("logit_rows", logit_rows)]
        arrays += [(("table", g), t.reshape(-1)) for g, t in enumerate(tables)]
        for key, plan in plans.items():
            for name, val in plan.items():
                if isinstance(val, np.ndarray):
                    arrays.append((("plan", key, name), val.astype(np.int32, copy=False).reshape(-1)))
        offsets, total = [], 0
        for _, a in arrays:
            offsets.append(total)
            total += _align(max(1, a.size))
        host, dev = self._meta_buffers(total)
        hv = host.numpy()
        for (_, a), off in zip(arrays, offsets):
            hv[off:off + a.size] = a
        dev[:total].copy_(host[:total], non_blocking=True)
        self.h2d_bytes_last_step = total * 4
        self._meta_event = torch.cuda.Event()
        self._meta_event.record()
        view = {name: dev[off:off + max(1, a.size)] for (name, a), off in zip(arrays, offsets)}
        dev_plans: Dict = {}
        for key, plan in plans.items():
            dev_plans[key] = {name: (view[("plan", key, name)] if isinstance(val, np.ndarray) else val)
                              for name, val in plan.items()}
        block_tables = [view[("table", g)][: S * tables[g].shape[1]].view(S, tables[g].shape[1])
                        for g in range(n_groups)]
        ctx = StepContext(n_tokens=T, n_seqs=S, n_logit_rows=R, token_ids=view["token_ids"],
                          positions=view["positions"][: T * n_streams].view(T, n_streams), seq_of_token=view["seq_of_token"], q_start=view["q_start"],
                          kv_len=view["kv_len"], state_slots=view["state_slots"], logit_rows=view["logit_rows"],
                          block_tables=block_tables, status=self.status, host=batch, plans=dev_plans)
        scalars = tuple((repr(key), name, val) for key, plan in plans.items() for name, val in sorted(plan.items())
                        if not isinstance(val, np.ndarray))
        layout = (dev.data_ptr(), tuple(a.size for _, a in arrays), scalars)
        return ctx, layout

    def check_status(self) -> None:
        """Waits for the device and raises if a kernel of an earlier step flagged a bad input."""
        self._status_host.copy_(self.status, non_blocking=False)
        code = int(self._status_host[0])
        if code:
            self.status.zero_()
            if code & ops.STATUS_WAIT_EXPIRED:
                ops.reset_chain_barrier()
            what = [n for b, n in ((ops.STATUS_BAD_TOKEN, "token id outside the vocabulary"),
                                   (ops.STATUS_BAD_PAGE, "block table entry outside the page pool"),
                                   (ops.STATUS_WAIT_EXPIRED, "a bounded wait inside a kernel gave up"),
                                   (ops.STATUS_NON_FINITE, "logits are not finite"),
                                   (ops.STATUS_BAD_PLAN, "a work list points outside its workspace")) if code & b]
            raise StepError("device status: " + "; ".join(what))
