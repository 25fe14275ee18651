"""The Python entry point: load a model, generate, or drive the scheduler step by step.

The reference is a command-line binary (``generate``, ``bench``, ``score``:
src/main.rs:999-1013,960-977,857-866) whose runner offers ``prefill`` / ``step`` /
``reset`` (src/main.rs:224-343).  :class:`Engine` is the same surface as a Python
class: ``generate`` (prompt ids in, token ids out), ``add_request`` + ``step`` for
continuous batching, ``step_raw`` for replay, with the reference's option names for
sampling (temp, top_k, top_p, seed, the penalties).
"""
from __future__ import annotations

import itertools
from typing import Dict, Hashable, List, Mapping, Optional, Sequence, Union

import numpy as np
import torch

from ..config import EngineConfig
from ..kernels import ops
from ..sampling import Sampler, SamplingError, SamplingParams, NON_FINITE
from .runner import ModelRunner, StepEntry
from .scheduler import Request, Scheduled, Scheduler


class _Flight:
    """A step that has been enqueued on the device and whose tokens have not been read yet."""

    def __init__(self, batch, sampled, host_rows, logits, event, picked_h, h2d_bytes):
        self.batch, self.sampled, self.host_rows, self.logits = batch, sampled, host_rows, logits
        self.event, self.picked_h, self.h2d_bytes = event, picked_h, h2d_bytes
        self.n_rows = len(sampled)       # rows the device sampled; stays what it was if rows are dropped later


class Engine:
    def __init__(self, model: Union[str, Mapping], dtype: str = "bfloat16", random_seed: Optional[int] = None,
                 page_size: int = 16, num_pages: int = 0, max_tokens: int = 4096, max_batch_tokens: int = 2048,
                 max_seqs: int = 64, prefill_chunk: Optional[int] = None, device: str = "cuda:0",
                 random_std: float = 0.02, random_norm_std: float = 0.0):
        """``model``: a folder (config.json + model.safetensors), or a config mapping together with
        ``random_seed`` to draw the weights on the device."""
        cfg = EngineConfig(dtype=dtype, page_size=page_size, num_pages=num_pages, max_tokens=max_tokens,
                           max_seqs=max_seqs, max_batch_tokens=max_batch_tokens,
                           max_logit_rows=max(max_seqs, 64), device=device)
        if isinstance(model, str):
            self.runner = ModelRunner.from_dir(model, cfg)
        else:
            if random_seed is None:
                raise ValueError("a config mapping needs random_seed (random-weights mode)")
            self.runner = ModelRunner.from_random(model, cfg, seed=random_seed, std=random_std,
                                                  norm_std=random_norm_std)
        self.config = cfg
        r = self.runner
        self.scheduler = Scheduler(r.cache, max_batch_tokens, max_seqs, r.max_positions, prefill_chunk,
                                   admit=r.admit, release=r.release)
        self._samplers: Dict[Hashable, Sampler] = {}
        self._ids = itertools.count()
        n = cfg.max_logit_rows
        # pinned host buffers come in pairs: two steps can be under way (one running, the next one launched ahead)
        self._temps_hh = [torch.zeros(n, dtype=torch.float32).pin_memory() for _ in range(2)]
        self._unif_hh = [torch.zeros(n, dtype=torch.float32).pin_memory() for _ in range(2)]
        self._src_hh = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._picked_hh = [torch.zeros(n + 1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._temps_h, self._unif_h, self._picked_h = self._temps_hh[0], self._unif_hh[0], self._picked_hh[0]
        self._temps_d = torch.zeros(n, dtype=torch.float32, device=r.device)
        self._unif_d = torch.zeros(n, dtype=torch.float32, device=r.device)
        self._picked_d = torch.zeros(n, dtype=torch.int32, device=r.device)
        self._src_d = torch.zeros(n, dtype=torch.int32, device=r.device)
        self._next_ids_d = torch.zeros(n, dtype=torch.int32, device=r.device)
        self.h2d_bytes_last_step = 0
        self.d2h_bytes_last_step = 0
        # While a step runs, the next one is launched if the scheduler can tell its batch without this step's tokens
        # (all requests decoding, nobody waiting, device-side sampling): the ids stay on the device, the host reads
        # them one step late.  ``lookahead = False`` makes every step wait for its tokens before the next is built.
        self.lookahead = True
        self._flight: Optional[_Flight] = None
        self._launches = 0
        self.steps_launched_ahead = 0

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_ids: Sequence[int], max_new_tokens: int = 32, sampling: Optional[SamplingParams] = None,
                    eos_ids: Sequence[int] = (), rid: Optional[Hashable] = None, arrival: int = 0) -> Hashable:
        rid = next(self._ids) if rid is None else rid
        sampling = sampling or SamplingParams()
        req = Request(rid=rid, prompt=[int(t) for t in prompt_ids], max_new_tokens=int(max_new_tokens),
                      eos_ids=tuple(int(e) for e in eos_ids), sampling=sampling, arrival=arrival)
        for t in req.prompt:
            if not 0 <= t < self.runner.vocab_size:
                raise ValueError(f"token id {t} is outside the vocabulary of {self.runner.vocab_size}")
        self.scheduler.add(req)
        self._samplers[rid] = Sampler(sampling)
        return rid

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    # ------------------------------------------------------------------ one scheduler step
    def step(self) -> List[Request]:
        """Runs one step to its end: schedules and launches it (unless the previous call already launched it ahead),
        launches the step after it when that is possible, then reads this step's tokens and returns the requests
        that finished with it."""
        fl, self._flight = self._flight, None
        if fl is None:
            batch = self.scheduler.schedule()
            if not batch:
                if self.scheduler.has_work():
                    self.scheduler.step_index += 1     # nothing could run (arrivals in the future): time passes
                return []
            fl = self._launch(batch, None)
        nxt = None
        try:
            if self.lookahead and fl.sampled and not fl.host_rows:
                ahead = self.scheduler.lookahead(fl.batch)
                if ahead:
                    nxt = self._launch(ahead, fl)
                    self.steps_launched_ahead += 1
            chosen = self._collect(fl)
        except Exception:
            self._drop_flight(nxt)
            raise
        done = self.scheduler.advance(fl.batch, chosen)
        for r in done:
            self._samplers.pop(r.rid, None)
        if nxt is not None:
            gone = {id(r) for r in done}
            if gone:                                   # ended by an end-of-sequence token: its row ran for nothing
                nxt.batch = [s for s in nxt.batch if id(s.request) not in gone]
                nxt.sampled = [(i, s) for i, s in nxt.sampled if id(s.request) not in gone]
            if nxt.batch:
                self._flight = nxt
        return done

    def _drop_flight(self, fl: Optional["_Flight"]) -> None:
        """Forgets a step launched ahead whose results will not be used (its kernels still run to their end)."""
        if fl is not None:
            fl.event.synchronize()

    def drain(self) -> List[Request]:
        """Waits for a step launched ahead and takes its tokens in, so that nothing is under way; returns the
        requests that finished with it."""
        done: List[Request] = []
        while self._flight is not None:
            look, self.lookahead = self.lookahead, False
            try:
                done += self.step()
            finally:
                self.lookahead = look
        return done

    def _launch(self, batch: List[Scheduled], prev: Optional["_Flight"]) -> "_Flight":
        """Enqueues one step: sampling parameters up, the forward pass and the device's token choice, the chosen
        ids down, an event behind them.  With ``prev`` the tokens are the ids ``prev`` chose, taken on the device."""
        k = self._launches & 1
        self._launches += 1
        self._temps_h, self._unif_h, self._picked_h = self._temps_hh[k], self._unif_hh[k], self._picked_hh[k]
        sampled = [(i, s) for i, s in enumerate(x for x in batch if x.samples)]
        only = [s for _, s in sampled]
        host_rows = self._prepare_sampling(only)
        device_tokens = None
        if prev is None:
            entries = [StepEntry(s.request.rid, s.tokens, [len(s.tokens) - 1] if s.samples else []) for s in batch]
        else:
            row_of = {id(s.request): i for i, s in prev.sampled}
            src = self._src_hh[k].numpy()
            for j, s in enumerate(batch):
                src[j] = row_of[id(s.request)]
            n = len(batch)
            self._src_d[:n].copy_(self._src_hh[k][:n], non_blocking=True)
            ops.gather_i32(self._next_ids_d, self._picked_d, self._src_d, n)
            device_tokens = self._next_ids_d
            entries = [StepEntry(s.request.rid, [0], [0]) for s in batch]
        logits = self.runner.step(entries, device_tokens=device_tokens, post=self._sample_post if sampled else None)
        R = len(sampled)
        if R:
            self._picked_h[:R].copy_(self._picked_d[:R], non_blocking=True)
        self._picked_h[R:R + 1].copy_(self.runner.status, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        h2d = self.runner.h2d_bytes_last_step + 8 * R + (4 * len(batch) if prev is not None else 0)
        return _Flight(batch, sampled, host_rows, logits, event, self._picked_h, h2d)

    def _prepare_sampling(self, sampled: Sequence[Scheduled]) -> List[int]:
        """Uploads temperatures and uniforms of the rows the device will sample; returns the rows that
        need the host sampler instead (cuts or penalties)."""
        R = len(sampled)
        if not R:
            return []
        th, uh = self._temps_h.numpy(), self._unif_h.numpy()
        host_rows = []
        for i, s in enumerate(sampled):
            sp: SamplingParams = s.request.sampling
            if sp.needs_host():
                host_rows.append(i)
                th[i] = 0.0
                uh[i] = 0.0
            else:
                th[i] = sp.temp
                uh[i] = self._samplers[s.request.rid].rng.uniform() if sp.temp > 0 else 0.0
        self._temps_d[:R].copy_(self._temps_h[:R], non_blocking=True)
        self._unif_d[:R].copy_(self._unif_h[:R], non_blocking=True)
        return host_rows

    def _sample_post(self, logits: torch.Tensor, n_rows: int) -> None:
        """The device's token choice, run right after the forward pass (inside the graph of a captured step)."""
        ops.sample(logits, n_rows, self._picked_d, self.runner.status, self._temps_d, self._unif_d)

    def _collect(self, fl: "_Flight") -> Dict[Hashable, int]:
        """Waits for the step's chosen ids (and brings the logits of host-sampled rows back) and records them."""
        R = fl.n_rows
        host_logits = {i: fl.logits[i].to("cpu").numpy() for i in fl.host_rows}      # also waits for the stream
        self.h2d_bytes_last_step = fl.h2d_bytes
        self.d2h_bytes_last_step = 4 * (R + 1) + (4 * fl.logits.shape[1] * len(fl.host_rows) if fl.host_rows else 0)
        fl.event.synchronize()
        picked = fl.picked_h.numpy()
        if int(picked[R]) != 0:
            self.runner.check_status()
        out = {}
        for i, s in fl.sampled:
            smp = self._samplers[s.request.rid]
            if i in host_logits:
                out[s.request.rid] = smp.pick(host_logits[i])
            else:
                t = int(picked[i])
                if t < 0:
                    raise SamplingError(NON_FINITE)
                smp.note(t)
                out[s.request.rid] = t
        return out

    # ------------------------------------------------------------------ whole generations
    def generate(self, prompt_ids, max_new_tokens: int = 32, temperature: float = 0.0, top_k: int = 0,
                 top_p: float = 1.0, seed: int = 0, eos_ids: Sequence[int] = (), **penalties):
        """Token ids of the continuation.  ``prompt_ids`` is one prompt (list of ints) or a list of
        prompts; the result has the same nesting.  Further keyword arguments are the penalty options
        of :class:`~rustingstrata_b200.sampling.SamplingParams`."""
        single = len(prompt_ids) > 0 and not isinstance(prompt_ids[0], (list, tuple, np.ndarray))
        prompts = [prompt_ids] if single else list(prompt_ids)
        rids = []
        for i, p in enumerate(prompts):
            sp = SamplingParams(temp=temperature, top_k=top_k, top_p=top_p, seed=seed + i, **penalties)
            rids.append(self.add_request(p, max_new_tokens, sp, eos_ids))
        results: Dict[Hashable, List[int]] = {}
        while len(results) < len(rids):
            for r in self.step():
                if r.rid in rids:
                    results[r.rid] = list(r.generated)
        outs = [results[r] for r in rids]
        return outs[0] if single else outs

    # ------------------------------------------------------------------ timed prefill and decode
    def bench(self, pp: Sequence[int] = (512, 4096), tg: int = 128, reps: int = 3, batch: int = 1, seed: int = 0) -> List[dict]:
        """The reference's ``bench`` (src/main.rs:1192-1265) as a method: for every prompt length in ``pp``, ``reps``
        times: ``batch`` prompts of seeded random ids are run to the end of their prompts (timed: prefill tok/s), then
        ``tg`` tokens each are decoded greedily (timed: decode tok/s over all requests).  Wall-clock times around
        ``step`` with a device synchronisation on both sides.  Returns one record per prompt length with mean, min
        and max of both rates, and ``roofline``: the decode step's bytes (weights once, the live cache) over the HBM
        peak and the prompts' multiply-adds over the tensor peak, both at the mean rate."""
        import time
        from . import roofline
        rng = np.random.default_rng(seed)
        out = []
        pk = roofline.peaks()
        model = self.runner.model
        for n in pp:
            pre, dec = [], []
            for _ in range(reps):
                self.drain()
                for _ in range(batch):
                    self.add_request(rng.integers(0, self.runner.vocab_size, size=n).tolist(), tg + 1, SamplingParams())
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                look, self.lookahead = self.lookahead, False   # the prompts' time must not hold the first decode step
                while self.scheduler.waiting or any(r.prefilling for r in self.scheduler.running):
                    self.step()
                torch.cuda.synchronize()
                self.lookahead = look
                t1 = time.perf_counter()
                steps = 0
                while self.has_work():
                    self.step()
                    steps += 1
                torch.cuda.synchronize()
                t2 = time.perf_counter()
                pre.append(n * batch / (t1 - t0))
                dec.append(batch * steps / (t2 - t1))
            stat = lambda xs: {"mean": sum(xs) / len(xs), "min": min(xs), "max": max(xs)}  # noqa: E731
            rec = {"pp": int(n), "tg": int(tg), "batch": int(batch), "prefill_tok_s": stat(pre), "decode_tok_s": stat(dec)}
            pre_ms = n * batch / rec["prefill_tok_s"]["mean"] * 1000
            dec_ms = batch / rec["decode_tok_s"]["mean"] * 1000 if rec["decode_tok_s"]["mean"] > 0 else float("inf")
            rec["roofline"] = {
                "prefill": roofline.prefill_roofline(model, [n] * batch, [n] * batch, batch, pre_ms, pk, self.config.dtype),
                # the cache a decode step reads grows from n to n + tg tokens per request: the middle stands for all
                "decode": roofline.decode_roofline(model, self.runner.kv_bytes_per_token, batch * (n + tg / 2.0), dec_ms, pk),
            }
            out.append(rec)
        return out

    # ------------------------------------------------------------------ device-resident greedy decode
    def decode_steps_device_timed(self, n_steps: int, warmup: int = 3) -> float:
        """Runs ``warmup + n_steps`` greedy decode steps of all running requests with the chosen ids staying on
        the device between steps (the host only counts lengths), and returns the milliseconds per step of the last
        ``n_steps``, measured with CUDA events.  The warm-up steps let this loop's own CUDA graph be captured (the
        first step of a new layout runs eagerly, the second captures) before the clock starts.  The generated ids
        are appended to the requests afterwards."""
        self.drain()
        reqs = list(self.scheduler.running)
        if not reqs or any(r.prefilling for r in reqs) or self.scheduler.waiting:
            raise RuntimeError("device decode needs every request past its prompt and none waiting")
        B = len(reqs)
        r = self.runner
        first = torch.tensor([q.all_tokens[-1] for q in reqs], dtype=torch.int32).pin_memory()
        self._picked_d[:B].copy_(first, non_blocking=True)
        total = warmup + n_steps
        history = torch.zeros((total, B), dtype=torch.int32, device=r.device)
        entries = [StepEntry(q.rid, [0], [0]) for q in reqs]
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self._temps_h[:B].zero_()
        self._temps_d[:B].copy_(self._temps_h[:B], non_blocking=True)
        for i in range(total):
            if i == warmup:
                torch.cuda.synchronize()
                ev0.record()
                launched0 = ops.launch_count() + r.kernels_replayed
            r.step(entries, device_tokens=self._picked_d, post=self._sample_post)
            history[i].copy_(self._picked_d[:B], non_blocking=True)
        ev1.record()
        torch.cuda.synchronize()
        r.check_status()
        ms = ev0.elapsed_time(ev1) / n_steps
        self.kernels_in_timed_steps = ops.launch_count() + r.kernels_replayed - launched0
        hist = history.cpu().numpy()
        for j, q in enumerate(reqs):
            q.generated.extend(int(t) for t in hist[:, j])
            q.computed += total
        return ms

    # ------------------------------------------------------------------ replay hook
    def step_raw(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """The runner's step function, untouched by the scheduler (what trace replay calls)."""
        return self.runner.step(entries)

    def release(self, rid: Hashable) -> None:
        self.runner.release(rid)
