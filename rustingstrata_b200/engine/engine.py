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
        self._temps_h = torch.zeros(n, dtype=torch.float32).pin_memory()
        self._unif_h = torch.zeros(n, dtype=torch.float32).pin_memory()
        self._temps_d = torch.zeros(n, dtype=torch.float32, device=r.device)
        self._unif_d = torch.zeros(n, dtype=torch.float32, device=r.device)
        self._picked_d = torch.zeros(n, dtype=torch.int32, device=r.device)
        self._picked_h = torch.zeros(n + 1, dtype=torch.int32).pin_memory()
        self.h2d_bytes_last_step = 0
        self.d2h_bytes_last_step = 0

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
        """Schedules and runs one step, chooses the next tokens, returns the requests that finished."""
        batch = self.scheduler.schedule()
        if not batch:
            if self.scheduler.has_work():
                self.scheduler.step_index += 1     # nothing could run (arrivals in the future): time passes
            return []
        entries = [StepEntry(s.request.rid, s.tokens, [len(s.tokens) - 1] if s.samples else []) for s in batch]
        sampled = [s for s in batch if s.samples]
        host_rows = self._prepare_sampling(sampled)
        logits = self.runner.step(entries, post=self._sample_post if sampled else None)
        chosen = self._collect(sampled, host_rows, logits)
        done = self.scheduler.advance(batch, chosen)
        for r in done:
            self._samplers.pop(r.rid, None)
        return done

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

    def _collect(self, sampled: Sequence[Scheduled], host_rows: List[int], logits: Optional[torch.Tensor]
                 ) -> Dict[Hashable, int]:
        """Brings the chosen ids (and the logits of host-sampled rows) back and records them."""
        if not sampled:
            self.runner.check_status()
            return {}
        R = len(sampled)
        self._picked_h[:R].copy_(self._picked_d[:R], non_blocking=True)
        self._picked_h[R:R + 1].copy_(self.runner.status, non_blocking=True)
        host_logits = {i: logits[i].to("cpu").numpy() for i in host_rows}      # also waits for the stream
        self.h2d_bytes_last_step = self.runner.h2d_bytes_last_step + 8 * R
        self.d2h_bytes_last_step = 4 * (R + 1) + 4 * logits.shape[1] * len(host_rows)
        torch.cuda.current_stream().synchronize()
        picked = self._picked_h.numpy()
        if int(picked[R]) != 0:
            self.runner.check_status()
        out = {}
        for i, s in enumerate(sampled):
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

    # ------------------------------------------------------------------ device-resident greedy decode
    def decode_steps_device_timed(self, n_steps: int) -> float:
        """Runs ``n_steps`` greedy decode steps of all running requests with the chosen ids staying on
        the device between steps (the host only counts lengths), and returns the milliseconds per step
        measured with CUDA events.  The generated ids are appended to the requests afterwards."""
        reqs = list(self.scheduler.running)
        if not reqs or any(r.prefilling for r in reqs) or self.scheduler.waiting:
            raise RuntimeError("device decode needs every request past its prompt and none waiting")
        B = len(reqs)
        r = self.runner
        first = torch.tensor([q.all_tokens[-1] for q in reqs], dtype=torch.int32).pin_memory()
        self._picked_d[:B].copy_(first, non_blocking=True)
        history = torch.zeros((n_steps, B), dtype=torch.int32, device=r.device)
        entries = [StepEntry(q.rid, [0], [0]) for q in reqs]
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record()
        self._temps_h[:B].zero_()
        self._temps_d[:B].copy_(self._temps_h[:B], non_blocking=True)
        for i in range(n_steps):
            r.step(entries, device_tokens=self._picked_d, post=self._sample_post)
            history[i].copy_(self._picked_d[:B], non_blocking=True)
        ev1.record()
        torch.cuda.synchronize()
        r.check_status()
        ms = ev0.elapsed_time(ev1) / n_steps
        hist = history.cpu().numpy()
        for j, q in enumerate(reqs):
            q.generated.extend(int(t) for t in hist[:, j])
            q.computed += n_steps
        return ms

    # ------------------------------------------------------------------ replay hook
    def step_raw(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """The runner's step function, untouched by the scheduler (what trace replay calls)."""
        return self.runner.step(entries)

    def release(self, rid: Hashable) -> None:
        self.runner.release(rid)
