"""Continuous-batching scheduler: which tokens go into the next step.

The reference's scheduler lives in its server loop (``Sched`` + ``serve_slots``,
src/main.rs:2314-2500): queued chats are admitted into free slots oldest first, prefill
is cut into ``--chunk`` tokens per forward (src/gpu_model/prefill.rs:143), running
slots decode one token per forward, and decode is interleaved between prefill
forwards.  With a paged cache and a step function that mixes portions and single
tokens, this scheduler builds one mixed batch per step:

1. every running request that has its prompt in the cache contributes one decode token;
2. what is left of the token budget goes to prompt portions, oldest request first
   (a portion may be cut anywhere);
3. waiting requests are admitted in arrival order while a state slot is free and the
   pools can hold the request's whole prompt plus one page of decoding (or its whole
   life, if that is less) on top of everything the running requests still have to
   bring into the cache.

When pages run out for a decode token, the most recently admitted running request is
preempted: its pages are given back and it returns to the head of the waiting queue
with prompt = original prompt + tokens generated so far, to be recomputed.  The same
happens when no running request can take a single token (every one of them waits for
pages another holds): the newest yields until the oldest can go on.  A request that
can never fit (longer than the pool or than the model's positions) is rejected when it
is added; what is accepted there can always be admitted into an empty engine.  So
``schedule`` returns an empty batch only when every waiting request arrives later.
The scheduler is pure host logic over the cache manager.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache import CacheManager, OutOfSlots


class RequestRejected(ValueError):
    pass


class SchedulerStuck(RuntimeError):
    """Requests are running but none can take a token and nobody can yield (a fault of the bookkeeping, not a
    state a workload can reach): raised instead of returning empty batches for ever."""


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    max_new_tokens: int
    eos_ids: Tuple[int, ...] = ()
    sampling: object = None                 # SamplingParams, interpreted by the engine
    arrival: int = 0                        # step index from which the request may be admitted
    # progress
    generated: List[int] = field(default_factory=list)
    computed: int = 0                       # tokens of `all_tokens` that are in the cache
    preemptions: int = 0
    finished: bool = False
    finish_reason: Optional[str] = None

    @property
    def all_tokens(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def prefilling(self) -> bool:
        """True while tokens other than the newest one still have to enter the cache."""
        return self.computed < len(self.prompt) + len(self.generated) - (1 if self.generated else 0)


@dataclass
class Scheduled:
    """One request's share of the next step."""
    request: Request
    tokens: List[int]
    samples: bool            # whether the logits of the last of these tokens choose the next token


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_tokens: int, max_seqs: int, max_positions: int,
                 prefill_chunk: Optional[int] = None, admit=None, release=None):
        self.cache = cache
        # the engine passes its own admit/release so that per-request state is zeroed with the slot
        self._admit = admit or cache.admit
        self._release = release or cache.release
        self.max_batch_tokens = max_batch_tokens
        self.max_seqs = max_seqs
        self.max_positions = max_positions
        self.prefill_chunk = prefill_chunk or max_batch_tokens
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []        # in admission order
        self.step_index = 0
        self.preemptions = 0

    # ---------------------------------------------------------------- intake
    def add(self, req: Request) -> None:
        total = len(req.prompt) + req.max_new_tokens
        if not req.prompt:
            raise RequestRejected(f"request {req.rid!r}: empty prompt")
        if req.max_new_tokens <= 0:
            raise RequestRejected(f"request {req.rid!r}: max_new_tokens must be positive")
        if total > self.max_positions:
            raise RequestRejected(f"request {req.rid!r}: context full ({total} tokens; the model has "
                                  f"{self.max_positions} positions)")
        for g, (pool, need) in enumerate(zip(self.cache.pools, self.cache.groups)):
            # a group that keeps every key must hold the whole request; a window group the window and the page
            # that is being written
            most = self._pages_for(total)
            if need.window is not None:
                most = min(most, self._pages_for(need.window) + 1)
            if most > pool.num_pages:
                raise RequestRejected(f"request {req.rid!r}: context full ({total} tokens; cache group {g} holds "
                                      f"{pool.num_pages * self.cache.page_size})")
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---------------------------------------------------------------- helpers
    def _pages_for(self, n_tokens: int) -> int:
        return (n_tokens + self.cache.page_size - 1) // self.cache.page_size

    def _preempt_newest(self, keep: Request) -> bool:
        """Frees the most recently admitted running request other than ``keep``; False if there is none."""
        for r in reversed(self.running):
            if r is not keep:
                self.running.remove(r)
                self._release(r.rid)
                r.computed = 0
                r.preemptions += 1
                self.preemptions += 1
                self.waiting.appendleft(r)
                return True
        return False

    # ---------------------------------------------------------------- one step
    def schedule(self) -> List[Scheduled]:
        """The next step's batch; reserves nothing (the runner's step reserves pages itself), but
        guarantees the pages are there by preempting or deferring.  Empty only when nothing runs and every
        waiting request arrives later."""
        for _ in range(self.max_seqs + 2):
            batch = self._schedule_once()
            if batch or not self.running:
                return batch
            # requests are running and none can take a token: each waits for pages that another holds.  The
            # newest yields (recomputed later) until the oldest can go on.
            if not self._preempt_newest(keep=self.running[0]):
                break
        raise SchedulerStuck(f"{len(self.running)} running request(s) cannot take a token and nobody can yield "
                             f"(free pages per group: {[p.n_free for p in self.cache.pools]})")

    def _outstanding_pages(self) -> List[int]:
        """Per group, the pages the running requests still need for every token they are known to have (the rest
        of a prompt, the newest decoded token).  Window groups give pages back on the way, so this is an upper
        bound there."""
        out = [0] * len(self.cache.groups)
        for r in self.running:
            for g, k in enumerate(self.cache.pages_to_reserve(r.rid, len(r.all_tokens) - r.computed)):
                out[g] += k
        return out

    def _admission_pages(self, req: Request) -> int:
        """Pages a request must find free to be admitted: its whole prompt plus one page of decoding, or its
        whole life if that is less (``add`` accepts what fits the pool, so the extra page must not push a
        request that fills the pool's last page out for ever)."""
        todo = len(req.all_tokens) - req.computed
        life = max(todo, len(req.prompt) + req.max_new_tokens)
        return min(self._pages_for(todo) + 1, self._pages_for(life))

    def _schedule_once(self) -> List[Scheduled]:
        budget = self.max_batch_tokens
        batch: List[Scheduled] = []
        promised = [0] * len(self.cache.groups)      # pages this step will take, per group

        def fits(req: Request, n: int) -> bool:
            need = self.cache.pages_to_reserve(req.rid, n)
            return all(need[g] + promised[g] <= self.cache.n_free(g) for g in range(len(need)))

        def promise(req: Request, n: int) -> None:
            for g, k in enumerate(self.cache.pages_to_reserve(req.rid, n)):
                promised[g] += k

        # 1. decode tokens of running requests, oldest first; preempt the newest when pages run out
        for req in list(self.running):
            if req not in self.running or req.prefilling or budget <= 0:
                continue
            while not fits(req, 1):
                if not self._preempt_newest(keep=req):
                    break
                # a preempted request may already be in this step's batch
                batch = [s for s in batch if s.request in self.running]
                promised = [0] * len(promised)
                for s in batch:
                    promise(s.request, len(s.tokens))
            if not fits(req, 1):
                continue                              # alone and still no page: wait for a finish
            tok = req.all_tokens[req.computed:]
            assert len(tok) == 1
            batch.append(Scheduled(req, tok, True))
            promise(req, 1)
            budget -= 1

        # 2. prompt portions of running requests that are still prefilling, oldest first
        for req in self.running:
            if not req.prefilling or budget <= 0:
                continue
            budget -= self._schedule_portion(req, budget, batch, fits, promise)

        # 3. admit waiting requests in arrival order
        windowed = [g.window is not None for g in self.cache.groups]
        owed = None
        while self.waiting and budget > 0 and len(self.running) < self.max_seqs:
            req = self.waiting[0]
            if req.arrival > self.step_index:
                break
            if owed is None:
                owed = self._outstanding_pages()      # includes what this step has promised
            todo = len(req.all_tokens) - req.computed
            # The whole prompt plus one page of decoding (the request's whole life, if that is less) must fit in
            # what is free once the running requests have brought in all they still have to: a prompt that is
            # cut into portions takes its pages over several steps, and two prompts admitted on the strength of
            # the same free pages would starve each other.
            need_pages = self._admission_pages(req)
            ok = all(windowed[g] or need_pages + owed[g] <= self.cache.n_free(g) for g in range(len(promised)))
            if not ok:
                break
            try:
                self._admit(req.rid)
            except OutOfSlots:
                break
            self.waiting.popleft()
            self.running.append(req)
            for g, k in enumerate(self.cache.pages_to_reserve(req.rid, todo)):
                owed[g] += k
            budget -= self._schedule_portion(req, budget, batch, fits, promise)
        return batch

    def _schedule_portion(self, req: Request, budget: int, batch, fits, promise) -> int:
        todo = req.all_tokens[req.computed:]
        n = min(len(todo), budget, self.prefill_chunk)
        if n > 0 and not fits(req, n):               # the largest portion the free pages can take
            lo, hi = 0, n                             # fits(lo) holds (0 tokens need nothing), fits(hi) does not
            while hi - lo > 1:
                mid = (lo + hi) // 2
                if fits(req, mid):
                    lo = mid
                else:
                    hi = mid
            n = lo
        if n <= 0:
            return 0
        last = n == len(todo)
        batch.append(Scheduled(req, todo[:n], last))
        promise(req, n)
        return n

    # ---------------------------------------------------------------- the step after the one in flight
    def lookahead(self, batch: Sequence[Scheduled]) -> Optional[List[Scheduled]]:
        """The batch ``schedule`` would build after ``advance(batch, ...)``, if that can be said before the
        tokens of ``batch`` are known: nobody waits, every running request samples in ``batch`` (so all of
        them decode next), and the pages for one more token each are free.  Requests that end with ``batch`` by
        length are left out; one that ends by an end-of-sequence token is only found out afterwards, and the
        engine drops its row.  The tokens are placeholders (-1): the device feeds the ids it chose.  None when
        the next step has to wait for ``advance``."""
        if self.waiting or not batch or len(batch) != len(self.running):
            return None
        if any(not s.samples for s in batch) or {id(s.request) for s in batch} != {id(r) for r in self.running}:
            return None
        by_req = {id(s.request): s for s in batch}
        promised = [0] * len(self.cache.groups)
        out: List[Scheduled] = []
        for req in self.running:
            s = by_req[id(req)]
            if req.computed + len(s.tokens) != len(req.prompt) + len(req.generated):
                return None                                   # not its newest token: it will still be prefilling
            n_gen = len(req.generated) + 1
            if n_gen >= req.max_new_tokens or len(req.prompt) + n_gen >= self.max_positions:
                continue                                      # ends with the step in flight
            need = self.cache.pages_to_reserve(req.rid, 1)
            if any(need[g] + promised[g] > self.cache.n_free(g) for g in range(len(need))):
                return None                                   # pages run out: schedule() decides who yields
            for g, k in enumerate(need):
                promised[g] += k
            out.append(Scheduled(req, [-1], True))
        if not out or len(out) > self.max_batch_tokens:
            return None
        return out

    # ---------------------------------------------------------------- after the step
    def advance(self, batch: Sequence[Scheduled], new_tokens: Dict[Hashable, int]) -> List[Request]:
        """Records what the step computed and the tokens it chose; returns requests that finished
        (their pages are given back here)."""
        done = []
        for s in batch:
            req = s.request
            req.computed += len(s.tokens)
            if s.samples:
                t = int(new_tokens[req.rid])
                if t in req.eos_ids:
                    req.finished, req.finish_reason = True, "eos"
                else:
                    req.generated.append(t)
                    if len(req.generated) >= req.max_new_tokens:
                        req.finished, req.finish_reason = True, "length"
                    elif len(req.prompt) + len(req.generated) >= self.max_positions:
                        req.finished, req.finish_reason = True, "context"
            if req.finished:
                self.running.remove(req)
                self._release(req.rid)
                done.append(req)
        self.step_index += 1
        return done
