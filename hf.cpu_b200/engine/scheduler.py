"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes, finishes.

The reference serves one request at a time (src/main.c:54-153): it prefills in steps of ``--batch``
tokens asking for logits only at the last portion (src/ops.c:788-795), then samples, checks the stop
conditions and feeds the token back (src/ops.c:827-893).  The same order of operations holds per
request here, for many requests at once:

* every running request that is decoding gets its one token first; decodes never wait behind prompts;
* what is left of the token budget goes to portions of prompts, oldest request first; waiting requests
  are admitted first come first served while a slot is free and pages for their first portion exist;
* when pages run out, portions of prompts are dropped from the step first; if the decodes alone do not
  fit, the most recently admitted running request is preempted: its pages go back, it keeps the tokens
  it generated and its generator state, and it returns to the head of the waiting queue to be
  recomputed as prompt + generated tokens, so the tokens it samples do not change;
* a request that cannot fit even alone fails with ENOMEM, and only that request;
* a request whose first tokens are those of a running request starts on that request's full cache pages and
  computes only the rest (the reference forks the context of a prompt for its ``--n`` continuations,
  src/ops.c:808-825); while the other is still computing the tokens they share, it waits for them.  With
  ``keep_cache`` a finished request's pages are kept until the next request has had the chance to start on them
  (``--prefix-cache``, src/ops.c:771-776); they are the first to go when pages or slots are short.

While every running request decodes and none is about to reach its limit, ``run`` keeps one step ahead of
the host: the next step is launched with the token ids the sampling kernel has just written on the device,
before the host has read them, so that planning, the copies and the events of one step hide behind the GPU's
work on the next.  A request that turns out to have ended (an end token) has run one token too far; that
token is dropped.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache import OutOfPages
from ..sampling import Rng, SamplingParams, logprob, sample_host, top_logprobs
from .step import Engine, StepEntry

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


class RequestError(ValueError):
    """A request is refused at submission; ``code`` is the reference's status name."""

    def __init__(self, code: str, msg: str):
        super().__init__(msg)
        self.code = code


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    eos_ids: Sequence[int] = ()
    timeout: float = 0.0
    # state
    status: str = WAITING
    generated: List[int] = field(default_factory=list)
    computed: int = 0                  # tokens of prompt + generated that are in the cache
    budget: int = 0                    # generation limit after clipping to the context
    stop: Optional[str] = None         # eos | length | ctx | timeout | cancel | error
    error: Optional[str] = None
    limit_reason: str = "length"
    rng: Optional[Rng] = None
    arrival: int = 0
    preemptions: int = 0
    t_submit: float = 0.0
    t_first: float = 0.0
    t_done: float = 0.0
    logprobs: List = field(default_factory=list)
    keep_cache: bool = False           # when it ends, its pages stay until the next request could start on them
    reuse_cache: bool = True           # it may start on pages kept of a finished request
    shared: int = 0                    # tokens it did not compute: it started on another request's pages

    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    def token_slice(self, a: int, b: int) -> List[int]:
        """Tokens a..b-1 of prompt + generated, without building the whole list."""
        n = len(self.prompt)
        if a >= n:
            return self.generated[a - n:b - n]
        if b <= n:
            return self.prompt[a:b]
        return self.prompt[a:] + self.generated[:b - n]

    @property
    def pending(self) -> int:
        """Tokens that still have to run before the next token can be sampled."""
        return len(self.prompt) + len(self.generated) - self.computed


@dataclass
class TokenEvent:
    req: Hashable
    pos: int                           # index among the request's generated tokens
    token: int
    logprob: Optional[float] = None
    top: Optional[list] = None


@dataclass
class FinishEvent:
    req: Hashable
    stop: str
    error: Optional[str] = None


@dataclass
class Flight:
    """A step that has been launched and whose sampled tokens have not been read yet."""
    sampled: List["Request"]
    logits: Optional[torch.Tensor]
    pending: object = None             # sampling.device.Pending, or None when the tokens are in ``tokens`` already
    tokens: Optional[list] = None
    rows: Optional[np.ndarray] = None


@dataclass
class StepPlan:
    entries: List[StepEntry]
    requests: List[Request]
    preempted: List[Request]
    admitted: List[Request]
    failed: List[Request]


class Scheduler:
    def __init__(self, engine: Engine, max_num_seqs: int = 0, max_num_batched_tokens: int = 2048,
                 prefill_chunk: int = 0, device_sampling: bool = True, share_prefixes: bool = True):
        self.engine = engine
        self.max_num_seqs = min(max_num_seqs or engine.max_requests, engine.max_requests)
        self.max_num_batched_tokens = int(max_num_batched_tokens)
        self.prefill_chunk = int(prefill_chunk) if prefill_chunk else self.max_num_batched_tokens
        self.device_sampling = device_sampling and engine.device.type == "cuda"
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.requests: Dict[Hashable, Request] = {}
        self._arrivals = 0
        self.stats = {"steps": 0, "preemptions": 0, "tokens_in": 0, "tokens_out": 0, "finished": 0, "errors": 0,
                      "steps_ahead": 0, "tokens_shared": 0}
        self.share_prefixes = share_prefixes
        self.retained: Optional[Request] = None          # a finished request whose pages are kept (keep_cache)
        self.cancelled = set()
        self.run_ahead = self.device_sampling            # run() launches steady decode steps one ahead of the host
        self._host_ring = None                           # pinned buffers the sampled ids are copied into
        self._ring_at = 0

    # ---- submission ---------------------------------------------------------------------------
    def submit(self, req: Request) -> None:
        """Checks as the reference's: a prompt must be non-empty and shorter than the context limit
        (src/ops.c:752-756); ``max_tokens`` is clipped to the room left, stop reason ``ctx`` (src/ops.c:757-758)."""
        if req.id in self.requests and self.requests[req.id].status != FINISHED:
            raise RequestError("EINVAL", f"request id {req.id!r} is already in use")
        if self.retained is not None and self.retained.id == req.id:
            self.drop_retained()
        req.params.validate()
        V = self.engine.model.plan.vocab_size
        if len(req.prompt) == 0:
            raise RequestError("EINVAL", "empty prompt")
        for t in req.prompt:
            if not 0 <= int(t) < V:
                raise RequestError("EINVAL", f"token id {t} is outside the vocabulary of {V}")
        if len(req.prompt) >= self.engine.ctx_max:
            raise RequestError("ERANGE", f"prompt has {len(req.prompt)} tokens but --ctx-max is {self.engine.ctx_max}")
        req.budget = req.params.max_tokens
        if req.budget > self.engine.ctx_max - len(req.prompt):
            req.budget, req.limit_reason = self.engine.ctx_max - len(req.prompt), "ctx"
        req.rng = Rng(req.params.seed)
        req.status, req.arrival, req.t_submit = WAITING, self._arrivals, time.perf_counter()
        self._arrivals += 1
        self.requests[req.id] = req
        self.waiting.append(req)

    def cancel(self, req_id) -> None:
        self.cancelled.add(req_id)

    def abort(self, req_ids, why: str = "EIO: the step failed") -> list:
        """Ends the named requests at once, running or waiting, and gives back what they hold: for a caller whose
        step raised, so that nothing of the failed call is left to be scheduled with the next one."""
        events: list = []
        for rid in req_ids:
            r = self.requests.get(rid)
            if r is not None and r.status != FINISHED:
                self._finish(r, "error", events, why)
            self.cancelled.discard(rid)
        return events

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- planning a step ------------------------------------------------------------------------
    def _preempt(self, req: Request) -> None:
        self.engine.finish_request(req.id)
        self.running.remove(req)
        req.status, req.computed, req.shared = WAITING, 0, 0
        req.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(req)

    def plan(self) -> StepPlan:
        preempted: List[Request] = []
        failed: List[Request] = []
        if not self.waiting and self.running and len(self.running) <= self.max_num_batched_tokens \
                and all(r.pending == 1 and r.computed > 0 for r in self.running) \
                and self.engine.cache.can_reserve([(r.id, r.computed + 1) for r in self.running]):
            # the steady state: everyone decodes, nobody waits, the pages are there
            entries = [StepEntry(r.id, r.token_slice(r.computed, r.computed + 1), [0]) for r in self.running]
            return StepPlan(entries, list(self.running), preempted, [], failed)
        while True:
            chosen, admitted = self._choose(preempted, failed)
            if chosen or not self.running:
                break
            if self.drop_retained():
                continue
            # running requests exist but nothing can move: every page is held by requests that all need more
            victim = max(self.running, key=lambda r: r.arrival)
            if len(self.running) == 1:
                failed.append(victim)
                self.running.remove(victim)
                self.engine.finish_request(victim.id)
            else:
                self._preempt(victim)
                preempted.append(victim)
        entries, reqs = [], []
        for r, n in chosen:
            toks = r.token_slice(r.computed, r.computed + n)
            last = r.computed + n == len(r.prompt) + len(r.generated)
            entries.append(StepEntry(r.id, toks, [n - 1] if last else []))
            reqs.append(r)
        return StepPlan(entries, reqs, preempted, admitted, failed)

    def _choose(self, preempted: List[Request], failed: List[Request]):
        cache = self.engine.cache
        # 1. decodes: one token for every running request with a single pending token
        decodes = [r for r in self.running if r.pending == 1 and r.computed > 0]
        while decodes and not cache.can_reserve([(r.id, r.computed + 1) for r in decodes]):
            if self.drop_retained():
                continue
            victim = max(self.running, key=lambda r: r.arrival)
            if len(self.running) == 1:
                # alone and still short of pages: the pool cannot hold this request at all
                failed.append(victim)
                self.running.remove(victim)
                self.engine.finish_request(victim.id)
                decodes = []
                break
            self._preempt(victim)
            preempted.append(victim)
            decodes = [r for r in decodes if r is not victim]
        chosen = [(r, 1) for r in decodes]
        budget = self.max_num_batched_tokens - len(chosen)
        wants = [(r.id, r.computed + 1) for r in decodes]

        def fit_portion(r: Request) -> int:
            """The largest portion of r's pending tokens that the budget and the free pages allow."""
            hi = min(r.pending, budget, self.prefill_chunk)
            if hi <= 0 or not cache.can_reserve(wants + [(r.id, r.computed + 1)]):
                return 0
            lo = 1                          # lo always fits; more tokens never need fewer pages
            while lo < hi:
                mid = (lo + hi + 1) // 2
                if cache.can_reserve(wants + [(r.id, r.computed + mid)]):
                    lo = mid
                else:
                    hi = mid - 1
            return lo

        # 2. portions of prompts of running requests, oldest first
        for r in sorted(self.running, key=lambda r: r.arrival):
            if budget <= 0:
                break
            if r in decodes or r.pending == 0:
                continue
            n = fit_portion(r)
            if n > 0:
                chosen.append((r, n))
                wants.append((r.id, r.computed + n))
                budget -= n
        # 3. admit waiting requests, first come first served
        admitted: List[Request] = []
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            if self.engine.slots.free_count == 0 and not self.drop_retained():
                break
            r = self.waiting[0]
            if r in preempted:
                break                      # do not bring back in the same step what was just put out
            donor, share, later = self._donor(r)
            if later > share:
                break                      # a running request is still computing tokens this one can start on
            self.engine.add_request(r.id)
            if share:
                share = self.engine.fork_request(donor.id, r.id, share)
            r.computed = r.shared = share
            n = fit_portion(r)
            if n == 0:
                self.engine.finish_request(r.id)
                r.computed = r.shared = 0
                if self.drop_retained():
                    continue
                if not self.running and not chosen:
                    # nothing else holds pages and not even one token fits
                    failed.append(self.waiting.popleft())
                    continue
                break
            self.waiting.popleft()
            if self.retained is not None:
                self.drop_retained()       # the request it was kept for has started, on it or not
            self.stats["tokens_shared"] += share
            r.status = RUNNING
            self.running.append(r)
            admitted.append(r)
            chosen.append((r, n))
            wants.append((r.id, r.computed + n))
            budget -= n
        return chosen, admitted

    # ---- starting on another request's pages ------------------------------------------------------------
    @staticmethod
    def _common(a: List[int], b: List[int], limit: int) -> int:
        """How many of the first ``limit`` tokens of a and b are the same."""
        limit = min(limit, len(a), len(b))
        n = 0
        while n < limit:                   # whole slices first (compared at C speed), then the slice that differs
            m = min(n + 512, limit)
            if a[n:m] == b[n:m]:
                n = m
                continue
            while a[n] == b[n]:
                n += 1
            break
        return n

    def _donor(self, r: Request):
        """The request whose cache ``r`` can best start on: (donor, tokens shareable now, tokens shareable once
        a running donor has computed what it has in common with r).  Whole blocks only, and never r's last
        token: r has to run that one itself to have its logits."""
        if not self.share_prefixes or r.computed or not self.engine.can_fork:
            return None, 0, 0
        bs = self.engine.block_size
        mine = r.tokens()
        cap = (len(mine) - 1) // bs * bs
        if cap <= 0:
            return None, 0, 0
        best, best_now, best_later = None, 0, 0
        for d in self.running + ([self.retained] if self.retained is not None and r.reuse_cache else []):
            if d is r or not self.engine.has_request(d.id):
                continue
            theirs = d.tokens()
            same = min(self._common(mine, theirs, cap), cap) // bs * bs
            now = min(same, d.computed // bs * bs)
            if now > best_now:
                best, best_now = d, now
            if d is not self.retained:
                best_later = max(best_later, same)
        return best, best_now, max(best_later, best_now)

    def drop_retained(self) -> bool:
        """Gives back the pages kept of a finished request; False when there were none."""
        if self.retained is None:
            return False
        self.engine.finish_request(self.retained.id)
        self.retained = None
        return True

    # ---- running a step ---------------------------------------------------------------------------
    def _finish(self, r: Request, stop: str, events: list, error: Optional[str] = None) -> None:
        if r in self.running:
            self.running.remove(r)
            if r.keep_cache and self.share_prefixes and error is None and stop != "cancel":
                self.drop_retained()
                self.retained = r
            else:
                self.engine.finish_request(r.id)
        elif r in self.waiting:
            self.waiting.remove(r)
        r.status, r.stop, r.error, r.t_done = FINISHED, stop, error, time.perf_counter()
        self.stats["finished"] += 1
        if error:
            self.stats["errors"] += 1
        events.append(FinishEvent(r.id, stop, error))

    def step(self) -> list:
        """One scheduling round: plan, run the engine's step, sample, emit events."""
        events, flight = self._begin()
        if flight is not None:
            events += self._end(flight)
        return events

    def _begin(self):
        """Housekeeping, the plan, the engine's step and the launch of the sampling.  Returns the events so far
        and the step in flight (None when nothing was sampled)."""
        events: list = []
        now = time.perf_counter()
        for r in list(self.running) + list(self.waiting):
            if r.id in self.cancelled:
                self.cancelled.discard(r.id)
                self._finish(r, "cancel", events)
            elif r.timeout > 0 and now - r.t_submit > r.timeout:
                if r.generated or r.computed >= len(r.prompt):
                    self._finish(r, "timeout", events)
                else:
                    self._finish(r, "error", events, "ECANCEL: timed out during prefill")
        plan = self.plan()
        for r in plan.failed:
            r.status = FINISHED
            self._finish(r, "error", events, "ENOMEM: the page pool cannot hold this request")
        if not plan.entries:
            return events, None
        logits = self.engine.step(plan.entries)
        self.stats["steps"] += 1
        self.stats["tokens_in"] += sum(len(e.tokens) for e in plan.entries)
        sampled = [r for r, e in zip(plan.requests, plan.entries) if e.want]
        for r, e in zip(plan.requests, plan.entries):
            r.computed += len(e.tokens)
        if not sampled:
            return events, None
        return events, self._launch_sampling(logits, sampled)

    def _launch_sampling(self, logits: torch.Tensor, sampled: List[Request]) -> Flight:
        """On the GPU the sampling kernels run and only token ids come back; the host mirror serves the
        stand-in backend of the tests."""
        if self.device_sampling:
            from .. import sampling
            if self._host_ring is None:
                self._host_ring = [torch.empty(self.engine.max_requests + 1, dtype=torch.int32, pin_memory=True)
                                   for _ in range(4)]
            self._ring_at = (self._ring_at + 1) % len(self._host_ring)
            from .. import kernels
            with kernels.phase("sample"):
                pending = sampling.device.sample_rows_async(logits, sampled, self._host_ring[self._ring_at])
            return Flight(sampled, logits, pending=pending)
        rows = logits.float().cpu().numpy()
        return Flight(sampled, logits, tokens=[sample_host(rows[i], r.params, r.rng) for i, r in enumerate(sampled)], rows=rows)

    def _can_run_ahead(self, flight: Flight) -> bool:
        """True when the step after ``flight`` is known without its tokens: the same requests decode again, nobody
        waits, nobody reaches a limit or a deadline, nobody wants log-probabilities, and the pages are there."""
        if not (self.run_ahead and flight.pending is not None) or self.waiting or self.cancelled:
            return False
        if len(flight.sampled) != len(self.running) or len(self.running) > self.max_num_batched_tokens:
            return False
        for r, q in zip(flight.sampled, self.running):
            if r is not q or r.pending != 0 or r.timeout > 0 or r.params.logprobs > 0 or len(r.generated) + 2 > r.budget:
                return False
        return self.engine.cache.can_reserve([(r.id, r.computed + 1) for r in self.running])

    def _begin_ahead(self, flight: Flight) -> Flight:
        """Launches the next decode step of the requests of ``flight`` on the token ids it is still sampling."""
        entries = [StepEntry(r.id, [0], [0]) for r in flight.sampled]
        logits = self.engine.step(entries, token_source=flight.pending.device)
        self.stats["steps"] += 1
        self.stats["steps_ahead"] += 1
        self.stats["tokens_in"] += len(entries)
        for r in flight.sampled:
            r.computed += 1
        return self._launch_sampling(logits, list(flight.sampled))

    def _end(self, flight: Flight) -> list:
        """Reads the sampled tokens of a step, emits their events and ends the requests that are done."""
        events: list = []
        try:
            tokens = flight.tokens if flight.pending is None else flight.pending.tokens()
        except kernels.DeviceFault as e:
            # a bounded wait ran out or an index was refused on the device: the step's logits are not to be trusted
            for r in flight.sampled:
                if r.status != FINISHED:
                    self._finish(r, "error", events, f"EIO: {e}")
            return events
        for i, r in enumerate(flight.sampled):
            if r.status == FINISHED:
                continue                                  # ended while this step was in flight: its token is dropped
            tok = int(tokens[i])
            if not r.t_first:
                r.t_first = time.perf_counter()
            if tok in r.eos_ids:
                self._finish(r, "eos", events)          # the end token is not emitted (src/ops.c:849)
                continue
            ev = TokenEvent(r.id, len(r.generated), tok)
            if r.params.logprobs > 0:
                row = flight.rows[i] if flight.rows is not None else flight.logits[i].float().cpu().numpy()
                ev.logprob, ev.top = logprob(row, tok), top_logprobs(row, r.params.logprobs)
            r.generated.append(tok)
            self.stats["tokens_out"] += 1
            events.append(ev)
            if len(r.generated) >= r.budget:
                self._finish(r, r.limit_reason, events)
        return events

    def run(self, on_event: Optional[Callable] = None) -> list:
        """Step until every submitted request is finished; returns (and reports) all events."""
        out = []

        def emit(events):
            for ev in events:
                out.append(ev)
                if on_event:
                    on_event(ev)

        flight = None
        while flight is not None or self.has_work():
            if flight is None:
                events, flight = self._begin()
                emit(events)
                if flight is None:
                    continue
            ahead = self._begin_ahead(flight) if self._can_run_ahead(flight) else None
            emit(self._end(flight))
            flight = ahead
        return out
