"""Continuous batching above the step function.

The decisions are those of 7QiC/ccInfer's scheduler
(src/scheduler/scheduler.cpp:398-598): requests are admitted first come first
served; a step is built under a token budget (4096) and the free pages of the
cache; requests that are decoding come first, one token each; then portions of
prompts, at most ``prefill_chunk_size`` tokens (0 = whole prompts), shrunk to
what the free pages hold; a new prompt starts only while fewer than
``max_running`` requests have started; whoever ran goes to the back of the
order (round robin).  The first new token comes from a prompt's last portion.
A request ends at ``max_tokens`` or at the engine's longest context (the
reference never stops at an end-of-sequence token, src/model/model_runner.h:242;
here ``eos_token_id`` may be given and is off by default).

When pages run out (src/scheduler/scheduler.cpp:225-268, 811-845) the
reference suspends every blocked request and replays it; here ONE request is
preempted, the one that started last, so that older requests keep going: all
its pages are given back, its prompt becomes ``prompt + generated[:-1]`` and is
computed again without sampling, then decoding goes on from its last token.
Because a request's draw depends only on (seed, number of tokens it has
produced), a preempted request produces the same tokens as an undisturbed
one.

Unlike the reference (one SamplingParams per batch, requests that differ are
skipped, :489-498), every request keeps its own parameters and greedy and
temperature requests share a step.

Running ahead (``run_ahead=True``; the reference's loop waits for every step,
src/scheduler/scheduler.cpp:206-284): a step is launched before the tokens of
the step before it have been read.  A decoding request's entry then names the
token by ``PENDING``; the engine finds it on the device, where the sampling
kernel left it.  Everything that decides a step is known without the tokens
(lengths, pages, how many tokens a request has produced), except an
end-of-sequence stop: a request that stops that way has one more step in
flight, whose token is dropped.  The events of a step are returned by the
call after it; before a preemption or a cancellation the step in flight is
read first, so those never see a token that is still on the device.

The scheduler only needs of its engine: ``open_request``, ``close_request``,
``step(entries) -> logits``, ``sample(logits, params, out_index) -> tokens``,
``cache`` (a CacheManager) and ``max_context``; tests drive it with a fake.
Running ahead also needs ``sample_async(...) -> object with tokens()``.
"""
from __future__ import annotations

import collections
import dataclasses
from typing import Dict, Hashable, List, Optional, Sequence

from ..errors import InvalidArgument, KVBlockExhausted, RequestTooLong
from ..sampling.params import SamplingParams

PENDING = -1   # engine.PENDING: in place of a token that the sampling kernel left on the device


@dataclasses.dataclass
class ScheduledItem:
    req_id: Hashable
    tokens: List[int]
    sample: bool            # a new token is drawn from the last position
    kind: str               # "decode" or "prefill"


@dataclasses.dataclass
class TokenEvent:
    req_id: Hashable
    token: Optional[int]
    finished: bool
    reason: Optional[str] = None   # "max_tokens", "max_context", "eos", "cancelled"


class _Request:
    def __init__(self, req_id, prompt, params: SamplingParams):
        self.req_id = req_id
        self.initial_prompt = list(prompt)
        self.prompt = list(prompt)          # what has to be in the cache before decoding (grows on preemption)
        self.params = params
        self.generated: List[int] = []
        self.cursor = 0                     # tokens of ``prompt`` already cached
        self.opened = False                 # holds a slot in the engine
        self.started_at = -1                # order of first scheduling (for the preemption victim)
        self.replaying = False              # the prompt's last portion does not sample
        self.finished = False
        self.pending = 0                    # tokens drawn in a step whose results have not been read yet

    @property
    def n_out(self) -> int:
        """Tokens produced so far, those still on the device included."""
        return len(self.generated) + self.pending

    @property
    def prefill_done(self) -> bool:
        return self.cursor >= len(self.prompt)


class Scheduler:
    def __init__(self, engine, prefill_chunk_size: int = 512, max_tokens_per_step: int = 4096,
                 max_running: int = 16, eos_token_id: Optional[int] = None, run_ahead: bool = False):
        if prefill_chunk_size < 0 or max_tokens_per_step <= 0 or max_running <= 0:
            raise InvalidArgument("prefill_chunk_size >= 0, max_tokens_per_step > 0, max_running > 0")
        self.engine = engine
        self.prefill_chunk_size = prefill_chunk_size
        self.max_tokens_per_step = max_tokens_per_step
        self.max_running = max_running
        self.eos_token_id = eos_token_id
        self.waiting: collections.deque = collections.deque()
        self.active: Dict[Hashable, _Request] = {}
        self.order: List[Hashable] = []       # round-robin order of active requests
        self._start_counter = 0
        self.preemptions = 0
        self.steps = 0
        self.run_ahead = bool(run_ahead)
        self._inflight = None                 # (items, requests that sample, SampledTokens) of the step not yet read
        self._carry: List[TokenEvent] = []    # events read outside step(), returned by the next call

    # -- requests ---------------------------------------------------------------------
    def submit(self, req_id: Hashable, prompt: Sequence[int], params: SamplingParams = None) -> None:
        params = params or SamplingParams()
        params.validate()
        if req_id in self.active or any(r.req_id == req_id for r in self.waiting):
            raise InvalidArgument(f"request {req_id!r} is already known")
        if len(prompt) == 0:
            raise InvalidArgument("a prompt needs at least one token")
        if any((not isinstance(t, int)) or t < 0 for t in prompt):
            raise InvalidArgument("token ids are non-negative integers")
        if len(prompt) > self.engine.max_context:
            raise RequestTooLong(f"a prompt of {len(prompt)} tokens exceeds the longest context "
                                 f"{self.engine.max_context}")
        # a group that keeps every token must be able to hold the prompt (a window group gives pages back as the
        # request moves on: its pool bounds the size of a portion, not the length of a prompt)
        pool_tokens = min((g.num_pages * g.page_size for g in self.engine.cache.groups if g.window is None),
                          default=None)
        if pool_tokens is not None and len(prompt) > pool_tokens:
            raise RequestTooLong(f"a prompt of {len(prompt)} tokens can never fit the cache pool of "
                                 f"{pool_tokens} tokens")
        self.waiting.append(_Request(req_id, prompt, params))

    def cancel(self, req_id: Hashable) -> bool:
        for r in list(self.waiting):
            if r.req_id == req_id:
                self.waiting.remove(r)
                return True
        if req_id in self.active:
            self._resolve(self._carry)  # its last token may still be on the device
        r = self.active.get(req_id)
        if r is None:
            return False
        self._retire(r)
        return True

    def has_work(self) -> bool:
        return bool(self.waiting or self.active or self._inflight is not None or self._carry)

    # -- building a step ------------------------------------------------------------------
    def _admit(self, events: List[TokenEvent]) -> None:
        """Moves waiting requests into the active set while slots are free (first come first served)."""
        while self.waiting and self.engine.cache.slots.free_slots > 0:
            r = self.waiting.popleft()
            if r.params.max_tokens <= 0:  # finished at once (src/scheduler/scheduler.cpp:309-314)
                events.append(TokenEvent(r.req_id, None, True, "max_tokens"))
                continue
            self.engine.open_request(r.req_id)
            r.opened = True
            self.active[r.req_id] = r
            self.order.append(r.req_id)

    def plan(self) -> List[ScheduledItem]:
        """Decides the next step; changes nothing but the running order bookkeeping of starts."""
        cache = self.engine.cache
        free = [p.free_pages for p in cache.pools]
        budget = self.max_tokens_per_step
        items: List[ScheduledItem] = []
        self._blocked: List[Hashable] = []

        def fits(need):
            return all(n <= f for n, f in zip(need, free))

        def take(need):
            for g, n in enumerate(need):
                free[g] -= n

        # decoding requests first, one token each
        for rid in self.order:
            r = self.active[rid]
            if not r.prefill_done or budget <= 0:
                continue
            if r.pending and (r.n_out >= r.params.max_tokens or cache.get(rid).ctx_len + 1 > self.engine.max_context):
                continue  # it ends when its token has been read
            need = cache.pages_needed(rid, 1)
            if not fits(need):
                self._blocked.append(rid)
                continue
            take(need)
            budget -= 1
            items.append(ScheduledItem(rid, [PENDING if r.pending else r.generated[-1]], True, "decode"))
        # then portions of prompts
        started = sum(1 for r in self.active.values() if r.started_at >= 0)
        for rid in self.order:
            r = self.active[rid]
            if r.prefill_done or budget <= 0:
                continue
            if r.started_at < 0 and started >= self.max_running:
                continue
            remaining = len(r.prompt) - r.cursor
            n = remaining if self.prefill_chunk_size == 0 else min(remaining, self.prefill_chunk_size)
            n = min(n, budget)
            need = cache.pages_needed(rid, n)
            if not fits(need):
                n = self._largest_fit(rid, n, free)
                if n <= 0:
                    self._blocked.append(rid)
                    continue
                need = cache.pages_needed(rid, n)
            take(need)
            budget -= n
            last = r.cursor + n >= len(r.prompt)
            items.append(ScheduledItem(rid, r.prompt[r.cursor:r.cursor + n], last and not r.replaying, "prefill"))
            if r.started_at < 0:
                r.started_at = self._start_counter
                self._start_counter += 1
                started += 1
        return items

    def _largest_fit(self, rid, n, free) -> int:
        """The most tokens (<= n) of a portion whose pages fit what is free in every group."""
        cache = self.engine.cache
        rc = cache.get(rid)
        best = n
        for g, spec in enumerate(cache.groups):
            room = (rc.table_len(g) + free[g]) * spec.page_size - rc.ctx_len
            best = min(best, room)
        return max(0, best)

    def _preempt_one(self) -> bool:
        """Frees the pages of the request that started last (it will be computed again); False if none can be."""
        assert self._inflight is None  # step() reads the step in flight before it gets here
        victims = [r for r in self.active.values() if r.started_at >= 0 and self.engine.cache.get(r.req_id).ctx_len > 0]
        if len(victims) <= 1 and not self._blocked_other_than(victims):
            return False
        if not victims:
            return False
        v = max(victims, key=lambda r: r.started_at)
        self.engine.close_request(v.req_id)
        self.engine.open_request(v.req_id)
        if v.generated:
            v.prompt = v.initial_prompt + v.generated[:-1]
            v.replaying = True
        v.cursor = 0
        v.started_at = -1
        # it queues behind the others
        self.order.remove(v.req_id)
        self.order.append(v.req_id)
        self.preemptions += 1
        return True

    def _blocked_other_than(self, victims) -> bool:
        ids = {v.req_id for v in victims}
        return any(b not in ids for b in self._blocked)

    # -- running a step ----------------------------------------------------------------------
    def step(self) -> List[TokenEvent]:
        """Admits, builds and runs one step; returns the tokens it produced and the requests it ended.

        When running ahead, the tokens are those of the step before (this call launches its step first
        and then reads the earlier one)."""
        events: List[TokenEvent] = self._carry
        self._carry = []
        self._admit(events)
        self._finish_exhausted(events)
        items = self.plan() if self.active else []
        if not items and self._inflight is not None:
            # nothing to launch before the tokens in flight are known (requests at their last token, or
            # pages that only an ending request gives back)
            self._resolve(events)
            self._admit(events)
            self._finish_exhausted(events)
            items = self.plan() if self.active else []
        if not self.active:
            return events
        guard = 0
        while not items:
            # nothing fits: give one request's pages to the others, or fail if there is nothing to give
            guard += 1
            if guard > len(self.active) + 1 or not self._preempt_one():
                raise KVBlockExhausted("no request can make progress: the cache pool is too small for "
                                       "the requests that are running")
            items = self.plan()
        from .engine import StepEntry
        entries = [StepEntry(it.req_id, it.tokens, [len(it.tokens) - 1] if it.sample else []) for it in items]
        logits = self.engine.step(entries)
        reqs = [self.active[it.req_id] for it in items if it.sample]
        handle = None
        if reqs:
            args = (logits, [r.params for r in reqs], [r.n_out for r in reqs])
            handle = self.engine.sample_async(*args) if self.run_ahead else _Now(self.engine.sample(*args))
        self.steps += 1
        # what is known at launch
        ran = []
        for it in items:
            r = self.active[it.req_id]
            ran.append(it.req_id)
            if it.kind == "prefill":
                r.cursor += len(it.tokens)
                if r.prefill_done and r.replaying:
                    r.replaying = False  # decoding goes on from the token it already has
            if it.sample:
                r.pending += 1
        # whoever ran goes to the back (src/scheduler/scheduler.cpp:600-615)
        keep = [rid for rid in self.order if rid not in ran]
        self.order = keep + ran
        previous, self._inflight = self._inflight, ((reqs, handle) if reqs else None)
        if previous is not None:
            self._read(previous, events)
        if not self.run_ahead:
            self._resolve(events)
        return events

    def _resolve(self, events: List[TokenEvent]) -> None:
        """Reads the tokens of the step in flight, if there is one."""
        previous, self._inflight = self._inflight, None
        if previous is not None:
            self._read(previous, events)

    def _read(self, record, events: List[TokenEvent]) -> None:
        reqs, handle = record
        for r, tok in zip(reqs, handle.tokens()):
            if r.finished:
                continue  # it ended while this step was in flight; the token is dropped
            tok = int(tok)
            r.pending -= 1
            r.generated.append(tok)
            reason = None
            if len(r.generated) >= r.params.max_tokens:
                reason = "max_tokens"
            elif self.eos_token_id is not None and tok == self.eos_token_id:
                reason = "eos"
            events.append(TokenEvent(r.req_id, tok, reason is not None, reason))
            if reason:
                self._retire(r)

    def _finish_exhausted(self, events: List[TokenEvent]) -> None:
        """A request whose next token would not fit the longest context ends (src/scheduler/scheduler.cpp:477-481)."""
        for r in list(self.active.values()):
            if r.pending:
                continue  # after its token has been read
            if r.prefill_done and self.engine.cache.get(r.req_id).ctx_len + 1 > self.engine.max_context:
                events.append(TokenEvent(r.req_id, None, True, "max_context"))
                self._retire(r)

    def _retire(self, r: _Request) -> None:
        r.finished = True
        if r.opened:
            self.engine.close_request(r.req_id)
            r.opened = False
        self.active.pop(r.req_id, None)
        if r.req_id in self.order:
            self.order.remove(r.req_id)

    def drain(self) -> List[TokenEvent]:
        """Reads what is still in flight; the events that step() has not returned yet."""
        events, self._carry = self._carry, []
        self._resolve(events)
        return events

    def run(self) -> Dict[Hashable, List[int]]:
        """Steps until nothing is left; returns the new tokens of every request."""
        out: Dict[Hashable, List[int]] = {}
        while self.has_work():
            for ev in self.step():
                out.setdefault(ev.req_id, [])
                if ev.token is not None:
                    out[ev.req_id].append(ev.token)
        return out


class _Now:
    """Tokens that are already on the host, with the interface of the engine's asynchronous result."""

    def __init__(self, tokens):
        self._tokens = tokens

    def tokens(self):
        return self._tokens
