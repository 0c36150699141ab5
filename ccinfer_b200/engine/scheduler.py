"""Continuous batching above the step function.

The scheduler itself is native: ``csrc/host/scheduler.cpp`` behind the scheduler calls of
``csrc/host/ccinfer.h`` (``ccinfer_add_request``, ``ccinfer_cancel``, ``ccinfer_step``); this class gives it the
package's names, lets requests be named by any hashable id and supplies its hooks: a step is run by
``engine.step`` and sampled by ``engine.sample`` / ``engine.sample_async``.  What it decides:

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

import dataclasses
from typing import Dict, Hashable, List, Optional, Sequence

from ..errors import InvalidArgument
from ..native import SchedulerCore
from ..sampling.params import SamplingParams

PENDING = -1   # engine.PENDING: in place of a token that the sampling kernel left on the device


@dataclasses.dataclass
class TokenEvent:
    req_id: Hashable
    token: Optional[int]
    finished: bool
    reason: Optional[str] = None   # "max_tokens", "max_context", "eos"


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
        self.run_ahead = bool(run_ahead)
        self._number: Dict[Hashable, int] = {}      # the requests the native scheduler knows, by its numbers
        self._name: Dict[int, Hashable] = {}
        self._params: Dict[int, SamplingParams] = {}
        self._next = 1
        self._carry: List[TokenEvent] = []           # events read outside step(), returned by the next call
        self._results: Dict[int, object] = {}        # ticket of a step -> its sampled tokens (maybe still on the way)
        self._core = SchedulerCore(engine.cache.core, prefill_chunk_size, max_tokens_per_step, max_running,
                                   engine.max_context, eos_token_id, run_ahead,
                                   open=self._open, close=self._close, run=self._run, read=self._read)

    # -- hooks of the native scheduler -----------------------------------------------------
    def _open(self, req: int) -> int:
        rid = self._name[req]
        self.engine.open_request(rid)
        return self.engine.cache.get(rid).seq

    def _close(self, req: int) -> None:
        self.engine.close_request(self._name[req])

    def _run(self, plan, ticket: int) -> None:
        from .engine import StepEntry
        entries, params, out_index, at = [], [], [], 0
        for i in range(plan.n_items):
            n, req = plan.counts[i], plan.reqs[i]
            entries.append(StepEntry(self._name[req], plan.tokens[at:at + n], [n - 1] if plan.sample[i] else []))
            at += n
            if plan.sample[i]:
                params.append(self._params[req])
                out_index.append(plan.out_index[i])
        logits = self.engine.step(entries)
        if params:
            args = (logits, params, out_index)
            self._results[ticket] = self.engine.sample_async(*args) if self.run_ahead else _Now(self.engine.sample(*args))

    def _read(self, ticket: int, n: int):
        return self._results.pop(ticket).tokens()

    # -- requests ---------------------------------------------------------------------
    def submit(self, req_id: Hashable, prompt: Sequence[int], params: SamplingParams = None) -> None:
        params = params or SamplingParams()
        params.validate()
        if req_id in self._number:
            raise InvalidArgument(f"request {req_id!r} is already known")
        if any((not isinstance(t, int)) or t < 0 for t in prompt):
            raise InvalidArgument("token ids are non-negative integers")
        req = self._next
        self._core.add_request(req, prompt, params.max_tokens, params.top_k, params.top_p, params.temperature,
                               params.seed)
        self._next += 1
        self._number[req_id], self._name[req], self._params[req] = req, req_id, params

    def _forget(self, req: int) -> None:
        self._number.pop(self._name.pop(req), None)
        self._params.pop(req, None)

    def cancel(self, req_id: Hashable) -> bool:
        req = self._number.get(req_id)
        if req is None:
            return False
        found = self._core.cancel(req)
        self._carry += self._events()   # its token that was in flight has been read (it may have ended there)
        if found:
            self._forget(req)
        return found

    def has_work(self) -> bool:
        return bool(self._carry) or self._core.has_work()

    # -- figures ------------------------------------------------------------------------
    @property
    def steps(self) -> int:
        return self._core.stats().steps

    @property
    def preemptions(self) -> int:
        return self._core.stats().preemptions

    def counts(self) -> dict:
        """How many requests wait, are active, and are active with a prompt that is not yet all in the cache."""
        st = self._core.stats()
        return {"waiting": st.waiting, "active": st.active, "prefilling": st.prefilling}

    def active_ids(self) -> List[Hashable]:
        """The active requests in their running order."""
        return [self._name[req] for req in self._core.active()]

    # -- running ------------------------------------------------------------------------
    def _events(self) -> List[TokenEvent]:
        out = []
        for req, token, finished, reason in self._core.pop_events():
            out.append(TokenEvent(self._name[req], token, finished, reason))
            if finished:
                self._forget(req)
        return out

    def step(self) -> List[TokenEvent]:
        """Admits, builds and runs one step; returns the tokens it produced and the requests it ended.

        When running ahead, the tokens are those of the step before (this call launches its step first
        and then reads the earlier one)."""
        self._core.step()
        events, self._carry = self._carry, []
        return events + self._events()

    def drain(self) -> List[TokenEvent]:
        """Reads what is still in flight; the events that step() has not returned yet."""
        self._core.drain()
        events, self._carry = self._carry, []
        return events + self._events()

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
