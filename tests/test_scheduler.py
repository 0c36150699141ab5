"""The scheduler's decisions (no GPU), driven with a fake engine that has a real cache manager.

The cases follow 7QiC/ccInfer's tests/unit/test_scheduler.cpp: decodes batched, decode before prefill in a
mixed step (:296-329), round robin, 512-token portions (:387-441), the cap on started requests (:443-496),
replay without sampling (:498-548); and add what the reference does not decide: mixed sampling parameters in
one step, and what happens when pages run out.
"""
import hashlib
import os

import pytest

from ccinfer_b200.cache.manager import CacheManager, GroupSpec
from ccinfer_b200.engine.scheduler import Scheduler
from ccinfer_b200.errors import InvalidArgument, KVBlockExhausted, RequestTooLong, Unsupported
from ccinfer_b200.sampling import SamplingParams


class FakeEngine:
    """Logits of a position are a hash of all tokens up to it; a draw depends on (hash, seed, out_index)."""

    def __init__(self, pages=64, page=4, slots=8, max_context=None, window=None):
        groups = [GroupSpec(("all",), None, page, pages)]
        if window:
            groups.append(GroupSpec(("window", window), window, page, pages))
        self.cache = CacheManager(groups, slots)
        self.max_context = max_context or pages * page
        self.history = {}
        self.steps = []
        self.pending = {}        # request -> token drawn by sample_async (what the device would hold)
        self.reads = []          # number of steps launched when each result was read
        self._last_want = []

    def open_request(self, rid):
        self.cache.open(rid)
        self.history[rid] = []

    def close_request(self, rid):
        self.cache.close(rid)
        del self.history[rid]
        self.pending.pop(rid, None)

    def step(self, entries):
        self.steps.append([(e.req_id, list(e.tokens), list(e.want)) for e in entries])
        reserved = []
        try:
            for e in entries:
                self.cache.reserve(e.req_id, len(e.tokens))
                reserved.append(e.req_id)
        except KVBlockExhausted:
            for rid in reserved:
                self.cache.rollback(rid)
            raise
        rows = []
        self._last_want = [e.req_id for e in entries for _ in e.want]
        for e in entries:
            self.cache.commit(e.req_id)
            h = self.history[e.req_id]
            for i, t in enumerate(e.tokens):
                if t == -1:  # PENDING: the token of the request's last sample_async
                    assert len(e.tokens) == 1
                    t = self.pending[e.req_id]
                h.append(t)
                if i in e.want:
                    rows.append(hashlib.sha256(repr(h).encode()).hexdigest())
        self.cache.check_consistency()
        return _Rows(rows)

    def sample(self, logits, params, out_index):
        out = []
        for row, p, i in zip(logits.rows, params, out_index):
            key = row if p.temperature <= 0 else f"{row}:{p.seed}:{i}:{p.temperature}"
            out.append(int(hashlib.sha256(key.encode()).hexdigest(), 16) % 1000)
        return out


    def sample_async(self, logits, params, out_index):
        tokens = self.sample(logits, params, out_index)
        for rid, t in zip(self._last_want, tokens):
            self.pending[rid] = t
        return _Later(self, tokens)


class _Later:
    def __init__(self, eng, tokens):
        self._eng, self._tokens = eng, tokens

    def tokens(self):
        self._eng.reads.append(len(self._eng.steps))
        return self._tokens


class _Rows:
    def __init__(self, rows):
        self.rows = rows
        self.shape = (len(rows), 1000)


def _prompt(n, base=0):
    return [(base + 7 * i) % 997 for i in range(n)]


def test_decodes_are_batched_and_come_first():
    eng = FakeEngine()
    s = Scheduler(eng, prefill_chunk_size=8)
    s.submit("a", _prompt(5), SamplingParams(max_tokens=4))
    s.submit("b", _prompt(6, 100), SamplingParams(max_tokens=4))
    s.step()  # both prompts whole
    assert [(rid, len(t)) for rid, t, _ in eng.steps[-1]] == [("a", 5), ("b", 6)]
    s.submit("c", _prompt(20, 200), SamplingParams(max_tokens=2))
    s.step()
    kinds = [(rid, len(t), w) for rid, t, w in eng.steps[-1]]
    assert kinds == [("a", 1, [0]), ("b", 1, [0]), ("c", 8, [])]  # decodes first, then a portion without logits
    s.step()
    s.step()
    assert eng.steps[-1][-1] == ("c", _prompt(20, 200)[16:], [3])  # the last portion wants its last position


def test_portions_and_token_budget():
    eng = FakeEngine(pages=1024, page=16)
    s = Scheduler(eng, prefill_chunk_size=512, max_tokens_per_step=600)
    s.submit("a", _prompt(1100), SamplingParams(max_tokens=1))
    s.submit("b", _prompt(300, 5), SamplingParams(max_tokens=1))
    s.step()
    assert [(rid, len(t)) for rid, t, _ in eng.steps[-1]] == [("a", 512), ("b", 88)]  # 600 in all
    s.step()
    assert [(rid, len(t)) for rid, t, _ in eng.steps[-1]] == [("a", 512), ("b", 88)]
    whole = Scheduler(FakeEngine(pages=1024, page=16), prefill_chunk_size=0)
    whole.submit("a", _prompt(1100), SamplingParams(max_tokens=1))
    whole.step()
    assert len(whole.engine.steps[-1][0][1]) == 1100  # 0 = whole prompts


def test_round_robin_when_the_budget_is_short():
    eng = FakeEngine(pages=256, page=16)
    s = Scheduler(eng, prefill_chunk_size=16, max_tokens_per_step=16)
    for i in range(3):
        s.submit(f"r{i}", _prompt(40, i), SamplingParams(max_tokens=1))
    ran = []
    for _ in range(6):
        s.step()
        ran.append(eng.steps[-1][0][0])
    assert ran == ["r0", "r1", "r2", "r0", "r1", "r2"]


def test_cap_on_started_requests():
    eng = FakeEngine(pages=512, page=4, slots=8)
    s = Scheduler(eng, prefill_chunk_size=4, max_running=2)
    for i in range(4):
        s.submit(f"r{i}", _prompt(10, i), SamplingParams(max_tokens=3))
    s.step()
    assert [rid for rid, _, _ in eng.steps[-1]] == ["r0", "r1"]  # two started; the others wait their turn
    out = s.run()
    assert sorted(out) == ["r0", "r1", "r2", "r3"] and all(len(v) == 3 for v in out.values())


def test_max_tokens_context_limit_eos_and_cancel():
    eng = FakeEngine(pages=8, page=4, max_context=12)
    s = Scheduler(eng)
    s.submit("zero", _prompt(3), SamplingParams(max_tokens=0))
    s.submit("long", _prompt(10), SamplingParams(max_tokens=50))
    ev = s.step()
    assert ev[0].req_id == "zero" and ev[0].finished and ev[0].token is None
    events = list(ev)
    while s.has_work():
        events += s.step()
    toks = [e.token for e in events if e.req_id == "long" and e.token is not None]
    assert len(toks) == 3  # contexts 10, 11 and 12 gave a token each; a 13th position does not exist
    assert events[-1].finished and events[-1].reason == "max_context"
    assert eng.cache.stats()["groups"][0]["pages_used"] == 0
    with pytest.raises(RequestTooLong):
        s.submit("huge", _prompt(13))
    with pytest.raises(InvalidArgument):
        s.submit("empty", [])
    with pytest.raises(InvalidArgument):
        s.submit("neg", [1, -2])
    with pytest.raises(Unsupported):
        s.submit("topk", _prompt(3), SamplingParams(top_k=-1))
    with pytest.raises(Unsupported):
        s.submit("topp", _prompt(3), SamplingParams(top_p=0.0))
    s.submit("x", _prompt(4), SamplingParams(max_tokens=30))
    s.step()
    with pytest.raises(InvalidArgument):
        s.submit("x", _prompt(4))
    assert s.cancel("x") and not s.cancel("x") and not s.has_work()
    assert eng.cache.stats()["slots_free"] == 8
    # eos
    eng2 = FakeEngine()
    probe = Scheduler(eng2)
    probe.submit("p", _prompt(6), SamplingParams(max_tokens=5))
    full = probe.run()["p"]
    s2 = Scheduler(FakeEngine(), eos_token_id=full[2])
    s2.submit("p", _prompt(6), SamplingParams(max_tokens=5))
    assert s2.run()["p"] == full[:3]


def test_greedy_and_temperature_share_a_step():
    eng = FakeEngine()
    s = Scheduler(eng)
    s.submit("g", _prompt(5), SamplingParams(max_tokens=3))
    s.submit("t", _prompt(5), SamplingParams(max_tokens=3, temperature=0.8, seed=7))
    out = s.run()
    assert all(len(step) == 2 for step in eng.steps)  # never skipped for differing parameters
    assert out["g"] != out["t"]


@pytest.mark.parametrize("window", [None, 6])
def test_pages_run_out_preempts_the_youngest_and_tokens_do_not_change(window):
    reqs = {"a": (_prompt(9, 1), 14), "b": (_prompt(11, 2), 12), "c": (_prompt(7, 3), 16)}

    def run(pages):
        eng = FakeEngine(pages=pages, page=4, window=window)
        s = Scheduler(eng, prefill_chunk_size=8)
        for rid, (p, n) in reqs.items():
            s.submit(rid, p, SamplingParams(max_tokens=n, temperature=0.5, seed=3))
        out = s.run()
        assert all(p.used_pages == 0 for p in eng.cache.pools)
        return out, s.preemptions, eng

    calm, n0, _ = run(pages=64)
    tight, n1, eng = run(pages=9)  # all three do not fit at their final lengths (6 + 6 + 6 pages)
    assert n0 == 0 and n1 > 0
    assert tight == calm
    # the oldest request was never computed again: its tokens entered the cache exactly once
    fed = [t for step in eng.steps for rid, toks, _ in step if rid == "a" for t in toks]
    assert len(fed) == len(reqs["a"][0]) + reqs["a"][1] - 1
    # a replayed prompt's last portion asks for no logits when a token is already known
    assert any(rid != "a" and len(toks) > 1 and not want for step in eng.steps for rid, toks, want in step)


def test_a_request_that_cannot_fit_alone_fails_loudly():
    eng = FakeEngine(pages=3, page=4, max_context=1000)
    s = Scheduler(eng)
    s.submit("a", _prompt(10), SamplingParams(max_tokens=20))
    with pytest.raises(KVBlockExhausted):
        s.run()


def _workload(s):
    s.submit("a", _prompt(9, 1), SamplingParams(max_tokens=14, temperature=0.5, seed=3))
    s.submit("b", _prompt(11, 2), SamplingParams(max_tokens=1))
    s.submit("c", _prompt(30, 3), SamplingParams(max_tokens=16))
    s.submit("d", _prompt(5, 4), SamplingParams(max_tokens=40))   # ends at the context limit


@pytest.mark.parametrize("pages,eos", [(64, False), (64, True), (12, False), (12, True)])
def test_running_ahead_changes_no_token(pages, eos):
    """One step in flight: same tokens, same reasons, also with too few pages and with an end-of-sequence stop."""
    def run(ahead, eos_id):
        eng = FakeEngine(pages=pages, page=4, max_context=40)
        s = Scheduler(eng, prefill_chunk_size=8, run_ahead=ahead, eos_token_id=eos_id)
        _workload(s)
        out, reasons = {}, {}
        while s.has_work():
            for ev in s.step():
                if ev.token is not None:
                    out.setdefault(ev.req_id, []).append(ev.token)
                if ev.finished:
                    reasons[ev.req_id] = ev.reason
        assert all(p.used_pages == 0 for p in eng.cache.pools) and eng.cache.slots.free_slots == 8
        return out, reasons, s, eng

    base, _, _, _ = run(False, None)
    eos_id = base["c"][7] if eos else None
    calm, calm_reasons, s0, _ = run(False, eos_id)
    ahead, ahead_reasons, s1, eng = run(True, eos_id)
    assert ahead == calm and ahead_reasons == calm_reasons
    assert calm_reasons["d"] == "max_context" and calm_reasons["b"] == "max_tokens"
    if eos:
        assert calm_reasons["c"] == "eos" and len(calm["c"]) == 8
    if pages == 12:
        assert s1.preemptions > 0
    # results were read after the next step had been launched, except where nothing could be launched
    late = sum(1 for k, n in enumerate(eng.reads) if n > k + 1)
    assert late >= len(eng.reads) // 2


def test_cancel_while_a_step_is_in_flight():
    eng = FakeEngine()
    s = Scheduler(eng, run_ahead=True)
    s.submit("a", _prompt(5), SamplingParams(max_tokens=10))
    s.submit("b", _prompt(6, 9), SamplingParams(max_tokens=10))
    assert s.step() == []            # the first step's tokens are still in flight
    assert s.cancel("a")
    events = []
    while s.has_work():
        events += s.step()
    assert [e.req_id for e in events if e.req_id == "a"] == ["a"]   # the token that was in flight, no more
    assert len([e for e in events if e.req_id == "b" and e.token is not None]) == 10
    assert all(p.used_pages == 0 for p in eng.cache.pools)


@pytest.mark.parametrize("seed", range(int(os.environ.get("CCB_FUZZ_SEEDS", "8"))))   # 3,000 seeds passed
def test_random_workloads_with_and_without_running_ahead(seed):
    """Random prompts, lengths, sampling parameters, pool sizes, portion sizes and arrival times: a scheduler
    that runs ahead returns the same tokens and reasons as one that waits for every step, nothing is left in
    the cache, and the manager's books stay consistent throughout (the fake engine checks after every step)."""
    import random
    rnd = random.Random(seed)
    n = rnd.randint(3, 9)
    page = rnd.choice([2, 4, 8])
    max_context = rnd.choice([40, 64, 96])
    reqs = []
    for i in range(n):
        L = rnd.randint(1, max_context - 8)
        reqs.append((f"r{i}", _prompt(L, rnd.randint(0, 900)),
                     SamplingParams(max_tokens=rnd.randint(0, 30), temperature=rnd.choice([0.0, 0.7]), seed=i),
                     rnd.randint(0, 6)))
    longest = max(len(p) + sp.max_tokens for _, p, sp, _ in reqs)
    pages = max(-(-min(longest, max_context) // page) + 1, rnd.randint(6, 40))
    chunk = rnd.choice([0, 3, 8, 16])
    budget = rnd.choice([8, 24, 64])
    window = rnd.choice([None, None, 6])

    def run(ahead, eos_id):
        eng = FakeEngine(pages=pages, page=page, slots=4, max_context=max_context, window=window)
        s = Scheduler(eng, prefill_chunk_size=chunk, max_tokens_per_step=budget, max_running=rnd_running,
                      run_ahead=ahead, eos_token_id=eos_id)
        out, reasons, step_no = {}, {}, 0
        todo = sorted(reqs, key=lambda r: r[3])
        while todo or s.has_work():
            while todo and todo[0][3] <= step_no:
                rid, p, sp, _ = todo.pop(0)
                s.submit(rid, p, sp)
            for ev in s.step():
                if ev.token is not None:
                    out.setdefault(ev.req_id, []).append(ev.token)
                if ev.finished:
                    assert ev.req_id not in reasons
                    reasons[ev.req_id] = ev.reason
            step_no += 1
            assert step_no < 5000
        assert all(p.used_pages == 0 for p in eng.cache.pools) and eng.cache.slots.free_slots == 4
        assert set(reasons) == {r[0] for r in reqs}
        return out, reasons

    rnd_running = rnd.randint(1, 4)
    base, _ = run(False, None)
    produced = [t for toks in base.values() for t in toks]
    eos_id = rnd.choice(produced) if produced and rnd.random() < 0.5 else None
    calm = run(False, eos_id)
    ahead = run(True, eos_id)
    assert ahead == calm
    for rid, p, sp, _ in reqs:
        toks = calm[0].get(rid, [])
        assert len(toks) <= sp.max_tokens and len(p) + len(toks) <= max_context + 1


def test_which_kernel_takes_a_few_rows_product():
    """The measured rule, as a table: the shapes of the three model sizes at 1, 8 and 16 tokens."""
    from ccinfer_b200 import kernels

    def pick(M, N, K):
        return kernels.few_rows_product_kernel(M, N, K, 148, True, True, K % 32 == 0)

    # 8B: q|k|v 6144 x 4096, o 4096 x 4096, gate|up 24576 x 4096, down 4096 x 12288, vocabulary 151936 x 4096
    assert [pick(8, *s) for s in ((6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288), (151936, 4096))] == \
        ["fewrows", "fewrows", "tc", "fewrows", "tc"]
    assert [pick(1, *s) for s in ((6144, 4096), (4096, 4096), (4096, 12288))] == ["fewrows", "fewrows", "fewrows"]
    # 14B / 32B with one token: the same
    assert [pick(1, *s) for s in ((7168, 5120), (5120, 5120), (5120, 17408), (5120, 8192))] == \
        ["fewrows", "fewrows", "fewrows", "fewrows"]
    # what the ring kernel does not fit: long K to the tcgen05 kernel in slices, the rest to the register-streaming one
    assert kernels.few_rows_product_kernel(1, 5120, 17408, 148, True, False, True) == "tc_split"
    assert kernels.few_rows_product_kernel(1, 5120, 4096, 148, True, False, True) == "skinny"
    assert [pick(16, *s) for s in ((7168, 5120), (5120, 17408), (34816, 5120))] == ["fewrows", "fewrows", "tc"]
    # short K, more rows than the own kernels take, shapes no own kernel fits
    assert pick(8, 4096, 1024) == "skinny" and pick(17, 4096, 4096) == "library"
    assert kernels.few_rows_product_kernel(8, 4096, 4100, 148, False, False, False) == "library"
