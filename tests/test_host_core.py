"""The native host core through its C interface (csrc/host/ccinfer.h): no GPU, the runner is a Python function
that looks at the arrays of the step instead of launching kernels.

What 7QiC/ccInfer tests of its translator and manager in tests/unit/test_batch_translator.cpp and
tests/unit/test_kv_cache_manager.cpp is restated for this interface: the arrays of a mixed step, pages taken
on demand and returned when a step fails, nothing moved by a refused step.
"""

import numpy as np
import pytest

from ccinfer_b200 import native
from ccinfer_b200.errors import InvalidArgument, KVBlockExhausted, RequestTooLong, SlotExhausted


def _core(pages=16, page=4, window=None, seqs=4, tokens=32, context=48):
    groups = [(None, page, pages)]
    if window:
        groups.append((window, page, pages))
    return native.HostCore(groups, seqs, tokens, context)


class _Step:
    """Buffers for a core and a runner that records what it is shown."""

    def __init__(self, core, fail=False):
        self.core, self.fail = core, fail
        self.lay = [core.layout(0), core.layout(1)]
        self.bufs = [np.full(l.size_words, -7, dtype=np.int32) for l in self.lay]
        self.seen = None
        core.set_runner(self.run)

    def run(self, info):
        lay, buf = self.lay[info.layout], self.bufs[info.layout]
        T, B, R = info.n_tokens, info.n_entries, info.n_logit_rows
        take = lambda off, n: buf[off:off + n].copy()
        self.seen = dict(
            layout=info.layout, T=T, B=B, R=R, n_single=info.n_single, max_q=info.max_q_len, max_ctx=info.max_ctx,
            real=(info.n_real_tokens, info.n_real_entries), tokens=take(lay.token_ids, T), pos=take(lay.positions, T),
            eot=take(lay.entry_of_token, T), rows=take(lay.logit_rows, R), row_slot=take(lay.row_slot, R),
            cu=take(lay.cu_q, B + 1), pos0=take(lay.pos0, B), after=take(lay.ctx_after, B), slot=take(lay.state_slot, B),
            slot_map=[take(lay.slot_map[g], T) for g in range(lay.n_groups)],
            bt=[take(lay.block_table[g], B * lay.block_table_stride).reshape(B, -1) for g in range(lay.n_groups)],
            copies=[(info.copy_offset[c], info.copy_words[c]) for c in range(info.n_copies)],
            order=[info.order[k] for k in range(info.n_real_entries)])
        return 1 if self.fail else 0

    def forward(self, entries, pad_to=0):
        seqs = [e[0] for e in entries]
        counts = [len(e[1]) for e in entries]
        toks = np.asarray([t for e in entries for t in e[1]], dtype=np.int32)
        wc = [len(e[2]) for e in entries]
        wants = np.asarray([w for e in entries for w in e[2]], dtype=np.int32)
        return self.core.forward(seqs, counts, toks, wc, wants, pad_to, self.bufs[0].ctypes.data, self.bufs[1].ctypes.data)


def test_create_refuses_bad_options_with_a_message():
    with pytest.raises(InvalidArgument, match="max_tokens_per_step"):
        native.HostCore([(None, 4, 8)], 8, 4, 32)
    with pytest.raises(InvalidArgument, match="page pool"):
        native.HostCore([(None, 4, 0)], 2, 8, 32)
    with pytest.raises(InvalidArgument, match="page_size"):
        native.HostCore([(None, 0, 4)], 2, 8, 32)
    lib = native.lib()
    assert lib.ccinfer_create(None, None) == 1 and b"null" in lib.ccinfer_last_error(None)


def test_arrays_of_a_mixed_step():
    """A portion of a prompt beside two single tokens: single-token entries come first, positions continue each
    sequence, rows are in the caller's order, slots and block tables follow the pages taken."""
    core = _core(page=4)
    st = _Step(core)
    for s in (11, 22, 33):
        core.alloc_seq(s)
    st.forward([(11, [5, 6, 7, 8, 9], [4])])            # 11 holds 5 tokens: pages 0, 1
    st.forward([(22, [1, 2, 3], [])])                   # 22 holds 3: page 2
    assert st.seen["layout"] == 0 and st.seen["R"] == 0
    st.forward([(33, [40, 41, 42, 43, 44, 45], [0, 5]), (11, [10], [0]), (22, [4], [0])])
    v = st.seen
    assert (v["T"], v["B"], v["R"], v["n_single"], v["max_q"], v["max_ctx"]) == (8, 3, 4, 2, 6, 6)
    assert v["order"] == [1, 2, 0]                                        # the two single tokens first
    assert v["tokens"].tolist() == [10, 4, 40, 41, 42, 43, 44, 45]
    assert v["pos"].tolist() == [5, 3, 0, 1, 2, 3, 4, 5]
    assert v["eot"].tolist() == [0, 1, 2, 2, 2, 2, 2, 2]
    assert v["cu"].tolist() == [0, 1, 2, 8] and v["pos0"].tolist() == [5, 3, 0] and v["after"].tolist() == [6, 4, 6]
    assert v["slot"].tolist() == [0, 1, 2]
    assert v["rows"].tolist() == [2, 7, 0, 1] and v["row_slot"].tolist() == [2, 2, 0, 1]   # the caller's order
    # 33 took pages 3 and 4; 11's sixth token sits in its page 1 (slot 1 * 4 + 1), 22's fourth in page 2
    assert v["slot_map"][0].tolist() == [5, 11, 12, 13, 14, 15, 16, 17]
    assert v["bt"][0][0, :2].tolist() == [0, 1] and v["bt"][0][1, :1].tolist() == [2] and v["bt"][0][2, :2].tolist() == [3, 4]
    assert core.seq_state(33) == (2, 6, 0) and core.seq_state(11)[1] == 6
    # the ranges that must reach the device: the small arrays and the three rows of the block table, adjacent
    assert v["layout"] == 1                               # eight token rows: the large layout
    lay = st.lay[1]
    assert v["copies"] == [(0, lay.block_table[0] + 3 * lay.block_table_stride)]
    core.check()


def test_large_layout_padding_and_pending_tokens():
    core = _core(seqs=4, tokens=32)
    st = _Step(core)
    core.alloc_seq(1)
    core.alloc_seq(2)
    st.forward([(1, list(range(9)), [8])])
    assert st.seen["layout"] == 1                        # nine token rows do not fit the small layout of four
    st.forward([(2, [3], [0])])
    st.forward([(1, [-1], [0]), (2, [-1], [0])], pad_to=4)
    v = st.seen
    assert (v["layout"], v["T"], v["B"], v["R"], v["n_single"], v["real"]) == (0, 4, 4, 4, 4, (2, 2))
    assert v["tokens"].tolist() == [-1 - 0, -1 - 1, 0, 0]   # -1 - slot: resolved on the device
    assert v["eot"].tolist() == [0, 1, -1, -1] and v["slot"].tolist() == [0, 1, -1, -1]
    assert v["cu"].tolist() == [0, 1, 2, 3, 4] and v["rows"].tolist() == [0, 1, 2, 3]
    assert v["row_slot"].tolist() == [0, 1, -1, -1] and v["slot_map"][0].tolist()[2:] == [-1, -1]
    with pytest.raises(InvalidArgument, match="padded"):
        st.forward([(1, [5, 6], [])], pad_to=4)
    with pytest.raises(InvalidArgument, match="non-negative"):
        st.forward([(1, [-1, 3], [])])


def test_a_failed_step_moves_nothing():
    core = _core(pages=4, page=4, seqs=3)
    st = _Step(core)
    for s in (1, 2):
        core.alloc_seq(s)
    st.forward([(1, list(range(8)), [])])
    before = core.stats().pages_free[0]
    with pytest.raises(KVBlockExhausted):                # 1 needs one page, 2 needs two; two are free
        st.forward([(1, [0], []), (2, list(range(8)), [])])
    assert core.stats().pages_free[0] == before and core.seq_state(1) == (0, 8, 0) and core.seq_state(2)[1] == 0
    st.fail = True                                       # the device work fails: the same
    with pytest.raises(native.RunnerFailed):
        st.forward([(1, [0], []), (2, [1, 2], [])])
    assert core.stats().pages_free[0] == before and core.seq_state(2)[1] == 0 and core.block_table(2, 0) == []
    st.fail = False
    for bad, exc in (([(1, [], [])], InvalidArgument), ([(1, [1], []), (1, [2], [])], InvalidArgument),
                     ([(9, [1], [])], InvalidArgument), ([(1, [1], [1])], InvalidArgument),
                     ([(2, list(range(33)), [])], InvalidArgument),       # more tokens than a step takes
                     ([(1, list(range(41)), [])], RequestTooLong),        # 8 cached + 41 > max_context 48
                     ([], InvalidArgument)):
        with pytest.raises(exc):
            st.forward(bad)
    core.check()
    assert core.stats().steps == 1


def test_window_group_gives_pages_back_at_commit_and_rows_are_cleared():
    core = _core(pages=16, page=4, window=6, seqs=2, tokens=32, context=64)
    st = _Step(core)
    core.alloc_seq(1)
    st.forward([(1, list(range(13)), [])])
    assert core.block_table(1, 1) == [-1, -1] + core.block_table(1, 1)[2:] and core.block_table(1, 0)[:2] == [0, 1]
    core.free_seq(1)
    core.alloc_seq(2)                                     # takes the slot and the step-buffer row of 1
    st.forward([(2, [1, 2, 3], [])])                      # the same (large) layout and row as the 13 tokens before
    assert st.seen["layout"] == 1 and st.seen["bt"][0][0, 0] >= 0
    assert (st.seen["bt"][0][0, 1:4] == -1).all()       # what the longer sequence left in the row is gone
    with pytest.raises(SlotExhausted):
        core.alloc_seq(3), core.alloc_seq(4)
    core.check()


def test_scheduler_through_the_c_calls_alone():
    """ccinfer_add_request / ccinfer_step / ccinfer_cancel with no Python scheduler above them: the scheduler
    opens and closes sequences itself (no open/close hooks), the run hook takes the pages of each item through
    ccinfer_reserve/commit, the read hook answers with tokens that depend on the ticket alone."""
    core = _core(pages=12, page=4, seqs=3, tokens=16, context=40)
    ran, tickets = [], {}

    def run(plan, ticket):
        items, at = [], 0
        for i in range(plan.n_items):
            n = plan.counts[i]
            items.append((plan.reqs[i], plan.tokens[at:at + n], plan.sample[i], plan.out_index[i]))
            at += n
        for req, toks, _, _ in items:
            core.reserve(req, len(toks))
            core.commit(req)
        ran.append(items)
        tickets[ticket] = [100 * ticket + k for k in range(plan.n_sampled)]
        assert plan.params[0].max_tokens in (3, 5) and abs(plan.params[0].top_p - 0.9) < 1e-6

    sched = native.SchedulerCore(core, prefill_chunk_size=6, max_tokens_per_step=16, max_running=3, max_context=40,
                                 eos_token_id=None, run_ahead=False, run=run, read=lambda ticket, n: tickets.pop(ticket))
    sched.add_request(7, list(range(10)), max_tokens=3, top_k=0, top_p=0.9, temperature=0.0, seed=1)
    sched.add_request(8, list(range(4)), max_tokens=5, top_k=0, top_p=0.9, temperature=0.7, seed=2**63 + 5)
    with pytest.raises(InvalidArgument, match="already known"):
        sched.add_request(7, [1], 1, 0, 1.0, 0.0, 0)
    with pytest.raises(RequestTooLong):
        sched.add_request(9, list(range(41)), 1, 0, 1.0, 0.0, 0)
    with pytest.raises(InvalidArgument, match="top_k"):
        sched.add_request(9, [1], 1, -1, 1.0, 0.0, 0)
    sched.step()
    assert ran[-1] == [(7, list(range(6)), 0, 0), (8, list(range(4)), 1, 0)]   # a portion beside a whole prompt
    assert sched.pop_events() == [(8, 100, False, None)]
    assert core.seq_state(7)[1] == 6 and core.seq_state(8)[1] == 4 and sched.active() == [7, 8]
    sched.step()
    assert ran[-1] == [(8, [100], 1, 1), (7, [6, 7, 8, 9], 1, 0)]                # decoding first, then the rest
    assert sched.pop_events() == [(8, 200, False, None), (7, 201, False, None)]
    st = sched.stats()
    assert (st.steps, st.waiting, st.active, st.prefilling, st.in_flight) == (2, 0, 2, 0, 0)
    assert sched.cancel(8) and not sched.cancel(8) and core.stats().seqs == 1
    events = []
    while sched.has_work():
        sched.step()
        events += sched.pop_events()
    assert [e[1] for e in events] == [300, 400] and events[-1][2:] == (True, "max_tokens")
    assert core.stats().seqs == 0 and core.stats().pages_free[0] == 12
    core.check()
    # a hook that fails ends the call with its error, and nothing has moved
    sched.add_request(10, [1, 2, 3], 2, 0, 1.0, 0.0, 0)

    def broken(plan, ticket):
        raise KVBlockExhausted("no pages today")
    sched2 = native.SchedulerCore(core, 0, 16, 3, 40, None, False, run=broken, read=lambda t, n: [])
    sched2.add_request(11, [1, 2, 3], 2, 0, 1.0, 0.0, 0)
    with pytest.raises(KVBlockExhausted, match="no pages today"):
        sched2.step()
    assert sched2.stats().steps == 0 and core.seq_state(11)[1] == 0
    assert sched2.cancel(11) and sched.cancel(10)
    core.check()
