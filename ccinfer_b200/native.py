"""ctypes face of the C++ host core (``csrc/host/ccinfer.h``): cache manager, request slots, the arrays of a step,
and the scheduler above them.

Every C call returns an error code; here a non-zero code becomes the package's exception of the same name,
with the message of ``ccinfer_last_error``.  The library is built at the first use (``csrc/build.py``, group
"host"; g++ through nvcc, no device code) and there is no Python stand-in for it.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import POINTER, Structure, byref, c_float, c_int, c_int64, c_longlong, c_uint64, c_void_p

from .csrc import build as _build
from .errors import (CcinferError, ExtensionMissing, InvalidArgument, KVBlockDoubleFree, KVBlockExhausted,
                     KVInvalidBlockTable, RequestTooLong, SlotExhausted)

MAX_GROUPS = 8


class InvalidState(CcinferError):
    code = "InvalidState"


class RunnerFailed(CcinferError):
    """The device work of a step failed; the step's pages were given back."""
    code = "RunnerFailed"


ERRORS = {1: InvalidArgument, 2: KVBlockExhausted, 3: KVBlockDoubleFree, 4: KVInvalidBlockTable, 5: SlotExhausted,
          6: RequestTooLong, 7: InvalidState, 8: RunnerFailed}


class Group(Structure):
    _fields_ = [("window", c_int), ("page_size", c_int), ("num_pages", c_int)]


class Options(Structure):
    _fields_ = [("n_groups", c_int), ("groups", POINTER(Group)), ("max_seqs", c_int), ("max_tokens_per_step", c_int),
                ("max_context", c_int)]


class Layout(Structure):
    _fields_ = [("capacity_tokens", c_int), ("capacity_entries", c_int), ("size_words", c_int),
                ("token_ids", c_int), ("positions", c_int), ("entry_of_token", c_int), ("logit_rows", c_int),
                ("row_slot", c_int), ("cu_q", c_int), ("pos0", c_int), ("ctx_after", c_int), ("state_slot", c_int),
                ("n_groups", c_int), ("slot_map", c_int * MAX_GROUPS), ("block_table", c_int * MAX_GROUPS),
                ("block_table_stride", c_int)]


class StepInfo(Structure):
    _fields_ = [("layout", c_int), ("n_tokens", c_int), ("n_entries", c_int), ("n_real_tokens", c_int),
                ("n_real_entries", c_int), ("n_logit_rows", c_int), ("n_single", c_int), ("max_q_len", c_int),
                ("max_ctx", c_int), ("n_copies", c_int), ("copy_offset", c_int * (MAX_GROUPS + 1)),
                ("copy_words", c_int * (MAX_GROUPS + 1)), ("order", POINTER(c_int))]


class Stats(Structure):
    _fields_ = [("seqs", c_int), ("slots_total", c_int), ("slots_free", c_int), ("n_groups", c_int),
                ("pages_total", c_int * MAX_GROUPS), ("pages_free", c_int * MAX_GROUPS),
                ("pages_high_water", c_int * MAX_GROUPS), ("steps", c_longlong)]


RUNNER = ctypes.CFUNCTYPE(c_int, c_void_p, POINTER(StepInfo))


class SamplingParamsC(Structure):
    _fields_ = [("max_tokens", c_int), ("top_k", c_int), ("top_p", c_float), ("temperature", c_float),
                ("seed", c_uint64)]


class SchedulerOptions(Structure):
    _fields_ = [("prefill_chunk_size", c_int), ("max_tokens_per_step", c_int), ("max_running", c_int),
                ("max_context", c_int), ("eos_token_id", c_int), ("run_ahead", c_int)]


class Plan(Structure):
    _fields_ = [("n_items", c_int), ("reqs", POINTER(c_int64)), ("counts", POINTER(c_int)), ("tokens", POINTER(c_int)),
                ("sample", POINTER(c_int)), ("out_index", POINTER(c_int)), ("params", POINTER(SamplingParamsC)),
                ("n_sampled", c_int)]


OPEN_HOOK = ctypes.CFUNCTYPE(c_int, c_void_p, c_int64, POINTER(c_int64))
CLOSE_HOOK = ctypes.CFUNCTYPE(c_int, c_void_p, c_int64)
RUN_HOOK = ctypes.CFUNCTYPE(c_int, c_void_p, POINTER(Plan), c_int64)
READ_HOOK = ctypes.CFUNCTYPE(c_int, c_void_p, c_int64, c_int, POINTER(c_int))


class SchedulerHooks(Structure):
    _fields_ = [("open", OPEN_HOOK), ("close", CLOSE_HOOK), ("run", RUN_HOOK), ("read", READ_HOOK), ("user", c_void_p)]


class Event(Structure):
    _fields_ = [("req", c_int64), ("token", c_int), ("finished", c_int), ("reason", c_int)]


class SchedulerStats(Structure):
    _fields_ = [("steps", c_longlong), ("preemptions", c_longlong), ("waiting", c_int), ("active", c_int),
                ("prefilling", c_int), ("in_flight", c_int), ("events", c_int)]


REASONS = {0: None, 1: "max_tokens", 2: "max_context", 3: "eos"}

_lock = threading.Lock()
_lib = None


def lib():
    """The loaded host library (built at the first call)."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.library_path("host")
        try:
            h = ctypes.CDLL(path)
        except OSError as e:
            raise ExtensionMissing(f"cannot load {path}: {e}") from e
        E = c_void_p
        sig = {
            "ccinfer_create": [POINTER(Options), POINTER(E)],
            "ccinfer_get_layout": [E, c_int, POINTER(Layout)],
            "ccinfer_stats": [E, POINTER(Stats)],
            "ccinfer_get_groups": [E, POINTER(Group), c_int, POINTER(c_int)],
            "ccinfer_check": [E],
            "ccinfer_alloc_seq": [E, c_int64, POINTER(c_int)],
            "ccinfer_free_seq": [E, c_int64],
            "ccinfer_seq_state": [E, c_int64, POINTER(c_int), POINTER(c_int), POINTER(c_int)],
            "ccinfer_seq_block_table": [E, c_int64, c_int, POINTER(c_int), c_int, POINTER(c_int)],
            "ccinfer_pages_needed": [E, c_int64, c_int, POINTER(c_int)],
            "ccinfer_reserve": [E, c_int64, c_int],
            "ccinfer_commit": [E, c_int64],
            "ccinfer_rollback": [E, c_int64],
            "ccinfer_pool_take": [E, c_int, c_int64, c_int, POINTER(c_int)],
            "ccinfer_pool_give_back": [E, c_int, c_int64, POINTER(c_int), c_int],
            "ccinfer_pool_owner": [E, c_int, c_int, POINTER(c_int64), POINTER(c_int)],
            "ccinfer_slot_take": [E, POINTER(c_int)],
            "ccinfer_slot_give_back": [E, c_int],
            "ccinfer_set_runner": [E, RUNNER, c_void_p],
            "ccinfer_forward": [E, c_int, POINTER(c_int64), POINTER(c_int), POINTER(c_int), POINTER(c_int),
                                POINTER(c_int), c_int, c_void_p, c_void_p, POINTER(StepInfo)],
        }
        S = c_void_p
        sig.update({
            "ccinfer_scheduler_create": [E, POINTER(SchedulerOptions), POINTER(SchedulerHooks), POINTER(S)],
            "ccinfer_scheduler_stats": [S, POINTER(SchedulerStats)],
            "ccinfer_scheduler_active": [S, POINTER(c_int64), c_int, POINTER(c_int)],
            "ccinfer_add_request": [S, c_int64, POINTER(c_int), c_int, POINTER(SamplingParamsC)],
            "ccinfer_cancel": [S, c_int64, POINTER(c_int)],
            "ccinfer_has_work": [S, POINTER(c_int)],
            "ccinfer_step": [S],
            "ccinfer_drain": [S],
            "ccinfer_pop_events": [S, POINTER(Event), c_int, POINTER(c_int)],
        })
        for name, argtypes in sig.items():
            fn = getattr(h, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        h.ccinfer_scheduler_destroy.argtypes = [S]
        h.ccinfer_scheduler_destroy.restype = None
        h.ccinfer_scheduler_last_error.argtypes = [S]
        h.ccinfer_scheduler_last_error.restype = ctypes.c_char_p
        h.ccinfer_destroy.argtypes = [E]
        h.ccinfer_destroy.restype = None
        h.ccinfer_last_error.argtypes = [E]
        h.ccinfer_last_error.restype = ctypes.c_char_p
        _lib = h
        return h


class HostCore:
    """One engine of the host core.  Sequences are named by 64-bit integers."""

    def __init__(self, groups, max_seqs: int, max_tokens_per_step: int, max_context: int):
        """``groups``: (window or None, page_size, num_pages) per cache group."""
        self._lib = lib()
        self.n_groups = len(groups)
        arr = (Group * max(1, self.n_groups))(*[Group(int(w or 0), int(p), int(n)) for w, p, n in groups])
        opt = Options(self.n_groups, arr, int(max_seqs), int(max_tokens_per_step), int(max_context))
        self._h = c_void_p()
        rc = self._lib.ccinfer_create(byref(opt), byref(self._h))
        if rc:
            raise ERRORS.get(rc, CcinferError)((self._lib.ccinfer_last_error(None) or b"").decode())
        self._runner = None     # keeps the callback object alive
        self._ints = (c_int * MAX_GROUPS)()

    def close(self):
        if self._h:
            self._lib.ccinfer_destroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ok(self, rc: int) -> None:
        if rc:
            raise ERRORS.get(rc, CcinferError)((self._lib.ccinfer_last_error(self._h) or b"").decode())

    # -- sequences -------------------------------------------------------------------------
    def alloc_seq(self, seq: int) -> int:
        slot = c_int()
        self._ok(self._lib.ccinfer_alloc_seq(self._h, seq, byref(slot)))
        return slot.value

    def free_seq(self, seq: int) -> None:
        self._ok(self._lib.ccinfer_free_seq(self._h, seq))

    def seq_state(self, seq: int):
        """(slot, cached tokens, tokens of an uncommitted reservation)"""
        a, b, c = c_int(), c_int(), c_int()
        self._ok(self._lib.ccinfer_seq_state(self._h, seq, byref(a), byref(b), byref(c)))
        return a.value, b.value, c.value

    def table_len(self, seq: int, group: int) -> int:
        n = c_int()
        self._ok(self._lib.ccinfer_seq_block_table(self._h, seq, group, None, 0, byref(n)))
        return n.value

    def block_table(self, seq: int, group: int):
        n = c_int()
        self._ok(self._lib.ccinfer_seq_block_table(self._h, seq, group, None, 0, byref(n)))
        out = (c_int * max(1, n.value))()
        self._ok(self._lib.ccinfer_seq_block_table(self._h, seq, group, out, n.value, byref(n)))
        return list(out[:n.value])

    def pages_needed(self, seq: int, n_new: int):
        self._ok(self._lib.ccinfer_pages_needed(self._h, seq, n_new, self._ints))
        return list(self._ints[:self.n_groups])

    def reserve(self, seq: int, n_new: int) -> None:
        self._ok(self._lib.ccinfer_reserve(self._h, seq, n_new))

    def commit(self, seq: int) -> None:
        self._ok(self._lib.ccinfer_commit(self._h, seq))

    def rollback(self, seq: int) -> None:
        self._ok(self._lib.ccinfer_rollback(self._h, seq))

    # -- pools -----------------------------------------------------------------------------
    def pool_take(self, group: int, owner: int, n: int):
        out = (c_int * max(1, n))()
        self._ok(self._lib.ccinfer_pool_take(self._h, group, owner, n, out))
        return list(out[:max(0, n)])

    def pool_give_back(self, group: int, owner: int, pages) -> None:
        arr = (c_int * max(1, len(pages)))(*[int(p) if isinstance(p, int) else -1 for p in pages])
        self._ok(self._lib.ccinfer_pool_give_back(self._h, group, owner, arr, len(pages)))

    def pool_owner(self, group: int, page: int):
        """The owner's number, or None for a free page."""
        owner, free = c_int64(), c_int()
        self._ok(self._lib.ccinfer_pool_owner(self._h, group, page, byref(owner), byref(free)))
        return None if free.value else owner.value

    def slot_take(self) -> int:
        s = c_int()
        self._ok(self._lib.ccinfer_slot_take(self._h, byref(s)))
        return s.value

    def slot_give_back(self, slot: int) -> None:
        self._ok(self._lib.ccinfer_slot_give_back(self._h, slot))

    # -- figures ---------------------------------------------------------------------------
    def stats(self) -> Stats:
        st = Stats()
        self._ok(self._lib.ccinfer_stats(self._h, byref(st)))
        return st

    def check(self) -> None:
        self._ok(self._lib.ccinfer_check(self._h))

    def layout(self, which: int) -> Layout:
        out = Layout()
        self._ok(self._lib.ccinfer_get_layout(self._h, which, byref(out)))
        return out

    # -- a step ----------------------------------------------------------------------------
    def set_runner(self, fn) -> None:
        """``fn(info: StepInfo) -> int`` (0 = ok) runs the device work of a step laid out by ``forward``."""
        self._runner = RUNNER(lambda user, info: fn(info.contents)) if fn is not None else RUNNER()
        self._ok(self._lib.ccinfer_set_runner(self._h, self._runner, None))

    def forward(self, seqs, counts, tokens, want_counts, wants, pad_to: int, small_ptr: int, large_ptr: int) -> StepInfo:
        """ccinfer_forward: validate, take pages, lay the step out, run it, commit (or give everything back).

        ``tokens`` and ``wants`` are contiguous int32 NumPy arrays (all entries' tokens, all entries' wanted
        places, one after another); the others are sequences of one integer per entry."""
        B = len(seqs)
        info = StepInfo()
        ip = POINTER(c_int)
        rc = self._lib.ccinfer_forward(
            self._h, B, (c_int64 * max(1, B))(*seqs), (c_int * max(1, B))(*counts), tokens.ctypes.data_as(ip),
            (c_int * max(1, B))(*want_counts), wants.ctypes.data_as(ip), int(pad_to), small_ptr, large_ptr,
            byref(info))
        self._ok(rc)
        return info


_CODES = {cls: code for code, cls in ERRORS.items()}


class SchedulerCore:
    """One scheduler of the host core above a ``HostCore``.

    The four hooks are Python callables: ``open(req) -> seq``, ``close(req)``, ``run(plan, ticket)`` with
    ``plan`` a ``Plan`` structure, ``read(ticket, n) -> n tokens``.  An exception inside a hook ends the C call
    with the error code of its class; the call here then raises that same exception again."""

    def __init__(self, core: HostCore, prefill_chunk_size: int, max_tokens_per_step: int, max_running: int,
                 max_context: int, eos_token_id, run_ahead: bool, run, read, open=None, close=None):
        self._lib = lib()
        self._core = core   # the engine must outlive its scheduler
        self._error = None

        def guard(fn):
            def wrapped(*a):
                try:
                    fn(*a)
                    return 0
                except BaseException as e:   # nothing may pass through the C frames
                    self._error = e
                    return next((code for cls, code in _CODES.items() if isinstance(e, cls)), 8)
            return wrapped

        def _open(user, req, seq_out):
            seq_out[0] = open(req)

        def _read(user, ticket, n, out):
            tokens = read(ticket, n)
            for i in range(n):
                out[i] = int(tokens[i])

        # without open/close hooks the scheduler calls ccinfer_alloc_seq / ccinfer_free_seq itself (sequence = request)
        self._hooks = SchedulerHooks(OPEN_HOOK(guard(_open)) if open is not None else OPEN_HOOK(),
                                     CLOSE_HOOK(guard(lambda user, req: close(req))) if close is not None else CLOSE_HOOK(),
                                     RUN_HOOK(guard(lambda user, plan, ticket: run(plan.contents, ticket))),
                                     READ_HOOK(guard(_read)), None)
        opt = SchedulerOptions(int(prefill_chunk_size), int(max_tokens_per_step), int(max_running), int(max_context),
                               -1 if eos_token_id is None else int(eos_token_id), int(bool(run_ahead)))
        self._h = c_void_p()
        rc = self._lib.ccinfer_scheduler_create(core._h, byref(opt), byref(self._hooks), byref(self._h))
        if rc:
            raise ERRORS.get(rc, CcinferError)((self._lib.ccinfer_scheduler_last_error(None) or b"").decode())
        self._events = (Event * 256)()

    def close(self):
        if self._h:
            self._lib.ccinfer_scheduler_destroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ok(self, rc: int) -> None:
        error, self._error = self._error, None
        if rc:
            if error is not None:
                raise error
            raise ERRORS.get(rc, CcinferError)((self._lib.ccinfer_scheduler_last_error(self._h) or b"").decode())

    def add_request(self, req: int, prompt, max_tokens: int, top_k: int, top_p: float, temperature: float,
                    seed: int) -> None:
        n = len(prompt)
        arr = (c_int * max(1, n))(*prompt)
        sp = SamplingParamsC(max(-1, min(int(max_tokens), 2**31 - 1)), int(top_k), float(top_p), float(temperature),
                             int(seed) & (2**64 - 1))
        self._ok(self._lib.ccinfer_add_request(self._h, req, arr, n, byref(sp)))

    def cancel(self, req: int) -> bool:
        found = c_int()
        self._ok(self._lib.ccinfer_cancel(self._h, req, byref(found)))
        return bool(found.value)

    def has_work(self) -> bool:
        yes = c_int()
        self._ok(self._lib.ccinfer_has_work(self._h, byref(yes)))
        return bool(yes.value)

    def step(self) -> None:
        self._ok(self._lib.ccinfer_step(self._h))

    def drain(self) -> None:
        self._ok(self._lib.ccinfer_drain(self._h))

    def pop_events(self):
        """[(req, token or None, finished, reason or None)] of everything queued."""
        out, n = [], c_int()
        while True:
            self._ok(self._lib.ccinfer_pop_events(self._h, self._events, len(self._events), byref(n)))
            for ev in self._events[:n.value]:
                out.append((ev.req, None if ev.token < 0 else ev.token, bool(ev.finished), REASONS.get(ev.reason)))
            if n.value < len(self._events):
                return out

    def stats(self) -> SchedulerStats:
        st = SchedulerStats()
        self._ok(self._lib.ccinfer_scheduler_stats(self._h, byref(st)))
        return st

    def active(self):
        n = c_int()
        self._ok(self._lib.ccinfer_scheduler_active(self._h, None, 0, byref(n)))
        out = (c_int64 * max(1, n.value))()
        self._ok(self._lib.ccinfer_scheduler_active(self._h, out, n.value, byref(n)))
        return list(out[:n.value])
