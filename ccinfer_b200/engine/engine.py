"""The engine core: model + cache + ONE step function.

``Engine.step(entries)`` runs a batch of (request, its next tokens) — portions
of prompts beside single decoded tokens, cut anywhere — as one batch from the
cache and returns the logits at the wanted places.  It corresponds to
7QiC/ccInfer's translate -> inference -> commit (src/worker/worker.cpp:330-539,
src/worker/batch_translator.cpp:241-431, src/model/model_runner.h:25-247) with
these differences: logits are computed only for the wanted rows and handed
out (the reference computes all rows and keeps them inside the runner),
sampling is a separate call, and nothing is allocated per step.

Validation, the taking of pages, the step arrays and commit or rollback are the native host core's
(``csrc/host/host_core.cpp``, ``ccinfer_forward``); the device work of a step, i.e. the model's parts launching
their kernels, is the runner that this class registers there.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache.manager import CacheManager, GroupSpec
from ..config.registry import load_config
from ..errors import InvalidArgument, Unsupported
from ..native import RunnerFailed
from ..weights.loader import open_weights, random_fetch
from .plan import ModelPlan
from .runtime import Runtime
from .step import GroupStep, LayerCache, StepContext

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


@dataclasses.dataclass
class StepEntry:
    req_id: Hashable
    tokens: Sequence[int]        # [PENDING] = the token that the last sampling stored for this request
    want: Sequence[int] = ()     # places among ``tokens`` whose logits are wanted


# In place of a token id in a one-token entry: the token that ``Engine.sample_async`` last drew for the
# request.  It is still on the device; a scheduler that runs one step ahead has not read it yet.
PENDING = -1


class SampledTokens:
    """Tokens drawn by ``Engine.sample_async``: on their way to pinned host memory."""

    def __init__(self, host: torch.Tensor, event: "torch.cuda.Event", n: int):
        self._host, self._event, self._n = host, event, n

    def tokens(self) -> List[int]:
        """Waits for the copy and returns one host integer per logits row."""
        self._event.synchronize()
        return self._host[:self._n].tolist()


@dataclasses.dataclass
class EngineOptions:
    dtype: object = "bfloat16"
    device: str = "cuda:0"
    page_size: int = 16              # tokens per cache page (the reference's constant, src/cache/block.h:9)
    kv_tokens: Optional[int] = None  # tokens the pool of a group that keeps every token holds; default 1024 pages
    kv_memory_fraction: Optional[float] = None  # instead of kv_tokens: this share of the memory that is free once
                                                # the weights are on the device goes to the cache pools
    kv_group_tokens: Optional[dict] = None      # tokens of single groups' pools, by group key: {("window", 40): 256}
    max_requests: int = 64           # live requests = state slots (src/worker/worker.h:102)
    max_tokens_per_step: int = 4096  # the reference's compute budget (src/scheduler/scheduler.cpp:25)
    max_context: Optional[int] = None  # longest request; default min(model limit, pool)
    use_graphs: bool = True
    use_pdl: bool = True             # kernels may start while their predecessor finishes (see csrc/common.cuh)


class Engine:
    def __init__(self, plan: ModelPlan, fetch, options: EngineOptions = None):
        opt = options or EngineOptions()
        self.options = opt
        try:
            self.dtype = _DTYPES[opt.dtype]
        except KeyError:
            raise Unsupported(f"dtype {opt.dtype!r}: bfloat16 or float32") from None
        if opt.page_size <= 0:
            raise InvalidArgument("page_size must be > 0")
        if not (0 < opt.max_requests <= opt.max_tokens_per_step):
            # a step of max_requests single tokens (padded to a graph's size) must fit the token arrays
            raise InvalidArgument(f"max_requests ({opt.max_requests}) must lie in 1 .. max_tokens_per_step "
                                  f"({opt.max_tokens_per_step})")
        plan.validate()
        self.plan = plan
        self.vocab_size = plan.vocab_size
        self.rt = rt = Runtime(opt.device, self.dtype, opt.max_tokens_per_step, opt.max_requests)
        kernels.set_pdl(int(opt.use_pdl))
        for part in plan.parts():
            part.bind(rt, fetch)

        # ---- cache groups, storage and state ----
        P = opt.page_size
        if opt.kv_tokens is not None and opt.kv_memory_fraction is not None:
            raise InvalidArgument("give kv_tokens or kv_memory_fraction, not both")
        group_keys: List[tuple] = []
        windows: List[Optional[int]] = []
        token_bytes: List[int] = []   # per group: bytes one token costs in all its layers
        owners: Dict[int, object] = {}  # run entry -> its CacheNeed
        self._entry_group: Dict[int, int] = {}
        self._cache: Dict[int, Dict[str, torch.Tensor]] = {}
        self._state: Dict[int, torch.Tensor] = {}
        for i, e in enumerate(plan.order):
            mixer = plan.layers[e.layer].mixer
            need = mixer.cache_need()
            if e.cache_of is not None:
                if need is None:
                    raise InvalidArgument(f"order[{i}] reads a cache but its mixer keeps none")
                if getattr(mixer, "own_kv", False):
                    raise InvalidArgument(f"order[{i}] reads another entry's cache but its mixer writes keys")
            elif need is not None:
                if len({t.name for t in need.tensors}) != len(need.tensors) or not need.tensors:
                    raise InvalidArgument(f"order[{i}]: a cache need names at least one tensor, each once")
                if need.group_key not in group_keys:
                    group_keys.append(need.group_key)
                    windows.append(need.window)
                    token_bytes.append(0)
                g = group_keys.index(need.group_key)
                self._entry_group[i] = g
                token_bytes[g] += need.bytes_per_token(self.dtype)
                owners[i] = need
            sn = mixer.state_need()
            if sn is not None:
                self._state[i] = torch.zeros((opt.max_requests,) + tuple(sn.shape), dtype=sn.dtype, device=rt.device)
        for i, e in enumerate(plan.order):
            if e.cache_of is not None:
                if e.cache_of not in self._entry_group:
                    raise InvalidArgument(f"order[{i}] reads the cache of entry {e.cache_of}, which keeps none")
                self._entry_group[i] = self._entry_group[e.cache_of]
        pages = self._pages_per_group(opt, group_keys, windows, token_bytes)
        for i, need in owners.items():
            n = pages[self._entry_group[i]]
            self._cache[i] = {t.name: torch.zeros((n,) + t.page_shape(P), dtype=t.dtype or self.dtype, device=rt.device)
                              for t in need.tensors}
        # the longest request: what the smallest pool of a group that keeps every token holds (a window group
        # gives pages back as a request moves on and bounds no length), and the model's own limit
        all_keys = [n for n, w in zip(pages, windows) if w is None]
        limit = (min(all_keys) if all_keys else self._base_pages(opt, P)) * P
        if plan.max_position is not None:
            limit = min(limit, plan.max_position)
        self.max_context = min(opt.max_context, limit) if opt.max_context else limit
        self.cache = CacheManager([GroupSpec(k, w, P, n) for k, w, n in zip(group_keys, windows, pages)],
                                  opt.max_requests, opt.max_tokens_per_step, self.max_context)
        self.graph_safe = all(getattr(p, "graph_safe", True) for p in plan.parts())

        # ---- the step arrays: two layouts of the host core (a small one for steps of up to max_requests token
        # rows, i.e. every decode step, and a large one), each with one device buffer and two pinned staging
        # buffers in turn: the host may fill one while the copy of the other is in flight ----
        core = self.cache.core
        self._layouts = [core.layout(0), core.layout(1)]
        self._host_bufs = [[torch.zeros(l.size_words, dtype=torch.int32).pin_memory() for _ in range(2)]
                           for l in self._layouts]
        self._host_np = [[b.numpy() for b in pair] for pair in self._host_bufs]
        self._host_events = [[None, None], [None, None]]
        self._host_turn = 0
        self._dev_bufs = [torch.zeros(l.size_words, dtype=torch.int32, device=rt.device) for l in self._layouts]
        core.set_runner(self._run_step)
        self._runner_fn = None        # in place of the forward pass: see try_step
        self._runner_error = None
        self._step_logits = None
        self._step_bucket = 0
        n_rows = max(opt.max_requests, 1)
        self._sample_tokens = torch.zeros(opt.max_tokens_per_step, dtype=torch.int32, device=rt.device)
        self._sample_host = [torch.zeros((5, opt.max_tokens_per_step), dtype=torch.int32).pin_memory()
                             for _ in range(2)]
        self._sample_out = [torch.zeros(opt.max_tokens_per_step, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._sample_events = [None, None]
        self._sample_turn = 0
        # the token last drawn for each request slot, read by the next step's embedding for PENDING entries
        self._pending_tokens = torch.zeros(opt.max_requests, dtype=torch.int32, device=rt.device)
        self._pending_slots = set()   # slots whose pending token is valid
        self._last_row_slot = None    # (device view, host list) of the most recent step's logits rows
        self._last_logits = None      # (address, shape) of the logits that the most recent step returned
        self._sample_dev = torch.zeros((5, opt.max_tokens_per_step), dtype=torch.int32, device=rt.device)
        self.steps_run = 0
        self.last_h2d_bytes = 0       # bytes of the step arrays that the most recent step copied to the device
        self.graph_replays = 0
        self._graphs: Dict[int, tuple] = {}

    @staticmethod
    def _base_pages(opt: "EngineOptions", P: int) -> int:
        kv_tokens = opt.kv_tokens if opt.kv_tokens is not None else 1024 * P
        return max(1, -(-kv_tokens // P))

    def _pages_per_group(self, opt, group_keys, windows, token_bytes) -> List[int]:
        """Pages of each cache group's pool, from what a token costs there and a budget.

        A group that keeps every token gets ``kv_tokens`` tokens (default 1024 pages, the reference's pool:
        src/worker/worker.cpp:272), or its share of ``kv_memory_fraction`` of the free memory.  A window
        group never needs more than what ``max_requests`` requests can hold at once, the window plus the
        step's new tokens each, and gets no more than that.  ``kv_group_tokens`` sets single groups by their
        key (("all",) or ("window", W)).
        """
        P = opt.page_size
        explicit = dict(opt.kv_group_tokens or {})
        for key in explicit:
            if tuple(key) not in group_keys:
                raise InvalidArgument(f"kv_group_tokens names the group {key!r}; the model has {group_keys}")

        def window_cap(w):
            return opt.max_requests * (w // P + 2) + -(-opt.max_tokens_per_step // P)

        if opt.kv_memory_fraction is not None:
            if not (0.0 < opt.kv_memory_fraction <= 1.0):
                raise InvalidArgument("kv_memory_fraction lies in (0, 1]")
            budget = int(torch.cuda.mem_get_info(self.rt.device)[0] * opt.kv_memory_fraction)
            page_bytes = [b * P for b in token_bytes]
            capped = [window_cap(w) if w is not None else None for w in windows]
            fixed = sum(c * pb for c, pb in zip(capped, page_bytes) if c is not None)
            open_bytes = sum(pb for c, pb in zip(capped, page_bytes) if c is None)
            if fixed > budget // 2:   # the window groups would take most of it: every group the same count instead
                each = max(1, budget // max(1, sum(page_bytes)))
                pages = [min(each, c) if c is not None else each for c in capped]
            else:
                each = max(1, (budget - fixed) // max(1, open_bytes))
                pages = [c if c is not None else each for c in capped]
        else:
            base = self._base_pages(opt, P)
            pages = [base if w is None else min(base, window_cap(w)) for w in windows]
        for key, tokens in explicit.items():
            pages[group_keys.index(tuple(key))] = max(1, -(-int(tokens) // P))
        return pages

    # ------------------------------------------------------------------------------------
    @classmethod
    def from_model_dir(cls, model_dir: str, options: EngineOptions = None) -> "Engine":
        """The model class is chosen by config.json's architecture name."""
        opt = options or EngineOptions()
        arch, cfg = load_config(model_dir)
        plan = arch.build_plan(cfg)
        fetch = open_weights(model_dir, plan.tensor_specs(), opt.device, _DTYPES[opt.dtype],
                             shared=plan.shared_tensor_names())
        try:
            eng = cls(plan, fetch, opt)
        finally:
            fetch.close()
        eng.config = cfg
        return eng

    @classmethod
    def from_random(cls, config, seed: int, std: float = 0.02, options: EngineOptions = None) -> "Engine":
        """Random weights drawn on the device (nothing is written); for measurements on large shapes."""
        from ..config.registry import architecture_of
        opt = options or EngineOptions()
        arch = architecture_of(config.to_json())
        plan = arch.build_plan(config)
        fetch = random_fetch(plan.tensor_specs(), seed, std, opt.device, _DTYPES[opt.dtype],
                             shared=plan.shared_tensor_names())
        eng = cls(plan, fetch, opt)
        eng.config = config
        return eng

    # ------------------------------------------------------------------------------------
    def open_request(self, req_id: Hashable) -> int:
        """Gives the request a state slot (its state tensors are zeroed); returns the slot."""
        rc = self.cache.open(req_id)
        for st in self._state.values():
            st[rc.slot].zero_()
        return rc.slot

    def close_request(self, req_id: Hashable) -> None:
        """Gives back what the request holds: its pages in every group and its slot."""
        rc = self.cache.requests.get(req_id)
        if rc is not None:
            self._pending_slots.discard(rc.slot)
        self.cache.close(req_id)

    def context_len(self, req_id: Hashable) -> int:
        return self.cache.get(req_id).ctx_len

    # ------------------------------------------------------------------------------------
    def _context(self, info) -> StepContext:
        """The views of the step that the host core has just laid out; its arrays go to the device."""
        which, turn = info.layout, self._turn_in_use
        lay, host, dev = self._layouts[which], self._host_np[which][turn], self._dev_bufs[which]
        Tp, Bp, R = info.n_tokens, info.n_entries, info.n_logit_rows
        step = StepContext()
        step.n_tokens, step.n_entries, step.n_logit_rows = Tp, Bp, R
        step.n_single, step.max_q_len, step.max_ctx = info.n_single, info.max_q_len, info.max_ctx

        def dv(off, n):
            return dev[off:off + n]

        def hv(off, n):
            return host[off:off + n]

        step.token_ids = dv(lay.token_ids, Tp)
        step.positions = dv(lay.positions, Tp)
        step.entry_of_token = dv(lay.entry_of_token, Tp)
        step.logit_rows = dv(lay.logit_rows, max(R, 1))
        step.row_slot = dv(lay.row_slot, max(R, 1))
        step.pending_tokens = self._pending_tokens
        step.cu_q = dv(lay.cu_q, Bp + 1)
        step.pos0 = dv(lay.pos0, Bp)
        step.ctx_after = dv(lay.ctx_after, Bp)
        step.state_slot = dv(lay.state_slot, Bp)
        stride = lay.block_table_stride
        for g, spec in enumerate(self.cache.groups):
            step.groups.append(GroupStep(
                index=g, page_size=spec.page_size, num_pages=spec.num_pages, window=spec.window,
                slot_map=dv(lay.slot_map[g], Tp),
                block_table=dv(lay.block_table[g], Bp * stride).view(Bp, stride),
                host_slot_map=hv(lay.slot_map[g], Tp),
                host_block_table=hv(lay.block_table[g], Bp * stride).reshape(Bp, stride)))
        step.host = _HostView(hv(lay.token_ids, Tp), hv(lay.positions, Tp), hv(lay.entry_of_token, Tp),
                              hv(lay.logit_rows, R), hv(lay.cu_q, Bp + 1), hv(lay.pos0, Bp), hv(lay.ctx_after, Bp),
                              hv(lay.state_slot, Bp))
        # only the ranges that hold this step's data travel: the small arrays, and of every block table the
        # rows of the step's entries
        host_t = self._host_bufs[which][turn]
        copied = 0
        for c in range(info.n_copies):
            off, n = info.copy_offset[c], info.copy_words[c]
            dev[off:off + n].copy_(host_t[off:off + n], non_blocking=True)
            copied += n
        self.last_h2d_bytes = 4 * copied
        ev = torch.cuda.Event()
        ev.record()
        self._host_events[which][turn] = ev
        self._row_slot_dev = step.row_slot
        return step

    def _run_step(self, info) -> int:
        """The runner that the host core calls once a step is laid out: the device work.  0 = done; anything
        else makes the core give the step's pages back (the error itself is kept for ``step`` to raise)."""
        try:
            step = self._context(info)
            if self._runner_fn is not None:
                self._step_logits = self._runner_fn(step)
            elif self._step_bucket:
                self._step_logits = self._replay_decode(step, self._step_bucket, info.n_real_entries)
            else:
                self._step_logits = self._forward(step)
            return 0
        except BaseException as e:   # an exception must not cross the C frames between here and step()
            self._runner_error = e
            return 1

    def _launch(self, entries: List[StepEntry], bucket: int):
        """One call of the host core's ccinfer_forward for the entries given."""
        opt = self.options
        seqs, slots, counts, want_counts = [], [], [], []
        for e in entries:
            rc = self.cache.get(e.req_id)
            seqs.append(rc.seq)
            slots.append(rc.slot)
            counts.append(len(e.tokens))
            want_counts.append(len(e.want))
            if len(e.tokens) == 1 and e.tokens[0] == PENDING and rc.slot not in self._pending_slots:
                raise InvalidArgument(f"request {e.req_id!r}: PENDING stands for the token of a sample_async for the "
                                      f"request, and there was none since its last step")
        if len(entries) > opt.max_requests:
            raise InvalidArgument(f"{len(entries)} entries in a step, at most {opt.max_requests}")
        tokens = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int32, count=sum(counts))
        wants = np.fromiter((w for e in entries for w in e.want), dtype=np.int32, count=sum(want_counts))
        turn = self._host_turn
        self._host_turn ^= 1
        for which in (0, 1):
            if self._host_events[which][turn] is not None:
                self._host_events[which][turn].synchronize()   # its last copy has left the buffer
        self._turn_in_use = turn
        self._step_bucket = bucket
        self._runner_error = None
        self._step_logits = None
        self._last_logits = self._last_row_slot = None
        try:
            self.cache.core.forward(seqs, counts, tokens, want_counts, wants, bucket,
                                    self._host_bufs[0][turn].data_ptr(), self._host_bufs[1][turn].data_ptr())
        except RunnerFailed:
            raise self._runner_error from None
        # a pending token serves one step: this one read it, or brought the request's token itself
        self._pending_slots.difference_update(slots)
        # which request slot each logits row belongs to (a graph's rows are one per entry, in the core's order:
        # as a set of slots that is the same)
        self._last_row_slot = (self._row_slot_dev, slots if bucket else [s for s, n in zip(slots, want_counts)
                                                                         for _ in range(n)])
        return self._step_logits

    def try_step(self, entries: Sequence[StepEntry], fn):
        """Lays a step out as ``step`` does (pages taken, arrays on the device), calls ``fn(step_context)`` in
        place of the model's forward pass and then gives everything back: nothing is committed.  For tests of
        single parts, which need a real step to run in."""
        class _GiveBack(Exception):
            pass
        result = []

        def run(step):
            result.append(fn(step))
            raise _GiveBack()

        self._runner_fn = run
        try:
            self._launch([e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries], 0)
        except _GiveBack:
            pass
        finally:
            self._runner_fn = None
        return result[0] if result else None

    def _forward(self, step: StepContext) -> Optional[torch.Tensor]:
        plan = self.plan
        if getattr(plan.embedding, "takes_first_norm", False) and plan.order:
            stream = plan.embedding.forward(step, getattr(plan.layers[plan.order[0].layer], "first_norm", None))
        else:
            stream = plan.embedding.forward(step)
        for i, e in enumerate(plan.order):
            block = plan.layers[e.layer]
            cache = None
            if i in self._entry_group:
                src = i if e.cache_of is None else e.cache_of
                cache = LayerCache(self._cache[src], step.groups[self._entry_group[i]], own=e.cache_of is None)
            nxt = plan.layers[plan.order[i + 1].layer] if i + 1 < len(plan.order) else None
            stream.next_norm = getattr(nxt, "first_norm", None)
            block.forward(stream, step, cache, self._state.get(i))
        if step.n_logit_rows == 0:
            return None
        x = plan.final_norm.fold(stream, rows=step.logit_rows, n_rows=step.n_logit_rows)
        return plan.head.forward(x)

    # -- decode steps replayed from CUDA graphs ------------------------------------------------
    def _graph_bucket(self, entries: List[StepEntry]) -> int:
        """Size of the graph a step can be replayed from: 0 unless every entry is one token wanting its logits."""
        if not (self.options.use_graphs and self.graph_safe):
            return 0
        for e in entries:
            if len(e.tokens) != 1 or list(e.want) != [0]:
                return 0
        return self._bucket_of(len(entries))

    def _replay_decode(self, step: StepContext, bucket: int, n_real: int) -> torch.Tensor:
        """A decode step of up to ``bucket`` requests: the step arrays have been copied, the kernels are replayed.

        The launch sequence of a decode step depends on the number of rows only, and every buffer it
        touches has a fixed address (the small layout's device buffer, the scratch pool), so it is captured
        once per size (rows beyond the live requests are padding: they cache nothing and attend to nothing)."""
        if bucket not in self._graphs:
            self._forward(step)  # once eagerly: every scratch buffer exists before the capture ...
            self.rt.scratch.freeze()  # ... and none may move once a graph holds its address
            graph = torch.cuda.CUDAGraph()
            own0, lib0 = kernels.counters.own, kernels.counters.library
            with torch.cuda.graph(graph):
                out = self._forward(step)
            self._graphs[bucket] = (graph, out, kernels.counters.own - own0, kernels.counters.library - lib0)
        graph, out, n_own, n_lib = self._graphs[bucket]
        graph.replay()
        kernels.counters.own += n_own      # a replay launches what the capture recorded
        kernels.counters.library += n_lib
        self.graph_replays += 1
        return out[:n_real]

    def warm_up(self, batch_sizes: Sequence[int] = ()) -> List[int]:
        """Captures the decode graphs of the given batch sizes (default: every power of two up to
        max_requests) before the first request needs them, with throw-away requests of one token; returns
        the sizes captured.  A capture costs a fraction of a second per size at 36 layers, which the first
        decode step of that size would otherwise pay."""
        if not (self.options.use_graphs and self.graph_safe):
            return []
        sizes = sorted({self._bucket_of(b) for b in (batch_sizes or self._all_buckets())} - {0})
        done = []
        for b in sizes:
            if b in self._graphs or self.cache.slots.free_slots < b or min(p.free_pages for p in self.cache.pools) < b:
                continue
            ids = [("__warm_up__", i) for i in range(b)]
            try:
                for rid in ids:
                    self.open_request(rid)
                self.step([StepEntry(rid, [0], [0]) for rid in ids])
                done.append(b)
            finally:
                for rid in ids:
                    if rid in self.cache.requests:
                        self.close_request(rid)
        torch.cuda.synchronize(self.rt.device)
        return done

    def _bucket_of(self, n: int) -> int:
        """The size of the graph that takes a decode step of n requests: the next power of two, or
        max_requests where that is no power of two and lies below it."""
        if n > self.options.max_requests:
            return 0
        b = 1
        while b < n:
            b *= 2
        return min(b, self.options.max_requests)

    def _all_buckets(self) -> List[int]:
        out, b = [], 1
        while b < self.options.max_requests:
            out.append(b)
            b *= 2
        return out + [self.options.max_requests]

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs the tokens given, as one batch, from the cache; returns float logits [wanted, vocab].

        Rows are in the order of the entries and, within an entry, of its ``want``.
        Either the whole step happens (every request's cached length grows by its
        token count) or nothing does: if pages run out (KVBlockExhausted) or a
        launch fails, the pages taken for the step are given back.

        The logits are a view of a buffer of the engine: they stay valid until the
        next step is launched (copy them to keep them longer).
        """
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        logits = self._launch(entries, self._graph_bucket(entries))
        self.steps_run += 1
        if logits is None:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.rt.device)
        self._last_logits = (logits.data_ptr(), tuple(logits.shape))
        return logits

    def sample(self, logits: torch.Tensor, params: Sequence, out_index: Sequence[int]) -> List[int]:
        """One token per logits row: greedy where temperature <= 0, else a temperature draw, restricted to
        the top-k logits / the top-p share of the probability where the row's parameters say so.

        ``params[r]`` has ``temperature`` and ``seed`` (and may have ``top_k``, ``top_p``); ``out_index[r]`` is how many tokens the
        row's request has produced so far.  A draw depends on (seed, out_index) only, not on the
        batch.  Returns host integers (this waits for the step).
        """
        if logits.shape[0] == 0:
            return []
        return self.sample_async(logits, params, out_index).tokens()

    def sample_async(self, logits: torch.Tensor, params: Sequence, out_index: Sequence[int]) -> SampledTokens:
        """As ``sample`` for the logits of the most recent step, without waiting.

        The tokens go to pinned host memory (``SampledTokens.tokens()`` waits for them) and stay on the
        device per request: the request's next entry may bring ``[PENDING]`` in place of the token, so the
        next step can be launched before this one's tokens have been read.  At most two results may be
        outstanding.  Only the tensor that the most recent ``step`` returned leaves its tokens with the
        requests (a pending token serves the request's next step only); any other float [rows, vocab]
        tensor is sampled without that."""
        R = logits.shape[0]
        if len(params) != R or len(out_index) != R:
            raise InvalidArgument("one parameter set and one output index per logits row")
        turn = self._sample_turn
        self._sample_turn ^= 1
        if self._sample_events[turn] is not None:
            self._sample_events[turn].synchronize()  # the copies that used this turn's pinned buffers are over
        tokens = self._sample_tokens[:R]
        slot_dev = slots = None
        if (self._last_row_slot is not None and self._last_logits == (logits.data_ptr(), tuple(logits.shape))
                and len(self._last_row_slot[1]) == R):
            slot_dev, slots = self._last_row_slot
            self._last_logits = None   # the rows of a step leave their tokens once
        if R and all(p.temperature <= 0 for p in params):
            kernels.sample_rows(logits, tokens, slot_of_row=slot_dev, by_slot=self._pending_tokens)
        elif R:
            hp = self._sample_host[turn]
            hp[0, :R] = torch.tensor([float(p.temperature) for p in params], dtype=torch.float32).view(torch.int32)
            hp[1, :R] = torch.tensor([int(p.seed) & 0xFFFFFFFF for p in params], dtype=torch.int64).to(torch.int32)
            hp[2, :R] = torch.tensor(list(out_index), dtype=torch.int32)
            filtered = any(getattr(p, "top_k", 0) > 0 or getattr(p, "top_p", 1.0) < 1.0 for p in params)
            if filtered:
                hp[3, :R] = torch.tensor([int(getattr(p, "top_k", 0)) for p in params], dtype=torch.int32)
                hp[4, :R] = torch.tensor([float(getattr(p, "top_p", 1.0)) for p in params],
                                         dtype=torch.float32).view(torch.int32)
            self._sample_dev.copy_(hp, non_blocking=True)
            d = self._sample_dev
            kernels.sample_rows(logits, tokens, d[0, :R].view(torch.float32), d[1, :R], d[2, :R],
                                slot_of_row=slot_dev, by_slot=self._pending_tokens,
                                top_k=d[3, :R] if filtered else None,
                                top_p=d[4, :R].view(torch.float32) if filtered else None)
        if slots is not None:
            self._pending_slots.update(s for s in slots if s >= 0)
        out = self._sample_out[turn]
        if R:
            out[:R].copy_(tokens, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._sample_events[turn] = ev
        return SampledTokens(out, ev, R)

    def check(self) -> None:
        """Synchronises and raises DeviceFault if a kernel reported a bad index since the last check."""
        self.rt.check_status()

    def stats(self) -> dict:
        s = self.cache.stats()
        s["steps"] = self.steps_run
        s["scratch_bytes"] = self.rt.scratch.bytes()
        return s


@dataclasses.dataclass
class _HostView:
    token_ids: np.ndarray
    positions: np.ndarray
    entry_of_token: np.ndarray
    logit_rows: np.ndarray
    cu_q: np.ndarray
    pos0: np.ndarray
    ctx_after: np.ndarray
    state_slot: np.ndarray
