"""Interfaces of the parts a model is put together from.

A model is data: a list of blocks and the order in which they run.  A block
arranges a token mixer, a feed-forward and norms around a residual stream.
Every part takes its sizes and constants as constructor arguments and the
names of its tensors from whoever builds the model; no part knows which model
it is in.

What a part must provide:

* ``tensor_specs()``: the tensors it wants, by full name, with shape and role.
* ``bind(rt, fetch)``: take the device tensors (``fetch(name)``), merge or
  re-lay them as its kernels want, allocate constant tables.
* a forward method (see each base class) that launches kernels on the current
  stream and returns views of scratch buffers from ``rt.scratch``.

A mixer further says what it needs to remember between steps:

* ``cache_need()``: the tensors it keeps per token, in pages (of all tokens, or
  of a window of them), or None;
* ``state_need()``: a tensor of fixed size per request, or None.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, List, Optional, Tuple

import torch


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    # "matrix": kept in the compute type (bfloat16 or float); "vector": small
    # per-channel weights, kept in float; "table": integers, kept as int32.
    role: str = "matrix"
    # how the random-weights mode fills it: "normal" = N(0, std), "one_plus_normal" = 1 + N(0, std)
    init: str = "normal"


@dataclasses.dataclass(frozen=True)
class CachedTensor:
    """One tensor a mixer keeps per token, in pages.

    ``shape`` is that of one token; a page holds ``page_size`` tokens along a new axis put at ``token_axis``
    of it: keys of shape (kv_heads, head_dim) with token_axis 1 live in [pages, kv_heads, page_size, head_dim]
    (one (page, head) is a contiguous tile), a latent vector of shape (r,) with token_axis 0 in
    [pages, page_size, r], where row ``slot_map[t]`` of the [pages * page_size, r] view is token t's.
    ``dtype`` None: the engine's compute type.
    """
    name: str
    shape: Tuple[int, ...]
    token_axis: int = 0
    dtype: Optional[torch.dtype] = None

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        if not (0 <= self.token_axis <= len(self.shape)):
            raise ValueError(f"cached tensor '{self.name}': token_axis {self.token_axis} outside its shape {self.shape}")
        return tuple(self.shape[:self.token_axis]) + (int(page_size),) + tuple(self.shape[self.token_axis:])

    def bytes_per_token(self, compute_dtype: torch.dtype) -> int:
        n = 1
        for d in self.shape:
            n *= int(d)
        return n * torch.empty((), dtype=self.dtype or compute_dtype).element_size()


@dataclasses.dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps of every token, in pages: any number of named tensors.

    ``window`` None: a query may read every earlier token, pages live as long as
    the request.  ``window`` W: a query at position p reads tokens p-W+1 .. p;
    pages wholly before that are given back while the request runs.  Layers
    with equal (window) share a page pool and block tables (a cache group);
    each layer has its own tensors of its own geometry.
    """
    tensors: Tuple[CachedTensor, ...]
    window: Optional[int] = None

    @classmethod
    def keys_and_values(cls, kv_heads: int, head_dim: int, window: Optional[int] = None) -> "CacheNeed":
        """Keys "k" and values "v" of an attention layer: [pages, kv_heads, page_size, head_dim] each."""
        shape = (int(kv_heads), int(head_dim))
        return cls((CachedTensor("k", shape, token_axis=1), CachedTensor("v", shape, token_axis=1)), window)

    @property
    def group_key(self):
        return ("window", self.window) if self.window is not None else ("all",)

    def bytes_per_token(self, compute_dtype: torch.dtype) -> int:
        return sum(t.bytes_per_token(compute_dtype) for t in self.tensors)


@dataclasses.dataclass(frozen=True)
class StateNeed:
    """A tensor of fixed shape per request (zeroed when a request gets its slot)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def bind(self, rt, fetch: Callable[[str], torch.Tensor]) -> None:
        pass

    #: False if forward() reads host-side values of the step (then a decode
    #: step with this part is never replayed from a CUDA graph)
    graph_safe = True


class Residual:
    """The residual stream of a step: ``h`` (float [T, D]) and a delta not yet added.

    A mixer or feed-forward hands its output over as ``pending``; the next norm
    adds it to ``h`` in the same pass in which it normalises (the sum is done in
    float).
    """

    def __init__(self, h: torch.Tensor):
        self.h = h
        self.pending: Optional[torch.Tensor] = None
        # A product that ended a mixer or a feed-forward may have done the sum itself and left the rows of the
        # norm that follows short of their factor (``UnscaledRows``); the norm's ``fold`` hands them on or
        # finishes them.  ``takes_unscaled`` says whether the part that the next ``fold`` serves takes such
        # rows; ``next_norm`` is the norm that the block after this one starts with (None: unknown).
        self.unscaled: Optional["UnscaledRows"] = None
        self.takes_unscaled = False
        self.next_norm = None
        # (norm, rows): the rows of ``norm`` are there already (the embedding wrote them with the stream)
        self.ready = None


class UnscaledRows:
    """The rows of a step after a norm of the form y = x * f(x) * w, without the factor f(x) of each row.

    A product is linear, so the factor can be applied to its result instead (before any activation): the
    kernels that take such rows do that, and the norm needs no kernel of its own.  ``x`` [T, dim] holds
    x * w in the compute type; ``ssq`` [16, parts] (float) partial sums of x^2 of each of the (at most 16)
    rows; the factor of row t is 1 / sqrt(sum_p ssq[t, p] / dim + eps).  ``finish()`` returns the normed rows
    as a plain tensor for a consumer that has no such kernel (``Runtime.rows`` calls it)."""

    def __init__(self, x, ssq, parts: int, dim: int, eps: float, norm, finish):
        self.x, self.ssq, self.parts, self.dim, self.eps, self.norm, self._finish = x, ssq, parts, dim, eps, norm, finish
        self.shape = x.shape

    @property
    def scale(self):
        return (self.ssq, self.parts, self.dim, self.eps)

    def finish(self):
        return self._finish()


class ResidualSink:
    """Where the last product of a mixer or feed-forward may put its result instead of returning it: added
    into ``stream.h``, with the rows of ``norm`` (the norm that folds the stream next) left as
    ``stream.unscaled``.  A part that ignores it changes nothing: what it returns becomes ``pending``."""

    def __init__(self, stream: Residual, norm):
        self.stream, self.norm = stream, norm


class Norm(Part):
    def fold(self, stream: Residual, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None):
        """h += pending, then return norm(h) in the compute type.

        With ``rows`` (int32 indices) only those rows are normalised and ``h`` is left as it is."""
        raise NotImplementedError

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        """norm over the last axis of a tensor of the compute type."""
        raise NotImplementedError


class PositionEncoding(Part):
    """How positions enter a mixer.

    The attention kernels know ONE rotation: pairs (j, j + head_dim / 2) of a head turned by the angle
    position * table[j].  Every encoding of the rotary family fits that form through two things it states:

    * ``rotary_table()``: float [head_dim / 2], the inverse frequency of each of the kernels' pairs (0 = the
      pair is not rotated), or None for no rotation at all;
    * ``head_permutation()``: which of the head's own coordinates sits at each place of the kernels' layout
      (None = as they are).  A mixer applies it to the rows of its query and key projections (and to the
      per-head norm weights) when it binds its weights; scores q.k do not change when q and k are permuted
      alike, values are not touched.  Partial rotation (the first r coordinates, pairs (i, i + r / 2)) and
      interleaved pairs (2i, 2i + 1) are permutations plus a table; see ``parts.position``.

    An encoding that changes scores by something else than a rotation of q and k (a bias that depends on
    the distance, say) states it in ``score_bias()``; the attention kernels here have no such argument and
    the package's mixer refuses it.
    """

    def rotary_table(self) -> Optional[torch.Tensor]:
        raise NotImplementedError

    def head_permutation(self) -> Optional[List[int]]:
        return None

    def score_bias(self):
        return None


class Mixer(Part):
    takes_unscaled = False   # True: ``forward`` hands x to ``Runtime.linear`` as it comes (it may be UnscaledRows)

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, x: torch.Tensor, step, cache, state) -> torch.Tensor:
        """x [T, D] (compute type) -> delta [T, D].

        ``step`` is the StepContext; ``cache`` the LayerCache of this run entry
        (or None); ``state`` the [max_requests, *shape] state tensor (or None),
        indexed by ``step.state_slot``.
        """
        raise NotImplementedError


class FeedForward(Part):
    takes_unscaled = False   # as for a mixer

    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """An arrangement of mixer, feed-forward and norms around the residual stream."""

    mixer: Mixer

    def forward(self, stream: Residual, step, cache, state) -> None:
        raise NotImplementedError
