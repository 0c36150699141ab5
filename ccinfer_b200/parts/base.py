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

* ``cache_need()``: keys and values per token, kept in pages (all of them, or a
  window), or None;
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
class CacheNeed:
    """Keys and values of every token, kept in pages.

    ``window`` None: a query may read every earlier key, pages live as long as
    the request.  ``window`` W: a query at position p reads keys p-W+1 .. p;
    pages wholly before that are given back while the request runs.  Layers
    with equal (window) share a page pool and block tables (a cache group);
    each layer has its own key and value tensors of its own geometry.
    """
    kv_heads: int
    head_dim: int
    window: Optional[int] = None

    @property
    def group_key(self):
        return ("window", self.window) if self.window is not None else ("all",)


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


class Norm(Part):
    def fold(self, stream: Residual, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None):
        """h += pending, then return norm(h) in the compute type.

        With ``rows`` (int32 indices) only those rows are normalised and ``h`` is left as it is."""
        raise NotImplementedError

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        """norm over the last axis of a tensor of the compute type."""
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary_table(self) -> Optional[torch.Tensor]:
        """Float inverse frequencies [head_dim / 2] for a rotate-half rotation, or None for none."""
        raise NotImplementedError


class Mixer(Part):
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
    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """An arrangement of mixer, feed-forward and norms around the residual stream."""

    mixer: Mixer

    def forward(self, stream: Residual, step, cache, state) -> None:
        raise NotImplementedError
