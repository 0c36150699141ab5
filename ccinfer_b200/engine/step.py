"""The batch of one step as the device sees it.

7QiC/ccInfer's translator builds seven int32 arrays per step and uploads each
to a fresh allocation (src/worker/batch_translator.cpp:241-431).  Here all
arrays of a step live at fixed offsets of ONE pinned host buffer and ONE device
buffer of fixed size: a step is one host-to-device copy, and because nothing
moves, a decode step can be replayed from a CUDA graph.

  token_ids[T]       the tokens the step brings, entries one after another (single-token entries first)
  positions[T]       absolute position of each token in its request
  entry_of_token[T]  which entry (request) a token belongs to; -1 for padding
  logit_rows[R]      token rows whose logits are wanted
  cu_q[B+1]          first token row of each entry (exclusive prefix sum)
  pos0[B]            position of the entry's first token (= tokens cached before)
  ctx_after[B]       tokens cached after the step (= pos0 + count)
  state_slot[B]      the request's state slot; -1 for padding
  per cache group:   slot_map[T] (where each token's k/v go; -1 = nowhere) and
                     block_table[B, stride] (logical page -> physical page, -1 = none)

The reference finds a token's request by a linear scan of query_start_loc
(src/kernel/attention/prefill_attn.cu:80-83); entry_of_token replaces that.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional

import numpy as np
import torch


@dataclasses.dataclass
class GroupStep:
    """A cache group's part of a step."""
    index: int
    page_size: int
    num_pages: int
    window: Optional[int]
    slot_map: torch.Tensor       # int32 [T]
    block_table: torch.Tensor    # int32 [B, stride] (a view with row stride = the full stride)
    host_slot_map: np.ndarray
    host_block_table: np.ndarray


@dataclasses.dataclass
class LayerCache:
    """What a mixer gets of the cache: the paged tensors it asked for in ``cache_need()`` (by name, each
    [pages, *page shape]) and its group's step arrays."""
    tensors: Dict[str, torch.Tensor]
    group: GroupStep
    own: bool                    # False: the pages belong to another run entry; read only

    @property
    def k(self) -> torch.Tensor:
        """Keys of an attention layer: [pages, kv_heads, page_size, head_dim]."""
        return self.tensors["k"]

    @property
    def v(self) -> torch.Tensor:
        return self.tensors["v"]


class StepContext:
    """Views (device) and arrays (host) of the current step; see the module docstring."""

    def __init__(self):
        self.n_tokens = 0
        self.n_entries = 0
        self.n_logit_rows = 0
        self.n_single = 0        # the first n_single entries (and token rows) bring one token each
        self.max_q_len = 0       # host facts for kernels that choose a launch shape
        self.max_ctx = 0
        self.token_ids = self.positions = self.entry_of_token = self.logit_rows = None
        self.cu_q = self.pos0 = self.ctx_after = self.state_slot = None
        self.row_slot = None        # request slot of each logits row
        self.pending_tokens = None  # int32 [slots]: the token last sampled per request slot (token id -1 - s)
        self.groups: List[GroupStep] = []
        self.host = None         # host copies of the same arrays
        self.residual_sink = None   # parts.base.ResidualSink offered to the last product of the part that runs

    def take_sink(self):
        """The sink offered to the part that is running, once (the part's LAST product may use it)."""
        sink, self.residual_sink = self.residual_sink, None
        return sink
