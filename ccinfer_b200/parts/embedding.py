"""Token embedding and output head.

  h0[t, :] = E[ids[t], :]                 (7QiC/ccInfer: src/kernel/elementwise/elementwise.cu:67-78)
  logits = x W_lm^T in float              (src/model/qwen3/qwen3_model.cpp:412-426)

The head runs on the rows whose logits are wanted, not on every token of the
step as the reference does.  A tied head names the embedding's tensor as its
weight and then shares its storage.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, Residual, TensorSpec


class TokenEmbedding(Part):
    def __init__(self, vocab: int, hidden: int, weight_name: str):
        self.vocab, self.hidden, self.weight_name = int(vocab), int(hidden), weight_name
        self.table = None
        self.rt = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.vocab, self.hidden))]

    def bind(self, rt, fetch):
        self.rt = rt
        self.table = fetch(self.weight_name)

    takes_first_norm = True

    def forward(self, step, first_norm=None) -> Residual:
        """``first_norm``: the norm that folds the stream first; where it can, its rows are written by the
        same kernel as the stream (``stream.ready``)."""
        rt = self.rt
        h = rt.scratch.get("residual", (rt.max_tokens, self.hidden), torch.float32)[:step.n_tokens]
        pending = getattr(step, "pending_tokens", None)
        y = None
        if first_norm is not None and hasattr(first_norm, "from_embedding"):
            y = first_norm.from_embedding(h, self.table, step.token_ids, pending)
        if y is None:
            kernels.embed_gather(h, self.table, step.token_ids, status=rt.status, pending=pending)
        stream = Residual(h)
        if y is not None:
            stream.ready = (first_norm, y)
        return stream


class OutputHead(Part):
    def __init__(self, hidden: int, vocab: int, weight_name: str):
        self.hidden, self.vocab, self.weight_name = int(hidden), int(vocab), weight_name
        self.w = None
        self.rt = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.vocab, self.hidden))]

    def bind(self, rt, fetch):
        self.rt = rt
        self.w = fetch(self.weight_name)

    def forward(self, x_rows: torch.Tensor) -> torch.Tensor:
        rt = self.rt
        R = x_rows.shape[0]
        if R <= rt.max_entries:  # the decode case: a fixed buffer, so that the step can be replayed
            logits = rt.scratch.get("logits", (rt.max_entries, self.vocab), torch.float32)[:R]
        else:
            logits = torch.empty((R, self.vocab), dtype=torch.float32, device=rt.device)
        rt.linear(logits, x_rows, self.w)
        return logits
