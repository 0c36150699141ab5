"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w (7QiC/ccInfer: src/kernel/norm/rms_norm.cu:24-60)."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Norm, Residual, TensorSpec, UnscaledRows


class RMSNorm(Norm):
    def __init__(self, dim: int, eps: float, weight_name: str, scratch_key: str = "normed"):
        self.dim, self.eps, self.weight_name, self.scratch_key = int(dim), float(eps), weight_name, scratch_key
        self.w = None
        self.rt = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.dim,), role="vector", init="one_plus_normal")]

    def bind(self, rt, fetch):
        self.rt = rt
        self.w = fetch(self.weight_name)

    def fold(self, stream: Residual, rows=None, n_rows=None):
        rt = self.rt
        T = stream.h.shape[0]
        ready, stream.ready = stream.ready, None
        if ready is not None and rows is None and ready[0] is self and stream.pending is None:
            return ready[1]   # written together with the stream (the embedding's kernel)
        un, stream.unscaled = stream.unscaled, None
        if un is not None and rows is None and un.norm is self and stream.pending is None:
            # the product before did the sum and left this norm's rows short of their factor
            return un if stream.takes_unscaled else un.finish()
        # (rows left for another norm than this one: h is complete, they are dropped)
        if rows is None:
            y = rt.scratch.get(self.scratch_key, (rt.max_tokens, self.dim), rt.dtype)[:T]
            kernels.residual_rmsnorm(y, stream.h, stream.pending, self.w, self.eps, status=rt.status)
            stream.pending = None  # it is part of h now
        else:
            n = rows.numel() if n_rows is None else n_rows
            y = rt.scratch.get(self.scratch_key + "_rows", (rt.max_tokens, self.dim), rt.dtype)[:n]
            kernels.residual_rmsnorm(y, stream.h, stream.pending, self.w, self.eps, row_idx=rows, n_rows=n,
                                     status=rt.status)
        return y

    def from_embedding(self, h, table, ids, pending):
        """norm(h) for h = table[ids], both written by one kernel; None where that kernel does not apply."""
        rt = self.rt
        if table.dtype != rt.dtype or table.shape[1] != self.dim or not table.is_contiguous():
            return None
        y = rt.scratch.get(self.scratch_key, (rt.max_tokens, self.dim), rt.dtype)[:h.shape[0]]
        kernels.embed_rmsnorm(y, h, table, ids, self.w, self.eps, status=rt.status, pending=pending)
        return y

    def unscaled_rows_from(self, stream: Residual, xw, ssq, parts: int):
        """What a product that adds into the stream itself leaves for this norm: ``xw`` gets h * w, ``ssq``
        [16, parts] the partial sums of h^2 (see ``Runtime.linear``).  None: this norm takes no such rows."""
        if xw.shape[1] != self.dim:
            return None
        h = stream.h
        return UnscaledRows(xw, ssq, parts, self.dim, self.eps, self, lambda: self.rows_of(h))

    def rows_of(self, h):
        """norm(h) of a stream that is complete (nothing pending), as a plain tensor."""
        rt = self.rt
        y = rt.scratch.get(self.scratch_key, (rt.max_tokens, self.dim), rt.dtype)[:h.shape[0]]
        kernels.residual_rmsnorm(y, h, None, self.w, self.eps, status=rt.status)
        return y

    def apply(self, x):
        y = torch.empty_like(x)  # the part alone, outside a step: not a buffer of the pool
        kernels.rmsnorm(y, x, self.w, self.eps)
        return y
