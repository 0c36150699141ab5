"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w (7QiC/ccInfer: src/kernel/norm/rms_norm.cu:24-60)."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Norm, Residual, TensorSpec


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

    def apply(self, x):
        y = torch.empty_like(x)  # the part alone, outside a step: not a buffer of the pool
        kernels.rmsnorm(y, x, self.w, self.eps)
        return y
