"""Position encodings.

RotaryHalf: rotate-half rotation over the whole head,
inv_freq[i] = 1 / theta^(2i / head_dim), angle = float(pos) * inv_freq[i]
(7QiC/ccInfer: src/model/rope/rope_cache.cpp:31-45, src/kernel/pos/rope.cu:41-46).
The reference tabulates cos and sin for every position up to
max_position_embeddings on the host; here only the inverse frequencies are a
table (evaluated in float64, rounded once to float) and the kernel takes sine
and cosine of the float angle, so no position bound comes from a table.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import PositionEncoding


class RotaryHalf(PositionEncoding):
    def __init__(self, head_dim: int, theta: float):
        if head_dim % 2:
            raise ValueError("rotate-half needs an even head size")
        self.head_dim, self.theta = int(head_dim), float(theta)
        self.inv_freq = None
        self.rt = None

    def bind(self, rt, fetch):
        self.rt = rt
        i = torch.arange(0, self.head_dim, 2, dtype=torch.float64)
        inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), i / self.head_dim)
        self.inv_freq = inv.to(torch.float32).to(rt.device)

    def rotary_table(self):
        return self.inv_freq

    def apply(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Rotates x [T, H, head_dim] on its own (the attention mixer fuses this with its cache write)."""
        T, H, hd = x.shape
        out = torch.empty_like(x)
        kernels.qk_norm_rope_kv_write(x.view(T, H * hd), out, None, None, positions, None, self.inv_freq, None,
                                      None, 1.0, H, 0, hd, 1)
        return out


class NoPosition(PositionEncoding):
    """No position encoding at all."""

    def rotary_table(self):
        return None
