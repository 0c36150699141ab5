"""Position encodings.

RotaryHalf: rotate-half rotation over the whole head,
inv_freq[i] = 1 / theta^(2i / head_dim), angle = float(pos) * inv_freq[i]
(7QiC/ccInfer: src/model/rope/rope_cache.cpp:31-45, src/kernel/pos/rope.cu:41-46).
The reference tabulates cos and sin for every position up to
max_position_embeddings on the host; here only the inverse frequencies are a
table and the kernel takes sine and cosine of the float angle, so no position
bound comes from a table.  The frequencies are evaluated as the reference
does, in 32-bit steps: exponent = float(2i) / float(head_dim), theta^exponent
rounded to float, 1.0f / that (a model trained with a 32-bit table sees the
frequencies it was trained with; evaluating in float64 and rounding once gives
another float for a third of the entries).  The power is taken in float64 and
rounded, i.e. correctly rounded, where the reference's powf is within an ulp.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import kernels
from .base import PositionEncoding


def rotary_inv_freq(rotary_dim: int, theta: float) -> np.ndarray:
    """float32 [rotary_dim / 2]: 1.0f / powf(theta, float(2i) / float(rotary_dim)), every step in 32 bits
    (src/model/rope/rope_cache.cpp:31-35)."""
    exponent = np.arange(0, rotary_dim, 2, dtype=np.float32) / np.float32(rotary_dim)
    power = np.power(np.float64(np.float32(theta)), exponent.astype(np.float64)).astype(np.float32)
    return (np.float32(1.0) / power).astype(np.float32)


class RotaryHalf(PositionEncoding):
    """Rotate-half rotation of the first ``rotary_dim`` coordinates of a head (default: all of them, as the
    reference: src/kernel/pos/rope.cu:37-46 pairs (i, i + head_dim / 2)).

    ``rotary_dim`` < head_dim: pairs (i, i + rotary_dim / 2), the other coordinates pass through.
    ``interleaved``: pairs (2i, 2i + 1) instead.  Both are a permutation of the head's coordinates into the
    kernels' layout plus a table with zeros for the pairs that do not turn (see PositionEncoding).
    """

    def __init__(self, head_dim: int, theta: float, rotary_dim: int = None, interleaved: bool = False):
        rotary_dim = int(head_dim if rotary_dim is None else rotary_dim)
        if head_dim % 2 or rotary_dim % 2 or not (0 < rotary_dim <= head_dim):
            raise ValueError(f"rotation of {rotary_dim} of {head_dim} coordinates: both even, 0 < rotary_dim <= head_dim")
        self.head_dim, self.theta, self.rotary_dim, self.interleaved = int(head_dim), float(theta), rotary_dim, interleaved
        self.inv_freq = None
        self.rt = None

    def bind(self, rt, fetch):
        self.rt = rt
        table = np.zeros(self.head_dim // 2, dtype=np.float32)
        table[:self.rotary_dim // 2] = rotary_inv_freq(self.rotary_dim, self.theta)
        self.inv_freq = torch.from_numpy(table).to(rt.device)

    def rotary_table(self):
        return self.inv_freq

    def head_permutation(self):
        hd, rd, half = self.head_dim, self.rotary_dim, self.head_dim // 2
        if rd == hd and not self.interleaved:
            return None
        # the kernels' pair j is places (j, j + half): the rotated pairs first, then the rest in pairs of its own
        firsts = [2 * i for i in range(rd // 2)] if self.interleaved else list(range(rd // 2))
        seconds = [2 * i + 1 for i in range(rd // 2)] if self.interleaved else [i + rd // 2 for i in range(rd // 2)]
        rest = list(range(rd, hd))
        firsts += rest[:len(rest) // 2]
        seconds += rest[len(rest) // 2:]
        assert len(firsts) == len(seconds) == half
        return firsts + seconds

    def apply(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Rotates x [T, H, head_dim] on its own (the attention mixer fuses this with its cache write)."""
        T, H, hd = x.shape
        perm = self.head_permutation()
        if perm is not None:
            idx = torch.tensor(perm, device=x.device)
            x = x[..., idx].contiguous()
        out = torch.empty_like(x)
        kernels.qk_norm_rope_kv_write(x.view(T, H * hd), out, None, None, positions, None, self.inv_freq, None,
                                      None, 1.0, H, 0, hd, 1)
        if perm is not None:
            back = torch.empty_like(idx)
            back[idx] = torch.arange(hd, device=x.device)
            out = out[..., back].contiguous()
        return out


class NoPosition(PositionEncoding):
    """No position encoding at all."""

    def rotary_table(self):
        return None
