"""Dense gated feed-forward: m = (silu(x Wg^T) * (x Wu^T)) Wd^T, no bias
(7QiC/ccInfer: src/model/qwen3/qwen3_model.cpp:325-384, src/kernel/mlp/silu_mul.cu:24-28).

The reference runs gate and up as two matrix products; here they are one
merged matrix [2F, D] and one product.  Where F is a multiple of 64 the rows
are laid out in blocks (64 of gate, the 64 of up for the same channels) so that
a tile of the tensor-core product owns matching channels and the activation
can be its epilogue; otherwise gate rows first, then up rows.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import FeedForward, TensorSpec


class SwiGLU(FeedForward):
    takes_unscaled = True

    def __init__(self, hidden: int, intermediate: int, names: dict):
        """``names``: tensor names under the keys gate, up, down."""
        self.hidden, self.inter, self.names = int(hidden), int(intermediate), dict(names)
        self.w_gate_up = self.w_down = None
        self.rt = None

    def tensor_specs(self):
        n = self.names
        return [TensorSpec(n["gate"], (self.inter, self.hidden)), TensorSpec(n["up"], (self.inter, self.hidden)),
                TensorSpec(n["down"], (self.hidden, self.inter))]

    def bind(self, rt, fetch):
        self.rt = rt
        gate, up = fetch(self.names["gate"]), fetch(self.names["up"])
        self.block = kernels.SWIGLU_BLOCK if self.inter % kernels.SWIGLU_BLOCK == 0 else 0
        if self.block:
            self.w_gate_up = kernels.interleave_gate_up(gate, up, self.block)
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = fetch(self.names["down"])

    def forward(self, x, step):
        rt = self.rt
        T = x.shape[0]
        act = rt.scratch.get("ffn_act", (rt.max_tokens, self.inter), rt.dtype)[:T]
        rt.gated_up(act, x, self.w_gate_up, self.block)
        out = rt.scratch.get("ffn_out", (rt.max_tokens, self.hidden), rt.dtype)[:T]
        return rt.linear(out, act, self.w_down, sink=step.take_sink())
