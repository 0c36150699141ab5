"""Dense gated feed-forward: m = (silu(x Wg^T) * (x Wu^T)) Wd^T, no bias
(7QiC/ccInfer: src/model/qwen3/qwen3_model.cpp:325-384, src/kernel/mlp/silu_mul.cu:24-28).

The reference runs gate and up as two matrix products; here they are one
merged matrix [2F, D] (gate rows first) and one product.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import FeedForward, TensorSpec


class SwiGLU(FeedForward):
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
        self.w_gate_up = torch.cat([fetch(self.names["gate"]), fetch(self.names["up"])], dim=0).contiguous()
        self.w_down = fetch(self.names["down"])

    def forward(self, x, step):
        rt = self.rt
        T = x.shape[0]
        gu = rt.scratch.get("ffn_gate_up", (rt.max_tokens, 2 * self.inter), rt.dtype)[:T]
        rt.linear(gu, x, self.w_gate_up)
        act = rt.scratch.get("ffn_act", (rt.max_tokens, self.inter), rt.dtype)[:T]
        kernels.silu_mul(act, gu)
        out = rt.scratch.get("ffn_out", (rt.max_tokens, self.hidden), rt.dtype)[:T]
        rt.linear(out, act, self.w_down)
        return out
