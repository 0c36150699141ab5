"""Arrangements of parts in a block.

PreNormBlock: a = Mixer(norm1(h)); h += a; m = FeedForward(norm2(h)); h += m
(7QiC/ccInfer: src/model/qwen3/qwen3_model.cpp:141-396).  Each sum is folded
into the norm that follows it, the last one into the model's final norm.
The last product of the mixer and of the feed-forward is offered a
``ResidualSink``: with few rows it adds its result to the stream itself and the
norm after it needs no kernel (``parts.base.UnscaledRows``).
"""
from __future__ import annotations

from .base import Block, FeedForward, Mixer, Norm, Residual, ResidualSink


class PreNormBlock(Block):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in (self.norm1, self.mixer, self.norm2, self.ffn))

    def tensor_specs(self):
        return (self.norm1.tensor_specs() + self.mixer.tensor_specs() + self.norm2.tensor_specs()
                + self.ffn.tensor_specs())

    def bind(self, rt, fetch):
        for p in (self.norm1, self.mixer, self.norm2, self.ffn):
            p.bind(rt, fetch)

    @property
    def first_norm(self):
        return self.norm1

    def forward(self, stream: Residual, step, cache, state) -> None:
        after = stream.next_norm                     # the norm that the block after this one starts with
        stream.takes_unscaled = self.mixer.takes_unscaled
        x = self.norm1.fold(stream)
        step.residual_sink = ResidualSink(stream, self.norm2)
        stream.pending = self.mixer.forward(x, step, cache, state)
        stream.takes_unscaled = self.ffn.takes_unscaled
        x = self.norm2.fold(stream)
        step.residual_sink = ResidualSink(stream, after) if after is not None else None
        stream.pending = self.ffn.forward(x, step)
        step.residual_sink = None
        stream.takes_unscaled = False
