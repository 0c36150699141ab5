"""Per-request sampling parameters.

Greedy (argmax, ties to the lowest id) and temperature sampling (a Gumbel-max
draw keyed by the request's seed and the number of tokens it has produced), the
draw restricted to the top-k logits and the top-p share of the probability where
asked, run in csrc/sampling.cu; Engine.sample() applies them to logits rows.
"""
from __future__ import annotations

import dataclasses

from ..errors import Unsupported


@dataclasses.dataclass
class SamplingParams:
    """Names, meanings and defaults of 7QiC/ccInfer's SamplingParams (src/base/types.h:54-60)."""
    max_tokens: int = 256       # generation limit
    top_k: int = 0              # 0 = off
    top_p: float = 1.0          # >= 1 = off
    temperature: float = 0.0    # <= 0 = greedy
    seed: int = 42

    def validate(self) -> None:
        # the reference refuses everything but greedy (src/model/model_runner.h:96-100); here temperature,
        # top_k and top_p are sampled with (they act on rows with a temperature above zero)
        if self.top_k < 0:
            raise Unsupported("top_k must be 0 (off) or a positive count")
        if not (0.0 < self.top_p):
            raise Unsupported("top_p must be above 0 (1 or more = off)")
