"""Per-request sampling parameters.

Greedy (argmax, ties to the lowest id) and temperature sampling (a Gumbel-max
draw keyed by the request's seed and the number of tokens it has produced) run
in csrc/sampling.cu; Engine.sample() applies them to logits rows.
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
        # the reference refuses everything but greedy (src/model/model_runner.h:96-100); temperature is added
        # here, top_k / top_p stay refused rather than ignored
        if self.top_k != 0 or self.top_p < 1.0:
            raise Unsupported("top_k / top_p sampling is not implemented (greedy and temperature are)")
