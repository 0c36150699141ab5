"""A model as data: its blocks and the order in which they run."""
from __future__ import annotations

import dataclasses
from typing import List, Optional

from ..parts.base import Block, Norm, Part


@dataclasses.dataclass
class RunEntry:
    """One position in the running order.

    ``layer`` indexes ``ModelPlan.layers``; naming a layer in two entries runs
    its weights twice, each run with a cache of its own.  ``cache_of`` names an
    earlier entry of the order whose cache this run reads instead of keeping
    one (its mixer then writes no keys or values).
    """
    layer: int
    cache_of: Optional[int] = None


@dataclasses.dataclass
class ModelPlan:
    embedding: Part          # forward(step) -> Residual
    layers: List[Block]
    order: List[RunEntry]
    final_norm: Norm
    head: Part               # forward(x_rows) -> float logits
    vocab_size: int
    max_position: Optional[int] = None

    def parts(self):
        return [self.embedding] + list(self.layers) + [self.final_norm, self.head]

    def tensor_specs(self):
        """All tensors of the model, each name once (a tied head names the embedding's tensor again)."""
        seen = {}
        for part in self.parts():
            for spec in part.tensor_specs():
                old = seen.get(spec.name)
                if old is not None and old.shape != spec.shape:
                    raise ValueError(f"tensor '{spec.name}' is wanted with shapes {old.shape} and {spec.shape}")
                seen.setdefault(spec.name, spec)
        return list(seen.values())

    def shared_tensor_names(self):
        """Names that more than one part wants (a tied head and its embedding)."""
        count = {}
        for part in self.parts():
            for spec in part.tensor_specs():
                count[spec.name] = count.get(spec.name, 0) + 1
        return {n for n, c in count.items() if c > 1}

    def validate(self):
        for i, e in enumerate(self.order):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"order[{i}] names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ValueError(f"order[{i}] reads the cache of entry {e.cache_of}, which does not run before it")
                if self.order[e.cache_of].cache_of is not None:
                    raise ValueError(f"order[{i}] reads the cache of entry {e.cache_of}, which has none of its own")
