"""ccinfer_b200: a small, whole inference engine for one GPU (B200, sm_100a).

Typed configuration and registry (config), weights by name (weights), model
parts (parts), paged cache manager (cache), step function, scheduler and entry
points (engine, llm, cli), sampling, and hand-written CUDA (csrc).
"""
from .errors import CcinferError

__all__ = ["CcinferError", "LLM", "SamplingParams", "Engine", "EngineOptions", "StepEntry"]


def __getattr__(name):
    if name in ("Engine", "EngineOptions", "StepEntry"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name == "SamplingParams":
        from .engine.scheduler import SamplingParams
        return SamplingParams
    if name == "LLM":
        from .llm import LLM
        return LLM
    raise AttributeError(name)
