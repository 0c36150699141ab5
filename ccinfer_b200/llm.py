"""The Python entry point: a model folder in, token ids in, token ids out.

7QiC/ccInfer is started as ``ccinfer-server --model-path PATH [--port N]
[--prefill-chunk-size N]`` and takes requests over HTTP with ``max_tokens``,
``temperature``, ``top_p``, ``top_k`` (src/main.cpp:33-61,
src/http/http_server.cpp:529-555).  There is no server here; the same names
are the arguments of ``LLM`` and ``SamplingParams``, and prompts are token ids
(the tokenizer is not part of the engine).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

from .engine.engine import Engine, EngineOptions
from .engine.scheduler import SamplingParams, Scheduler


class LLM:
    def __init__(self, model_path: Optional[str] = None, dtype: str = "bfloat16", prefill_chunk_size: int = 512,
                 page_size: int = 16, kv_tokens: Optional[int] = None, kv_memory_fraction: Optional[float] = None,
                 max_requests: int = 64,
                 max_tokens_per_step: int = 4096, max_context: Optional[int] = None, max_running: int = 16,
                 eos_token_id: Optional[int] = None, device: str = "cuda:0", use_graphs: bool = True,
                 warm_up: bool = False, engine: Optional[Engine] = None):
        """``model_path``: a folder with config.json and model.safetensors (the model class is chosen by
        config.json).  ``prefill_chunk_size``: most prompt tokens of one request in a step, 0 = whole prompts.
        ``warm_up``: capture the decode graphs of every batch size up to ``max_running`` now, not at the first
        step that needs one.  An ``engine`` built elsewhere (for instance ``Engine.from_random``) may be passed
        instead of a path."""
        if engine is None:
            if model_path is None:
                raise ValueError("model_path (or an engine) is required")
            engine = Engine.from_model_dir(model_path, EngineOptions(
                dtype=dtype, device=device, page_size=page_size, kv_tokens=kv_tokens,
                kv_memory_fraction=kv_memory_fraction, max_requests=max_requests,
                max_tokens_per_step=max_tokens_per_step, max_context=max_context, use_graphs=use_graphs))
        self.engine = engine
        if warm_up:
            engine.warm_up(range(1, max_running + 1))
        self.scheduler = Scheduler(engine, prefill_chunk_size=prefill_chunk_size,
                                   max_tokens_per_step=min(max_tokens_per_step, engine.options.max_tokens_per_step),
                                   max_running=max_running, eos_token_id=eos_token_id,
                                   run_ahead=hasattr(engine, "sample_async"))
        self._next_id = 0

    @classmethod
    def from_random(cls, config, weights_seed: int = 0, weights_std: float = 0.02, **options) -> "LLM":
        """A model of a typed configuration (or of a config.json dictionary) with the random weights that
        (weights_seed, weights_std) name, drawn on the device; ``options`` as for the constructor."""
        if isinstance(config, dict):
            from .config.registry import architecture_of
            config = architecture_of(config).parse_config(config)
        names = ("dtype", "device", "page_size", "kv_tokens", "kv_memory_fraction", "max_requests",
                 "max_tokens_per_step", "max_context", "use_graphs")
        engine = Engine.from_random(config, weights_seed, weights_std,
                                    EngineOptions(**{k: options[k] for k in names if k in options}))
        return cls(engine=engine, **options)

    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[List[int]]:
        """New token ids for each prompt (lists of token ids), in the order given."""
        if sampling_params is None:
            sampling_params = SamplingParams()
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams for all prompts, or one per prompt")
        ids = []
        for prompt, sp in zip(prompts, sampling_params):
            rid = f"gen-{self._next_id}"
            self._next_id += 1
            self.scheduler.submit(rid, [int(t) for t in prompt], sp)
            ids.append(rid)
        out = self.scheduler.run()
        self.engine.check()
        return [out.get(rid, []) for rid in ids]

    # -- the same, a step at a time ---------------------------------------------------------
    def add_request(self, prompt: Sequence[int], sampling_params: Optional[SamplingParams] = None, req_id=None):
        """Queues a request; returns its id (``req_id`` or a fresh one)."""
        if req_id is None:
            req_id = f"gen-{self._next_id}"
            self._next_id += 1
        self.scheduler.submit(req_id, [int(t) for t in prompt], sampling_params)
        return req_id

    def cancel(self, req_id) -> bool:
        return self.scheduler.cancel(req_id)

    def step(self):
        """One scheduler step; the events it returns (``TokenEvent(req_id, token, finished, reason)``) are those
        of the step before it when the scheduler runs one step ahead."""
        return self.scheduler.step()

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def forward(self, entries):
        """The raw step, for tests: ``entries`` = [(request id, its next tokens, places whose logits are wanted)];
        requests are opened at their first entry (close them with ``engine.close_request``).  Returns the float
        logits [wanted, vocab] on the host."""
        from .engine.engine import StepEntry
        batch = []
        for e in entries:
            e = e if isinstance(e, StepEntry) else StepEntry(*e)
            if e.req_id not in self.engine.cache.requests:
                self.engine.open_request(e.req_id)
            batch.append(e)
        return self.engine.step(batch).cpu().numpy()

    def stats(self) -> dict:
        s = self.engine.stats()
        s["scheduler_steps"] = self.scheduler.steps
        s["preemptions"] = self.scheduler.preemptions
        return s
