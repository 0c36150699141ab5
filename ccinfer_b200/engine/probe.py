"""A few eager steps of a random model at a chosen shape, for profilers.

    python -m ccinfer_b200.engine.probe --layers 2 --batch 8 --ctx 2048 --steps 2 [--prefill 2048]

Builds the Qwen3-8B layer shape (or the sizes given) with few layers and random weights, brings ``batch``
requests to ``ctx`` cached tokens, then runs ``steps`` decode steps without CUDA graphs (so that a
profiler sees every kernel) and, with ``--prefill N``, one prompt of N tokens in one step.  Small by
design: two layers hold about 1 GB on the device.
"""
from __future__ import annotations

import argparse
import sys

import numpy as np
import torch

from ..config.qwen3 import Qwen3Config
from .engine import Engine, EngineOptions, StepEntry


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--prefill", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--intermediate", type=int, default=12288)
    ap.add_argument("--vocab", type=int, default=151936)
    a = ap.parse_args(argv)
    cfg = Qwen3Config.from_json({
        "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": a.layers, "hidden_size": a.hidden,
        "num_attention_heads": a.heads, "num_key_value_heads": a.kv_heads, "head_dim": a.head_dim,
        "intermediate_size": a.intermediate, "vocab_size": a.vocab, "rope_theta": 1e6, "rms_norm_eps": 1e-6,
        "max_position_embeddings": 40960})
    longest = max(a.ctx + a.steps, a.prefill) + 64
    eng = Engine.from_random(cfg, 42, options=EngineOptions(
        dtype=a.dtype, kv_tokens=a.batch * (a.ctx + a.steps + 64) + a.prefill + 64, max_requests=a.batch + 1,
        max_tokens_per_step=max(2048, a.prefill, a.ctx), max_context=longest, use_graphs=False))
    rng = np.random.RandomState(0)
    for b in range(a.batch):
        eng.open_request(b)
        eng.step([StepEntry(b, rng.randint(0, cfg.vocab_size, size=a.ctx).tolist(), [])])
    torch.cuda.synchronize()
    for s in range(a.steps):
        eng.step([StepEntry(b, [5 + s], [0]) for b in range(a.batch)])
    torch.cuda.synchronize()
    if a.prefill:
        eng.open_request("p")
        eng.step([StepEntry("p", rng.randint(0, cfg.vocab_size, size=a.prefill).tolist(), [a.prefill - 1])])
        torch.cuda.synchronize()
    eng.check()
    print("probe ok", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
