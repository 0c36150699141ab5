"""The Qwen3-8B layer shape (4 of its 36 layers, full vocabulary) under different ways of cutting the work.

No plain reference at this size: the engine is compared with itself.  In 32-bit the cuttings must agree to
round-off; the bfloat16 path is then judged against the 32-bit path.  This is where the tensor-core kernels
(tcgen05 products and attention, TMA page loads, head size 128, groups of 4 q heads, pages of 16) run inside
the engine with realistic strides and more keys than one tile.
"""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

SHAPE = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 4, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 40960, "torch_dtype": "bfloat16",
}


def _engine(dtype):
    from ccinfer_b200.config import Qwen3Config
    from ccinfer_b200.engine.engine import Engine, EngineOptions
    return Engine.from_random(Qwen3Config.from_json(SHAPE), seed=42, std=0.02, options=EngineOptions(
        dtype=dtype, page_size=16, kv_tokens=2048, max_requests=8, max_tokens_per_step=1024, max_context=1024))


def _last_rows(rows, reqs, n=40):
    return {k: v for k, v in rows.items() if k[1] >= len(reqs[k[0]]) - n}


def _worst(a, b):
    return max(float(np.abs(a[k] - b[k]).max()) / max(1e-6, float(np.abs(b[k]).max())) for k in a)


def test_cuttings_agree_at_the_8b_layer_shape():
    rng = np.random.RandomState(0)
    reqs = {f"r{i}": rng.randint(0, SHAPE["vocab_size"], size=n).tolist() for i, n in enumerate([300, 70, 513, 140])}
    want_tail = 40  # compare the last 40 positions of every request (a row of logits is 600 KB)

    def run(dtype, steps):
        # ask for logits only where they are compared
        for st in steps:
            for e in st["entries"]:
                e["want"] = [w for w in e["want"]]
        eng = _engine(dtype)
        rows = helpers.replay(eng, steps)
        eng.cache.check_consistency()
        out = _last_rows(rows, reqs, want_tail)
        del eng
        torch.cuda.empty_cache()
        return out

    def tail_only(steps):
        seen = {}
        for st in steps:
            for e in st["entries"]:
                base = seen.get(e["id"], 0)
                n = len(reqs[e["id"]])
                e["want"] = [w for w in e["want"] if base + w >= n - want_tail]
                seen[e["id"]] = base + len(e["tokens"])
        return steps

    whole32 = run("float32", tail_only(helpers.trace_whole(reqs)))
    mixed32 = run("float32", tail_only(helpers.trace_mixed(reqs, max_live=4, seed=4)))
    assert set(whole32) == set(mixed32) and len(whole32) == 4 * want_tail
    assert _worst(mixed32, whole32) <= 2e-5
    whole16 = run("bfloat16", tail_only(helpers.trace_whole(reqs)))
    dec16 = run("bfloat16", tail_only(helpers.trace_prefill_then_decode(reqs, tail=32)))
    mixed16 = run("bfloat16", tail_only(helpers.trace_mixed(reqs, max_live=4, seed=4)))
    for name, rows in (("whole", whole16), ("decode32", dec16), ("mixed", mixed16)):
        assert _worst(rows, whole32) <= 3e-2, name


MID_SHAPE = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 4, "head_dim": 64, "intermediate_size": 4096,
    "vocab_size": 3000, "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 4096, "torch_dtype": "bfloat16",
}


def test_cuttings_agree_at_a_mid_size_shape_with_head_size_64():
    """Hidden 2048, head size 64, groups of 8 q heads, 64 tiles of gate|up: the sizes at which the few-rows
    products of a decode or mixed step go to the TMA-ring kernel (q|k|v, o, down and, with fewer tiles than
    SMs, gate|up with the activation as its epilogue) while portions of more than 16 tokens go to the
    library.  bfloat16 under three cuttings against the 32-bit path."""
    from ccinfer_b200.config import Qwen3Config
    from ccinfer_b200.engine.engine import Engine, EngineOptions
    from ccinfer_b200 import kernels
    rng = np.random.RandomState(3)
    reqs = {f"r{i}": rng.randint(0, MID_SHAPE["vocab_size"], size=n).tolist() for i, n in enumerate([150, 41, 260, 77])}

    def run(dtype, steps):
        eng = Engine.from_random(Qwen3Config.from_json(MID_SHAPE), seed=5, std=0.03, options=EngineOptions(
            dtype=dtype, page_size=16, kv_tokens=1024, max_requests=8, max_tokens_per_step=512, max_context=512))
        before = kernels.counters.own
        rows = helpers.replay(eng, steps)
        eng.cache.check_consistency()
        assert kernels.counters.own > before
        del eng
        torch.cuda.empty_cache()
        return rows

    whole32 = run("float32", helpers.trace_whole(reqs))
    mixed32 = run("float32", helpers.trace_mixed(reqs, max_live=4, seed=6))
    assert set(whole32) == set(mixed32)
    assert _worst(mixed32, whole32) <= 2e-5
    for name, steps in (("whole", helpers.trace_whole(reqs)),
                        ("decode32", helpers.trace_prefill_then_decode(reqs, tail=32)),
                        ("portions", helpers.trace_portions(reqs)),
                        ("mixed", helpers.trace_mixed(reqs, max_live=4, seed=6))):
        rows = run("bfloat16", steps)
        assert set(rows) == set(whole32), name
        assert _worst(rows, whole32) <= 3e-2, name
