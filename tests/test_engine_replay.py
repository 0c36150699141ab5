"""The engine against the plain implementation under every way of cutting the work.

Each request alone and whole; most of it in one step and the last 32 tokens one
by one; in portions of changing size down to two tokens; mixed with up to four
live requests and so few pages that they are used again.  In 32-bit and in
bfloat16, for three tiny configurations.
"""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

# relative to the largest logit of the request
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
CONFIGS = ["A", "B", "C", "D", "E"]
LENGTHS = {"A": [5, 11, 17, 64, 120], "B": [1, 9, 33, 64, 150, 97], "C": [3, 40, 77, 130, 96, 51],
           "D": [2, 70, 200, 129, 64, 333], "E": [1, 65, 150, 300, 128]}


def _requests(cfg, lengths, seed=5):
    rng = np.random.RandomState(seed)
    return {f"r{i}": rng.randint(0, cfg["vocab_size"], size=n).tolist() for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in CONFIGS:
        d = str(tmp_path_factory.mktemp(f"tiny{name}"))
        cfg, weights, page = helpers.make_model_dir(d, name, store="bfloat16" if name != "B" else "float32")
        reqs = _requests(cfg, LENGTHS[name])
        ref = {rid: helpers.plain_logits(cfg, weights, toks) for rid, toks in reqs.items()}
        out[name] = (d, cfg, page, reqs, ref)
    return out


def _engine(model_dir, dtype, page, pool_tokens):
    from ccinfer_b200.engine.engine import Engine, EngineOptions
    return Engine.from_model_dir(model_dir, EngineOptions(
        dtype=dtype, page_size=page, kv_tokens=pool_tokens, max_requests=8, max_tokens_per_step=pool_tokens,
        max_context=pool_tokens, use_graphs=False))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", CONFIGS)
@pytest.mark.parametrize("mode", ["whole", "decode32", "portions", "mixed"])
def test_replay_matches_plain(models, name, dtype, mode):
    d, cfg, page, reqs, ref = models[name]
    if mode == "whole":
        steps = helpers.trace_whole(reqs)
    elif mode == "decode32":
        steps = helpers.trace_prefill_then_decode(reqs, tail=32)
    elif mode == "portions":
        steps = helpers.trace_portions(reqs)
    else:
        steps = helpers.trace_mixed(reqs, max_live=4, seed=11)
    # a pool just large enough: pages of finished requests are used again by later ones
    pool = helpers.max_live_tokens(steps, round_to=max(64, page))
    eng = _engine(d, dtype, page, pool)
    rows = helpers.replay(eng, steps)
    assert len(rows) == sum(len(t) for t in reqs.values())
    helpers.compare(rows, ref, TOL[dtype], f"tiny {name} {dtype} {mode}")
    eng.cache.check_consistency()
    assert all(p.used_pages == 0 for p in eng.cache.pools)


@pytest.mark.parametrize("name", CONFIGS)
def test_cuts_agree_in_float32(models, name):
    """The same position under two cuttings: equal to 32-bit round-off, far below the distance to bfloat16."""
    d, cfg, page, reqs, ref = models[name]
    a = helpers.replay(_engine(d, "float32", page, 1024), helpers.trace_whole(reqs))
    b = helpers.replay(_engine(d, "float32", page, 1024), helpers.trace_mixed(reqs, seed=3))
    worst = max(float(np.abs(a[k] - b[k]).max()) / max(1e-6, float(np.abs(ref[k[0]]).max())) for k in a)
    assert worst <= 1e-5, worst
