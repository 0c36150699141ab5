"""The engine against the plain implementation under every way of cutting the work.

Each request alone and whole; most of it in one step and the last 32 tokens one
by one; in portions of changing size down to two tokens; mixed with up to four
live requests and so few pages that they are used again.  In 32-bit and in
bfloat16, for three tiny configurations.
"""
import numpy as np
import pytest

import helpers

pytestmark = pytest.mark.gpu

# relative to the largest logit of the request; bfloat16: about twice the worst a B200 run has shown for the
# configuration (every test prints its own as "[worst] ...")
TOL = {"float32": 2e-5}   # seen: 1.2e-6 at most
TOL16 = {"A": 6e-3, "B": 1.3e-2, "C": 1.5e-2, "D": 1.5e-2, "E": 1.6e-2}   # seen: 2.6e-3, 6.4e-3, 7.5e-3, 7.1e-3, 8.0e-3


def _tol(name, dtype):
    return TOL["float32"] if dtype == "float32" else TOL16[name]

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
        out[name] = (d, cfg, page, reqs, ref, weights)
    return out


def _engine(model_dir, dtype, page, pool_tokens, use_graphs=False, max_requests=8, max_tokens_per_step=None):
    from ccinfer_b200.engine.engine import Engine, EngineOptions
    return Engine.from_model_dir(model_dir, EngineOptions(
        dtype=dtype, page_size=page, kv_tokens=pool_tokens, max_requests=max_requests,
        max_tokens_per_step=max_tokens_per_step or pool_tokens, max_context=pool_tokens, use_graphs=use_graphs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", CONFIGS)
@pytest.mark.parametrize("mode", ["whole", "decode32", "portions", "mixed"])
def test_replay_matches_plain(models, name, dtype, mode):
    d, cfg, page, reqs, ref, _ = models[name]
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
    worst = helpers.compare(rows, ref, _tol(name, dtype), f"tiny {name} {dtype} {mode}")
    print(f"[worst] tiny {name}, {dtype}, {mode}: {worst:.3e}")
    eng.cache.check_consistency()
    assert all(p.used_pages == 0 for p in eng.cache.pools)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "E"])
@pytest.mark.parametrize("mode", ["decode32", "mixed", "long portions"])
def test_replay_from_graphs_matches_plain(models, name, dtype, mode):
    """Decode steps replayed from CUDA graphs (three live requests in a graph of four: one padding row) and
    portions of more than 64 tokens after a cached prefix beside them, on the tensor-core attention kernels
    of the bfloat16 path (head size 64 and 128)."""
    d, cfg, page, reqs, ref, _ = models[name]
    if mode == "decode32":
        three = {rid: reqs[rid] for rid in list(reqs)[1:4]}
        steps = helpers.trace_many_decoders(three, decode_steps=32, per_prefill_step=2)
    elif mode == "mixed":
        steps = helpers.trace_mixed(reqs, max_live=3, seed=12, prefill_frac=0.3)
    else:
        steps = helpers.trace_mixed(reqs, max_live=3, seed=13, prefill_frac=0.8, portion_choices=(70, 130, 65, 2, 100))
    pool = helpers.max_live_tokens(steps, round_to=max(64, page))
    eng = _engine(d, dtype, page, pool, use_graphs=True)
    rows = helpers.replay(eng, steps)
    worst = helpers.compare(rows, ref, _tol(name, dtype), f"tiny {name} {dtype} graphs {mode}")
    print(f"[worst] tiny {name}, {dtype}, graphs, {mode}: {worst:.3e}")
    assert eng.graph_replays > 0 and (mode != "decode32" or 4 in eng._graphs)
    eng.cache.check_consistency()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "E"])
@pytest.mark.parametrize("n_live", [17, 33, 48, 49, 64])
@pytest.mark.parametrize("graphs", [False, True])
def test_many_decoding_requests_match_plain(models, name, dtype, n_live, graphs):
    """Decode steps of 17 to 64 rows: from 17 rows on the products of the bfloat16 path go to the library,
    from 49 on the attention is no longer fused with the rotation and the cache write, and the graphs of 32
    and 64 rows are captured."""
    d, cfg, page = models[name][:3]
    rng = np.random.RandomState(n_live)
    reqs = {f"m{i}": rng.randint(0, cfg["vocab_size"], size=int(rng.randint(8, 60))).tolist() for i in range(n_live)}
    weights = models[name][5]
    ref = {rid: helpers.plain_logits(cfg, weights, toks) for rid, toks in reqs.items()}
    steps = helpers.trace_many_decoders(reqs, decode_steps=5)
    pool = helpers.max_live_tokens(steps, round_to=max(64, page))
    eng = _engine(d, dtype, page, pool, use_graphs=graphs, max_requests=64, max_tokens_per_step=512)
    rows = helpers.replay(eng, steps)
    assert len(rows) == sum(len(t) for t in reqs.values())
    worst = helpers.compare(rows, ref, _tol(name, dtype), f"tiny {name} {dtype} {n_live} decoding requests")
    print(f"[worst] tiny {name}, {dtype}, {n_live} decoding requests, graphs {graphs}: {worst:.3e}")
    assert (eng.graph_replays > 0) == graphs
    eng.cache.check_consistency()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graphs_when_the_request_limit_is_no_power_of_two(models, dtype):
    """Twenty-four request slots: steps of 17 to 24 decoding requests are replayed from a graph of 24 rows (the
    next power of two does not exist for this engine), smaller ones from graphs of 16 and below."""
    d, cfg, page = models["E"][:3]
    weights = models["E"][5]
    for n_live in (5, 17, 24):
        rng = np.random.RandomState(n_live)
        reqs = {f"m{i}": rng.randint(0, cfg["vocab_size"], size=int(rng.randint(8, 40))).tolist() for i in range(n_live)}
        ref = {rid: helpers.plain_logits(cfg, weights, toks) for rid, toks in reqs.items()}
        steps = helpers.trace_many_decoders(reqs, decode_steps=4)
        pool = helpers.max_live_tokens(steps, round_to=max(64, page))
        eng = _engine(d, dtype, page, pool, use_graphs=True, max_requests=24, max_tokens_per_step=512)
        rows = helpers.replay(eng, steps)
        helpers.compare(rows, ref, _tol("E", dtype), f"tiny E {dtype} {n_live} of 24 slots")
        assert eng.graph_replays >= 3 and sorted(eng._graphs) == [{5: 8, 17: 24, 24: 24}[n_live]]
        eng.cache.check_consistency()
    assert eng._all_buckets() == [1, 2, 4, 8, 16, 24] and eng._bucket_of(25) == 0


@pytest.mark.parametrize("name", CONFIGS)
def test_cuts_agree_in_float32(models, name):
    """The same position under two cuttings: equal to 32-bit round-off, far below the distance to bfloat16."""
    d, cfg, page, reqs, ref, _ = models[name]
    a = helpers.replay(_engine(d, "float32", page, 1024), helpers.trace_whole(reqs))
    b = helpers.replay(_engine(d, "float32", page, 1024), helpers.trace_mixed(reqs, seed=3))
    worst = max(float(np.abs(a[k] - b[k]).max()) / max(1e-6, float(np.abs(ref[k[0]]).max())) for k in a)
    assert worst <= 1e-5, worst


SHARPEN = 8.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "E"])
def test_sharp_attention_shows_every_key(tmp_path_factory, name, dtype):
    """Scores eight times larger: a query's attention sits on one or two keys somewhere in its context (with
    scores of deviation 8 the best of 400 keys outweighs all others together), so a key that was dropped,
    misplaced or read from a stale page moves the logits by about their own size, where the flat attention
    of small random weights gives one key in hundreds less than the bfloat16 tolerance.  Long requests, mixed
    steps with pages used again, long portions and graphs, all against the plain implementation.

    The bounds are those of the ordinary replay tests times the same factor: an error of a query or a key
    reaches the score multiplied by it, and the score is the exponent of a weight."""
    d = str(tmp_path_factory.mktemp(f"sharp{name}"))
    cfg, weights, page = helpers.make_model_dir(d, name, sharpen=SHARPEN)
    reqs = _requests(cfg, [3, 257, 410, 129, 600, 64], seed=9)
    ref = {rid: helpers.plain_logits(cfg, weights, toks) for rid, toks in reqs.items()}
    tol = SHARPEN * _tol(name, dtype)
    for mode, steps, graphs in (
            ("whole", helpers.trace_whole(reqs), False),
            ("mixed", helpers.trace_mixed(reqs, max_live=4, seed=21), False),
            ("long portions", helpers.trace_mixed(reqs, max_live=3, seed=22, prefill_frac=0.8,
                                                  portion_choices=(70, 130, 65, 2, 200)), True),
            ("decode32", helpers.trace_prefill_then_decode(reqs, tail=32), True)):
        pool = helpers.max_live_tokens(steps, round_to=max(64, page))
        eng = _engine(d, dtype, page, pool, use_graphs=graphs)
        rows = helpers.replay(eng, steps)
        worst = helpers.compare(rows, ref, tol, f"sharp {name} {dtype} {mode}")
        print(f"[worst] sharp {name}, {dtype}, {mode}: {worst:.3e}")
        eng.cache.check_consistency()
