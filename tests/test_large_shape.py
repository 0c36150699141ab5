"""Real layer sizes against the plain implementation, under every way of cutting the work.

The Qwen3-8B layer shape (4 of its 36 layers, every other size as the model has it, full vocabulary) and a
mid-size shape with head size 64.  The weights are the random model that the seed names (the counter-based
stream, restated in tests/plain_qwen3.py and drawn here on the GPU), rounded once to bfloat16 so that the
32-bit and the bfloat16 engine and the plain implementation hold the same values.  The plain
implementation runs whole sequences in float64 on the GPU (it is plain torch).  This is where the
tensor-core kernels (tcgen05 products and attention, TMA page loads, head size 128, groups of 4 q heads,
pages of 16) run inside the engine with realistic strides and more keys than one tile.  The reference's
counterpart is its logits test against an outside oracle (tests/integration/test_logits_match.cpp:509-575).
"""
import numpy as np
import pytest
import torch

import helpers
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

SHAPE_8B_4_OF_36_LAYERS = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 4, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 40960, "torch_dtype": "bfloat16",
}
MID_SHAPE = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 4, "head_dim": 64, "intermediate_size": 4096,
    "vocab_size": 3000, "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 4096, "torch_dtype": "bfloat16",
}
# relative to the largest logit of the request; bfloat16: about twice the worst seen on a B200 (printed by
# every run as "[worst] ...")
TOL32 = 2e-5
TOL16 = {"8b": 3e-2, "mid": 2.6e-2}   # seen: 1.5e-2, 1.3e-2 (and 8.4e-6, 4.5e-6 in 32-bit)


class _Model:
    """Weights of a shape (on the GPU, bfloat16 values held in float), requests and their plain logits."""

    def __init__(self, shape, seed, std, lengths=None, tail=10 ** 9, weights=None, reqs=None):
        self.shape, self.tail = shape, tail
        if weights is None:
            w = plain.stream_weights(shape, seed, std, device="cuda")
            weights = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}
        self.weights = weights
        if reqs is None:
            rng = np.random.RandomState(seed)
            reqs = {f"r{i}": rng.randint(0, shape["vocab_size"], size=n).tolist() for i, n in enumerate(lengths)}
        self.reqs, self.ref, self.scale = reqs, {}, {}
        for rid, toks in self.reqs.items():   # float64, whole sequence; a row of logits is kept where it is compared
            logits = plain.forward(shape, self.weights, toks)
            keep = range(max(0, len(toks) - tail), len(toks))
            self.ref[rid] = {p: logits[p].cpu().numpy() for p in keep}
            self.scale[rid] = float(logits.abs().max())
            del logits
        torch.cuda.empty_cache()

    def with_requests(self, reqs):
        """The same weights with other requests."""
        return _Model(self.shape, 0, 0.0, tail=self.tail, weights=self.weights, reqs=reqs)

    def engine(self, dtype, **opts):
        from ccinfer_b200.config import Qwen3Config
        from ccinfer_b200.config.registry import architecture_of
        from ccinfer_b200.engine.engine import Engine, EngineOptions
        cfg = Qwen3Config.from_json(self.shape)
        plan = architecture_of(cfg.to_json()).build_plan(cfg)
        tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
        roles = {s.name: s.role for s in plan.tensor_specs()}

        def fetch(name):
            return self.weights[name].to(torch.float32 if roles[name] == "vector" else tdt).contiguous()

        return Engine(plan, fetch, EngineOptions(dtype=dtype, page_size=16, **opts))

    def tail_only(self, steps):
        """Asks for logits only where they are compared (a row of the 8B vocabulary is 600 KB)."""
        seen = {}
        for st in steps:
            for e in st["entries"]:
                base = seen.get(e["id"], 0)
                n = len(self.reqs[e["id"]])
                e["want"] = [w for w in e["want"] if base + w >= n - self.tail]
                seen[e["id"]] = base + len(e["tokens"])
        return steps

    def worst(self, rows):
        assert set(rows) == {(rid, p) for rid in self.ref for p in self.ref[rid]}
        return max(float(np.abs(row - self.ref[rid][p]).max()) / self.scale[rid] if np.isfinite(row).all()
                   else float("inf") for (rid, p), row in rows.items())


def _run(model, dtype, steps, **opts):
    eng = model.engine(dtype, **opts)
    rows = helpers.replay(eng, model.tail_only(steps))
    eng.cache.check_consistency()
    assert all(p.used_pages == 0 for p in eng.cache.pools)
    del eng
    torch.cuda.empty_cache()
    return rows


def _cuttings(reqs, seed):
    return [("whole", helpers.trace_whole(reqs)),
            ("decode32", helpers.trace_prefill_then_decode(reqs, tail=32)),
            ("portions", helpers.trace_portions(reqs)),
            # portions of more than 64 tokens after a cached prefix, beside nothing: the tcgen05 attention with
            # keys before its first query
            ("long portions", helpers.trace_portions(reqs, sizes=(70, 2, 130, 1, 65, 200))),
            ("mixed", helpers.trace_mixed(reqs, max_live=4, seed=seed)),
            # the scheduler's own shape of a step: portions of up to 512 tokens beside single decoded tokens
            ("mixed, long portions", helpers.trace_mixed(reqs, max_live=4, seed=seed + 1,
                                                         portion_choices=(128, 200, 65, 512, 2)))]


@pytest.fixture(scope="module")
def model_8b():
    return _Model(SHAPE_8B_4_OF_36_LAYERS, seed=42, std=0.02, lengths=[300, 70, 513, 140], tail=40)


@pytest.fixture(scope="module")
def model_mid():
    return _Model(MID_SHAPE, seed=5, std=0.03, lengths=[150, 41, 260, 77, 600], tail=10 ** 9)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_8b_layer_shape_matches_plain_under_every_cutting(model_8b, dtype):
    m = model_8b
    opts = dict(kv_tokens=2048, max_requests=8, max_tokens_per_step=1024, max_context=1024)
    for name, steps in _cuttings(m.reqs, seed=4):
        worst = m.worst(_run(m, dtype, steps, **opts))
        print(f"[worst] 8B layer shape, {dtype}, {name}: {worst:.3e}")
        assert worst <= (TOL32 if dtype == "float32" else TOL16["8b"]), name


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mid_shape_with_head_size_64_matches_plain_under_every_cutting(model_mid, dtype):
    """Hidden 2048, head size 64, groups of 8 q heads, 64 tiles of gate|up: the sizes at which the few-rows
    products of a decode or mixed step go to the TMA-ring kernel (q|k|v, o, down and, with fewer tiles than
    SMs, gate|up with the activation as its epilogue) while portions of more than 16 tokens go to the
    library."""
    from ccinfer_b200 import kernels
    m = model_mid
    opts = dict(kv_tokens=2048, max_requests=8, max_tokens_per_step=1024, max_context=1024)
    before = kernels.counters.own
    for name, steps in _cuttings(m.reqs, seed=6):
        worst = m.worst(_run(m, dtype, steps, **opts))
        print(f"[worst] mid shape, {dtype}, {name}: {worst:.3e}")
        assert worst <= (TOL32 if dtype == "float32" else TOL16["mid"]), name
    assert kernels.counters.own > before


@pytest.mark.parametrize("n_live", [17, 33, 49, 64])
def test_mid_shape_many_decoding_requests_match_plain(model_mid, n_live):
    """Decode steps of 17 to 64 rows at sizes where the products are real work: library products from 17
    rows on, the unfused attention from 49, replayed from the graphs of 32 and 64 rows."""
    rng = np.random.RandomState(n_live)
    reqs = {f"m{i}": rng.randint(0, MID_SHAPE["vocab_size"], size=int(rng.randint(8, 90))).tolist()
            for i in range(n_live)}
    m = model_mid.with_requests(reqs)
    steps = helpers.trace_many_decoders(reqs, decode_steps=4, per_prefill_step=7)
    for dtype in ("float32", "bfloat16"):
        eng = m.engine(dtype, kv_tokens=64 * 96, max_requests=64, max_tokens_per_step=1024, max_context=128)
        rows = helpers.replay(eng, m.tail_only(steps))
        worst = m.worst(rows)
        print(f"[worst] mid shape, {dtype}, {n_live} decoding requests: {worst:.3e}")
        assert worst <= (TOL32 if dtype == "float32" else TOL16["mid"])
        assert eng.graph_replays > 0
        del eng
        torch.cuda.empty_cache()


def test_8b_layer_shape_steps_of_more_than_2048_rows_match_plain(model_8b):
    """Steps of 2,048 rows and more (in bfloat16 gate|up with its activation runs on the two-SM tcgen05 kernel
    from 1,024 rows on, with tiles of 256 rows): a prompt of 2,300 tokens whole (rows that fill no tile), and
    one of 2,560 tokens as 512 tokens and then 2,048 more after them, beside a short request's prompt and
    decoded tokens."""
    rng = np.random.RandomState(11)
    V = SHAPE_8B_4_OF_36_LAYERS["vocab_size"]
    reqs = {"long": rng.randint(0, V, size=2300).tolist(), "cut": rng.randint(0, V, size=2560).tolist(),
            "short": rng.randint(0, V, size=40).tolist()}
    m = model_8b.with_requests(reqs)
    steps = [
        {"entries": [{"id": "long", "tokens": reqs["long"], "want": list(range(2300))}], "end": ["long"]},
        {"entries": [{"id": "cut", "tokens": reqs["cut"][:512], "want": []},
                     {"id": "short", "tokens": reqs["short"][:38], "want": list(range(38))}], "end": []},
        {"entries": [{"id": "short", "tokens": reqs["short"][38:39], "want": [0]},
                     {"id": "cut", "tokens": reqs["cut"][512:], "want": list(range(2048))}], "end": ["cut"]},
        {"entries": [{"id": "short", "tokens": reqs["short"][39:], "want": [0]}], "end": ["short"]},
    ]
    for dtype in ("float32", "bfloat16"):
        rows = _run(m, dtype, [dict(s) for s in steps], kv_tokens=4096 + 512, max_requests=4, max_tokens_per_step=2304,
                    max_context=2624)
        worst = m.worst(rows)
        print(f"[worst] 8B layer shape, {dtype}, steps of 2,048 rows and more: {worst:.3e}")
        assert worst <= (TOL32 if dtype == "float32" else TOL16["8b"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mid_shape_the_same_trace_twice_gives_the_same_bits(model_mid, dtype):
    """Nothing in a step depends on which block or warp ran first (partial sums are added in fixed orders, counters
    only say who is last): a mixed trace with decode steps from graphs gives bit-identical logits twice, on two
    engines."""
    m = model_mid
    opts = dict(kv_tokens=2048, max_requests=8, max_tokens_per_step=1024, max_context=1024, use_graphs=True)
    steps = helpers.trace_mixed(m.reqs, max_live=4, seed=12, portion_choices=(128, 200, 65, 2, 16))
    first = _run(m, dtype, [dict(s) for s in steps], **opts)
    second = _run(m, dtype, [dict(s) for s in steps], **opts)
    assert set(first) == set(second)
    assert all(np.array_equal(first[k], second[k]) for k in first)
