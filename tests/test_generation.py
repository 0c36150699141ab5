"""Generation through the entry points against the plain implementation: Python, command line, trace replay."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("genA"))
    cfg, w, page = helpers.make_model_dir(d, "A")
    return d, cfg, w, page


@pytest.fixture(scope="module")
def model_b(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("genB"))
    cfg, w, page = helpers.make_model_dir(d, "B", store="float32")
    return d, cfg, w, page


def _prompts(cfg, lengths, seed):
    rng = np.random.RandomState(seed)
    return [rng.randint(0, cfg["vocab_size"], size=n).tolist() for n in lengths]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_tiny_a(model_a, dtype):
    """Three requests, prompts of 5, 11 and 17 tokens, 8 greedy tokens each, pages of 4."""
    from ccinfer_b200 import LLM, SamplingParams
    d, cfg, w, page = model_a
    prompts = _prompts(cfg, [5, 11, 17], 0)
    llm = LLM(d, dtype=dtype, page_size=page, kv_tokens=128, max_requests=4, max_tokens_per_step=64)
    got = llm.generate(prompts, SamplingParams(max_tokens=8))
    want = [plain.generate(cfg, w, p, 8) for p in prompts]
    assert got == want
    assert all(p.used_pages == 0 for p in llm.engine.cache.pools)


def test_temperature_generation_tiny_b_in_portions(model_b):
    """Four requests, prompts of 1, 9, 33 and 64 tokens in portions of 7 beside running decodes,
    12 tokens each at temperature 0.8 with seed 7, pages of 8."""
    from ccinfer_b200 import LLM, SamplingParams
    d, cfg, w, page = model_b
    prompts = _prompts(cfg, [1, 9, 33, 64], 1)
    llm = LLM(d, dtype="float32", page_size=page, kv_tokens=512, prefill_chunk_size=7, max_requests=4,
              max_tokens_per_step=64)
    got = llm.generate(prompts, SamplingParams(max_tokens=12, temperature=0.8, seed=7))
    want = [plain.generate(cfg, w, p, 12, temperature=0.8, seed=7) for p in prompts]
    assert got == want
    assert got != [plain.generate(cfg, w, p, 12) for p in prompts]  # it is not greedy in disguise


def test_top_k_and_top_p_generation(model_b):
    """Requests with different filters in one batch: top_k = 1 is greedy whatever the temperature; a
    request with top_k and top_p draws the tokens of the plain rule, step by step."""
    from ccinfer_b200 import LLM, SamplingParams
    d, cfg, w, page = model_b
    prompts = _prompts(cfg, [9, 20, 5], 2)
    llm = LLM(d, dtype="float32", page_size=page, kv_tokens=512, max_requests=4, max_tokens_per_step=64)
    params = [SamplingParams(max_tokens=10, temperature=1.3, seed=3, top_k=1),
              SamplingParams(max_tokens=10, temperature=0.9, seed=11, top_k=20, top_p=0.7),
              SamplingParams(max_tokens=10, temperature=1.0, seed=5)]
    got = llm.generate(prompts, params)
    assert got[0] == plain.generate(cfg, w, prompts[0], 10)
    assert got[2] == plain.generate(cfg, w, prompts[2], 10, temperature=1.0, seed=5)
    toks, safe = list(prompts[1]), True
    for i in range(10):
        logits = plain.forward(cfg, w, toks, plain.F64)[-1]
        want, margin = plain.sample_filtered(logits, 0.9, 11, i, 20, 0.7)
        if margin < 1e-5:
            safe = False   # a cut on a rounding edge: what follows may differ legitimately
            break
        assert got[1][i] == want, i
        toks.append(want)
    assert safe or i >= 3


def test_pages_run_out_during_generation(model_b):
    """So few pages that a request is preempted and computed again: the tokens are those of a calm run."""
    from ccinfer_b200 import LLM, SamplingParams
    d, cfg, w, page = model_b
    prompts = _prompts(cfg, [20, 26, 17], 2)
    sp = [SamplingParams(max_tokens=24, temperature=0.6, seed=5), SamplingParams(max_tokens=20),
          SamplingParams(max_tokens=28, temperature=1.1, seed=9)]
    llm = LLM(d, dtype="float32", page_size=page, kv_tokens=13 * page, prefill_chunk_size=16, max_requests=4,
              max_tokens_per_step=64)
    got = llm.generate(prompts, sp)
    assert llm.scheduler.preemptions > 0
    want = [plain.generate(cfg, w, p, s.max_tokens, s.temperature, s.seed) for p, s in zip(prompts, sp)]
    assert got == want
    llm.engine.cache.check_consistency()


def test_many_requests_two_cache_groups_and_too_few_pages(tmp_path_factory):
    """Twenty requests of random lengths and sampling parameters through the scheduler on a model with two
    cache groups (layer 1 of Tiny D reads a window: its pages are given back while a request runs), with so few
    pages that requests give way and are computed again, prompts in portions beside decoding requests, one step
    in flight: every request's tokens are those of the plain implementation, nothing is left in the cache."""
    from ccinfer_b200 import LLM, SamplingParams
    d = str(tmp_path_factory.mktemp("genD"))
    cfg, w, page = helpers.make_model_dir(d, "D")
    rng = np.random.RandomState(31)
    prompts = _prompts(cfg, [int(n) for n in rng.randint(1, 90, size=20)], 8)
    sp = [SamplingParams(max_tokens=int(rng.randint(1, 40)), temperature=float(rng.choice([0.0, 0.7, 1.2])), seed=i)
          for i in range(20)]
    llm = LLM(d, dtype="float32", page_size=page, kv_tokens=20 * page, prefill_chunk_size=24, max_requests=6,
              max_running=6, max_tokens_per_step=96, max_context=160)
    assert llm.scheduler.run_ahead
    got = llm.generate(prompts, sp)
    assert llm.scheduler.preemptions > 0
    want = [plain.generate(cfg, w, p, s.max_tokens, s.temperature, s.seed) for p, s in zip(prompts, sp)]
    assert got == want
    llm.engine.cache.check_consistency()
    assert all(pool.used_pages == 0 for pool in llm.engine.cache.pools) and llm.engine.cache.slots.free_slots == 6


def test_running_ahead_reads_tokens_a_step_late_and_changes_none(model_b):
    """The entry point launches a step before it reads the tokens of the step before (they stay on the
    device for the next embedding).  Same tokens as a scheduler that waits for every step, also when a
    request stops at an end-of-sequence token while its next step is already in flight."""
    from ccinfer_b200 import LLM, SamplingParams
    from ccinfer_b200.engine.engine import PENDING, StepEntry
    from ccinfer_b200.engine.scheduler import Scheduler
    from ccinfer_b200.errors import InvalidArgument
    d, cfg, w, page = model_b
    prompts = _prompts(cfg, [9, 30, 5], 4)
    sp = [SamplingParams(max_tokens=14, temperature=0.5, seed=3), SamplingParams(max_tokens=16),
          SamplingParams(max_tokens=11)]
    want = [plain.generate(cfg, w, p, s.max_tokens, s.temperature, s.seed) for p, s in zip(prompts, sp)]
    eos = want[1][7]
    stop = [t[:t.index(eos) + 1] if eos in t else t for t in want]
    for eos_id, expect in ((None, want), (eos, stop)):
        llm = LLM(d, dtype="float32", page_size=page, kv_tokens=512, prefill_chunk_size=8, max_requests=4,
                  max_tokens_per_step=64, eos_token_id=eos_id)
        assert llm.scheduler.run_ahead
        assert llm.generate(prompts, sp) == expect
        waits = Scheduler(llm.engine, prefill_chunk_size=8, max_tokens_per_step=64, eos_token_id=eos_id)
        for i, (p, s) in enumerate(zip(prompts, sp)):
            waits.submit(i, p, s)
        out = waits.run()
        assert [out[i] for i in range(3)] == expect
        assert all(p.used_pages == 0 for p in llm.engine.cache.pools)
    # PENDING stands alone and needs a token drawn for the request
    eng = llm.engine
    eng.open_request("z")
    with pytest.raises(InvalidArgument):
        eng.step([StepEntry("z", [PENDING], [0])])
    lg = eng.step([StepEntry("z", prompts[0], [len(prompts[0]) - 1])])
    first = eng.sample_async(lg, [SamplingParams()], [0])
    with pytest.raises(InvalidArgument):
        eng.step([StepEntry("z", [PENDING, 3], [0])])
    lg = eng.step([StepEntry("z", [PENDING], [0])])          # launched before the first token is read
    second = eng.sample(lg, [SamplingParams()], [1])
    assert first.tokens() + second == plain.generate(cfg, w, prompts[0], 2)
    # a pending token serves one step, and only the logits of the most recent step leave one
    lg = eng.step([StepEntry("z", [second[0]], [0])])       # the token itself: the pending one is used up
    with pytest.raises(InvalidArgument):
        eng.step([StepEntry("z", [PENDING], [0])])
    third = eng.sample_async(lg.clone(), [SamplingParams()], [2]).tokens()   # a copy is not the step's tensor
    with pytest.raises(InvalidArgument):
        eng.step([StepEntry("z", [PENDING], [0])])
    assert eng.sample_async(lg, [SamplingParams()], [2]).tokens() == third
    eng.step([StepEntry("z", [PENDING], [0])])
    assert first.tokens() + second + third == plain.generate(cfg, w, prompts[0], 3)
    eng.close_request("z")
    eng.check()


def test_cache_pool_sized_from_free_memory(model_a):
    """kv_memory_fraction: the pools take that share of what is free once the weights are loaded."""
    from ccinfer_b200.engine.engine import Engine, EngineOptions
    from ccinfer_b200.errors import InvalidArgument
    d, cfg, w, page = model_a
    free = torch.cuda.mem_get_info()[0]
    eng = Engine.from_model_dir(d, EngineOptions(dtype="float32", page_size=page, kv_memory_fraction=0.01,
                                                 max_requests=2, max_tokens_per_step=32, max_context=64))
    per_page = cfg["num_hidden_layers"] * 2 * cfg["num_key_value_heads"] * page * cfg["head_dim"] * 4
    pages = eng.cache.groups[0].num_pages
    assert 0.8 * 0.01 * free / per_page <= pages <= 0.01 * free / per_page
    with pytest.raises(InvalidArgument):
        Engine.from_model_dir(d, EngineOptions(dtype="float32", kv_tokens=64, kv_memory_fraction=0.5))


def test_warm_up_captures_graphs_and_changes_nothing(model_a):
    """The decode graphs captured ahead of the first request, with throw-away requests: everything they
    held is given back, and generation afterwards replays them and gives the plain tokens."""
    from ccinfer_b200 import LLM, SamplingParams
    d, cfg, w, page = model_a
    llm = LLM(d, dtype="bfloat16", page_size=page, kv_tokens=128, max_requests=4, max_tokens_per_step=64,
              max_running=4, warm_up=True)
    eng = llm.engine
    assert sorted(eng._graphs) == [1, 2, 4]
    assert all(p.used_pages == 0 for p in eng.cache.pools) and eng.cache.slots.free_slots == 4
    eng.cache.check_consistency()
    assert eng.warm_up() == []                       # nothing left to capture
    replays = eng.graph_replays
    prompts = _prompts(cfg, [5, 11, 17], 0)
    got = llm.generate(prompts, SamplingParams(max_tokens=8))
    assert got == [plain.generate(cfg, w, p, 8) for p in prompts]
    assert eng.graph_replays > replays and sorted(eng._graphs) == [1, 2, 4]


def test_long_decoding_and_first_tokens(model_b):
    """A one-token prompt decoded far, every position compared; and the first tokens of a sequence."""
    from ccinfer_b200.engine.engine import Engine, EngineOptions
    d, cfg, w, page = model_b
    toks = _prompts(cfg, [230], 3)[0]
    ref = helpers.plain_logits(cfg, w, toks)
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 3e-2)):
        eng = Engine.from_model_dir(d, EngineOptions(dtype=dtype, page_size=page, kv_tokens=256, max_requests=2,
                                                     max_tokens_per_step=32))
        steps = [{"entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for t in toks]
        rows = helpers.replay(eng, steps)
        helpers.compare(rows, {"x": ref}, tol, f"long decoding {dtype}")
        first = {k: v for k, v in rows.items() if k[1] < 4}
        helpers.compare(first, {"x": ref}, tol, f"first tokens {dtype}")


def test_python_entry_point_a_step_at_a_time(model_a):
    """add_request / step / cancel / forward of the Python entry point: the tokens of generate(), a request
    cancelled on the way, and the raw step against the plain logits."""
    from ccinfer_b200 import LLM, SamplingParams
    d, cfg, w, page = model_a
    llm = LLM(d, dtype="float32", page_size=page, kv_tokens=256, prefill_chunk_size=8, max_requests=4)
    prompts = _prompts(cfg, [6, 19, 3], 12)
    ids = [llm.add_request(p, SamplingParams(max_tokens=7)) for p in prompts]
    out, n = {}, 0
    while llm.has_work():
        for ev in llm.step():
            if ev.token is not None:
                out.setdefault(ev.req_id, []).append(ev.token)
        n += 1
        if n == 3:
            assert llm.cancel(ids[1])
    assert out[ids[0]] == plain.generate(cfg, w, prompts[0], 7) and out[ids[2]] == plain.generate(cfg, w, prompts[2], 7)
    assert len(out.get(ids[1], [])) < 7 and not llm.cancel(ids[1])
    logits = llm.forward([("raw", prompts[1], [0, len(prompts[1]) - 1])])
    ref = helpers.plain_logits(cfg, w, prompts[1])
    assert logits.shape == (2, cfg["vocab_size"]) and np.abs(logits - ref[[0, -1]]).max() <= 2e-5 * np.abs(ref).max()
    llm.engine.close_request("raw")
    assert all(p.used_pages == 0 for p in llm.engine.cache.pools)


def test_command_line(model_a):
    d, cfg, w, page = model_a
    prompt = _prompts(cfg, [9], 4)[0]
    cmd = [sys.executable, os.path.join(ROOT, "bin", "ccinfer"), "--model-path", d, "--dtype", "float32",
           "--prefill-chunk-size", "4", "--page-size", str(page), "--kv-tokens", "64", "--max-tokens", "5",
           "--prompt-ids", ",".join(map(str, prompt)), "--stats"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["token_ids"] == plain.generate(cfg, w, prompt, 5)
    bad = subprocess.run(cmd[:2] + ["--model-path", "/nonexistent", "--prompt-ids", "1"], capture_output=True,
                         text=True, timeout=300)
    assert bad.returncode == 2 and "ModelLoadFailed" in bad.stderr


def test_command_line_random_config(tmp_path):
    """--random-config draws on the device the model that --write-random-model writes for the same seed: the
    same tokens either way, and those of the plain implementation on the stream's weights; --dump-config."""
    import tiny_configs
    cfg = dict(tiny_configs.TINY_B)
    cj = str(tmp_path / "config.json")
    with open(cj, "w") as f:
        json.dump(cfg, f)
    exe = [sys.executable, os.path.join(ROOT, "bin", "ccinfer")]
    common = ["--dtype", "float32", "--page-size", "8", "--kv-tokens", "128", "--max-tokens", "6", "--random-prompts", "7,12",
              "--prompt-seed", "3", "--weights-seed", "11", "--weights-std", "0.05", "--temperature", "0.7"]
    a = subprocess.run(exe + ["--random-config", cj] + common, capture_output=True, text=True, timeout=300)
    assert a.returncode == 0, a.stderr
    d = str(tmp_path / "model")
    w = subprocess.run(exe + ["--model-path", d, "--write-random-model", cj, "--weights-seed", "11", "--weights-std", "0.05"],
                       capture_output=True, text=True, timeout=300)
    assert w.returncode == 0, w.stderr
    b = subprocess.run(exe + ["--model-path", d] + common, capture_output=True, text=True, timeout=300)
    assert b.returncode == 0, b.stderr
    assert a.stdout == b.stdout and len(a.stdout.strip().splitlines()) == 2
    weights = {k: v.to(torch.bfloat16).float() if cfg["torch_dtype"] == "bfloat16" else v
               for k, v in plain.stream_weights(cfg, 11, 0.05).items()}
    prompts = [np.random.RandomState(3).randint(0, cfg["vocab_size"], size=n).tolist() for n in (7,)]
    first = json.loads(a.stdout.strip().splitlines()[0])
    assert first["token_ids"] == plain.generate(cfg, weights, prompts[0], 6, 0.7, 42)
    dump = subprocess.run(exe + ["--random-config", cj, "--dump-config"], capture_output=True, text=True, timeout=300)
    assert dump.returncode == 0 and json.loads(dump.stdout)["num_hidden_layers"] == cfg["num_hidden_layers"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_b, dtype, tmp_path):
    """bin/trace_run as a user calls it: a mixed trace over a small pool, files compared with the plain logits."""
    d, cfg, w, page = model_b
    reqs = {f"q{i}": p for i, p in enumerate(_prompts(cfg, [40, 3, 75, 64, 18], 5))}
    steps = helpers.trace_mixed(reqs, max_live=4, seed=2)
    pool = helpers.max_live_tokens(steps)
    out_dir = tmp_path / "out"
    lines = "".join(json.dumps({"step": i, **st}) + "\n" for i, st in enumerate(steps))
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out",
                        str(out_dir), "--max-tokens", str(pool)], input=lines, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.split() == [x for i in range(len(steps)) for x in ("done", str(i))]
    ref = {rid: helpers.plain_logits(cfg, w, toks) for rid, toks in reqs.items()}
    V = cfg["vocab_size"]
    rows, seen = {}, {rid: 0 for rid in reqs}
    for i, st in enumerate(steps):
        n_want = sum(len(e["want"]) for e in st["entries"])
        arr = np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(n_want, V)
        r_ = 0
        for e in st["entries"]:
            for wnt in e["want"]:
                rows[(e["id"], seen[e["id"]] + wnt)] = arr[r_]
                r_ += 1
            seen[e["id"]] += len(e["tokens"])
    assert len(rows) == sum(len(t) for t in reqs.values())
    helpers.compare(rows, ref, 2e-5 if dtype == "float32" else 3e-2, f"trace_run {dtype}")
