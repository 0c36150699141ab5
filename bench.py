#!/usr/bin/env python3
"""Decode and prefill throughput at the Qwen3-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  The default run: 36 layers,
hidden 4096, 32 q heads, 8 kv heads, head size 128, intermediate 12288,
vocabulary 151936, bfloat16, a batch of 8 requests decoding after 2,048-token
prompts.  It prints ONE JSON line:

  value      decoded tokens a second: the median of --runs (5) runs of K timed steps each, from CUDA events
             around every step
  e2e        the same through the Python entry point's scheduler, by wall clock, over at least 256 steps
             (named in config): host prompts in, every step one copy of the step's arrays from pinned memory
             and one read of the sampled token ids into host lists.  The scheduler runs one step ahead: a
             step is launched before the tokens of the step before it are read (the embedding takes them
             from the device)
  prefill    one 2,048-token prompt in one step: tokens a second and the fraction of the bf16 peak
  roofline   the decode step's bytes (every weight once + the cache of the live requests) / its time
  points     decode at batch 1 and 64, decode at batch 8 after 8,192- and 32,768-token prompts, prefill of
             8,192- and 16,384-token prompts (in steps of 2,048 tokens, as the scheduler cuts them)
  clocks     SM clock and throttle reasons sampled during the timed regions

Every timed decode step reads 15 GB of weights, far more than the 126 MB L2, so no flush is needed
between iterations.  With --gpus N > 1 it prints one line that says so and exits with 2.

    python bench.py --profile-steps N [--layers L] [--batch B] [--context C] [--profile-prefill T] [--shape 8b|14b|32b]

is for profilers: N decode steps of B requests at C cached tokens WITHOUT CUDA graphs (so that a profiler sees
every kernel) and, with --profile-prefill T, one prompt of T tokens in one step; few layers keep it small.

    python bench.py --workload mix14b | long32b [--layers L]

runs one of the two other workloads of the reference's benchmark record through the scheduler (a mixed
continuous batch at the Qwen3-14B shape; four 16,384-token prompts at the Qwen3-32B shape) and prints a
line of its own: output tokens a second, the distribution of the step calls, the pages' high water.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 36, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 40960, "torch_dtype": "bfloat16",
}
# The two other workloads that the reference's benchmark record names, at their own layer shapes
SHAPES = {
    "mix14b": dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408),
    "long32b": dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            j = json.load(f)
        return {"hbm_gbs": float(j["hbm_gbs"]), "bf16_tflops": float(j["bf16_tflops"]),
                "bf16_tflops_sustained": float(j.get("bf16_tflops_sustained", j["bf16_tflops"])),
                "source": "measured"}
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi sampling of the SM clock and the throttle reasons while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self._proc = None
        self._file = None

    def start(self):
        try:
            self._file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self._file, stderr=subprocess.DEVNULL)
        except OSError:
            self._proc = None

    def stop(self):
        if self._proc is None:
            return
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self._proc.kill()
        self._file.flush()
        self._file.seek(0)
        for line in self._file:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.rows.append(parts)
        self._file.close()
        os.unlink(self._file.name)
        self._proc = None

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": int(statistics.median(int(r[0]) for r in self.rows)),
                "sm_max_mhz": int(self.rows[0][1]), "reasons": reasons, "samples": len(self.rows)}


def model_numbers(cfg, layers):
    D, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nq + 2 * nkv) * hd * D + D * nq * hd + 3 * F * D
    linear_params = layers * per_layer
    weight_bytes = 2 * (linear_params + V * D) + 4 * (layers * (2 * D + 2 * hd) + D)
    kv_bytes_per_token = layers * 2 * nkv * hd * 2

    def prefill_flops(T):
        return 2.0 * T * linear_params + layers * 2.0 * T * T * nq * hd + 2.0 * V * D

    return weight_bytes, kv_bytes_per_token, prefill_flops


def run_workload(args) -> int:
    """--workload mix14b: 32 requests, prompts of 64..4,096 tokens in 512-token portions beside running
    decodes, 128 new tokens each, half greedy and half at temperature 0.7 (Qwen3-14B shape).
    --workload long32b: 4 requests of 16,384 tokens, then 128 greedy tokens each (Qwen3-32B shape).
    Through the Python entry point's scheduler; prints one JSON line of its own."""
    import numpy as np
    import torch
    from ccinfer_b200.config import Qwen3Config
    from ccinfer_b200.engine.engine import Engine, EngineOptions
    from ccinfer_b200.engine.scheduler import Scheduler
    from ccinfer_b200.sampling import SamplingParams

    cfg_json = dict(SHAPES[args.workload])
    layers_full = cfg_json["num_hidden_layers"]
    layers = args.layers or layers_full
    cfg_json["num_hidden_layers"] = layers
    cfg = Qwen3Config.from_json(cfg_json)
    rng = np.random.RandomState(1)
    V, new = cfg.vocab_size, 128
    if args.workload == "mix14b":
        lens = rng.randint(64, 4097, size=32).tolist()
        params = [SamplingParams(max_tokens=new, temperature=0.0 if i % 2 == 0 else 0.7, seed=i) for i in range(32)]
        seed = 43
    else:
        lens = [16384] * 4
        params = [SamplingParams(max_tokens=new) for _ in lens]
        seed = 44
    n = len(lens)
    page = 16
    per_req = [-(-(L + new + 1) // page) * page for L in lens]
    opt = EngineOptions(dtype="bfloat16", page_size=page, kv_tokens=sum(per_req), max_requests=n,
                        max_tokens_per_step=4096, max_context=max(per_req))
    t0 = time.time()
    engine = Engine.from_random(cfg, seed=seed, std=0.02, options=opt)
    torch.cuda.synchronize()
    print(f"[bench] {args.workload}: model on the device in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    chunk = args.chunk or 512
    sched = Scheduler(engine, prefill_chunk_size=chunk, max_tokens_per_step=4096, max_running=n, run_ahead=True)
    for i, L in enumerate(lens):
        sched.submit(i, rng.randint(0, V, size=L).tolist(), params[i])
    sampler = ClockSampler()
    sampler.start()
    torch.cuda.synchronize()
    produced, calls, decode_calls = 0, [], []
    t_start = time.perf_counter()
    while sched.has_work():
        c = sched.counts()
        decode_only = c["prefilling"] == 0 and c["waiting"] == 0
        t = time.perf_counter()
        events = sched.step()
        ms = (time.perf_counter() - t) * 1e3
        n_out = sum(1 for ev in events if ev.token is not None)
        calls.append(ms)
        if decode_only:
            decode_calls.append((ms, n_out))
        produced += n_out
    torch.cuda.synchronize()
    wall = time.perf_counter() - t_start
    sampler.stop()
    engine.check()
    assert produced == n * new and all(p.used_pages == 0 for p in engine.cache.pools)
    calls.sort()
    # steps that hold decoding requests only, without the first three (a CUDA graph is captured there)
    decode_tail = None
    steady = decode_calls[3:]
    if steady and sum(ms for ms, _ in steady) > 0:
        decode_tail = sum(n for _, n in steady) / (sum(ms for ms, _ in steady) * 1e-3)
    prompt_tokens = int(sum(lens))
    line = {
        "metric": f"output tokens/s ({args.workload}: {n} requests, {prompt_tokens:,} prompt tokens in {chunk}-token "
                  f"portions beside decodes, {new} new tokens each)",
        "value": round(produced / wall, 1), "unit": "tokens/s", "n_gpus": 1, "workload": args.workload,
        "higher_is_better": True, "dtype": "bf16", "wall_s": round(wall, 3), "output_tokens": produced,
        "prompt_tokens": prompt_tokens, "all_tokens_per_s": round((produced + prompt_tokens) / wall, 1),
        "decode_only_tokens_per_s": None if decode_tail is None else round(decode_tail, 1),
        "steps": sched.steps, "step_call_ms": {"p50": round(calls[len(calls) // 2], 3),
                                               "p90": round(calls[int(len(calls) * 0.9)], 3),
                                               "max": round(calls[-1], 3)},
        "pages_high_water": max(p.high_water for p in engine.cache.pools), "pages": engine.cache.groups[0].num_pages,
        "preemptions": sched.preemptions, "graph_replays": engine.graph_replays,
        "data": f"synthetic: uniform random token ids, random weights (seed {seed}, N(0, 0.02))",
        "config": {"model": {"mix14b": "Qwen3-14B shape", "long32b": "Qwen3-32B shape"}[args.workload],
                   "layers": layers, "layers_full": layers_full, "hidden": cfg.hidden_size,
                   "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "requests": n,
                   "page_size": page, "prefill_chunk": chunk, "max_tokens_per_step": 4096},
        "clocks": sampler.summary(),
    }
    print(json.dumps(line))
    return 0


def run_profile_steps(args) -> int:
    """A few eager steps of a random model at a chosen layer shape, for profilers (nothing is timed)."""
    import numpy as np
    import torch
    from ccinfer_b200.config import Qwen3Config
    from ccinfer_b200.engine.engine import Engine, EngineOptions, StepEntry

    cfg_json = dict({"8b": QWEN3_8B, "14b": SHAPES["mix14b"], "32b": SHAPES["long32b"]}[args.shape])
    cfg_json["num_hidden_layers"] = args.layers or 2
    cfg = Qwen3Config.from_json(cfg_json)
    B, ctx, steps, pre = args.batch, args.context, args.profile_steps, args.profile_prefill
    longest = max(ctx + steps, pre) + 64
    eng = Engine.from_random(cfg, 42, options=EngineOptions(
        dtype="bfloat16", kv_tokens=B * (ctx + steps + 64) + pre + 64, max_requests=B + 1,
        max_tokens_per_step=max(2048, pre, ctx), max_context=longest, use_graphs=False, use_pdl=args.pdl))
    rng = np.random.RandomState(0)
    for b in range(B):
        eng.open_request(b)
        eng.step([StepEntry(b, rng.randint(0, cfg.vocab_size, size=ctx).tolist(), [])])
    torch.cuda.synchronize()
    for s in range(steps):
        eng.step([StepEntry(b, [5 + s], [0]) for b in range(B)])
    torch.cuda.synchronize()
    if pre:
        eng.open_request("p")
        eng.step([StepEntry("p", rng.randint(0, cfg.vocab_size, size=pre).tolist(), [pre - 1])])
        torch.cuda.synchronize()
    eng.check()
    print(f"[bench] profile steps done: {steps} decode steps of {B} requests at {ctx} tokens"
          + (f", one prompt of {pre} tokens" if pre else ""), file=sys.stderr)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--points", default="1,64", help="further decode batch sizes, '' for none")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--pdl", type=int, default=1, help="0 off, 1 products start early, 2 every kernel")
    ap.add_argument("--chunk", type=int, default=None,
                    help="prompt portion of the two workloads (default 512, the entry point's own default)")
    ap.add_argument("--runs", type=int, default=5, help="runs of K timed steps; the value is their median")
    ap.add_argument("--long-points", default="8192,32768", help="contexts of the further batch-8 decode points")
    ap.add_argument("--prefill-points", default="8192,16384", help="lengths of the further prefill points")
    ap.add_argument("--profile-steps", type=int, default=0,
                    help="for profilers: this many eager decode steps (no CUDA graphs) and nothing else")
    ap.add_argument("--profile-prefill", type=int, default=0, help="with --profile-steps: one prompt of this length")
    ap.add_argument("--shape", default="8b", choices=["8b", "14b", "32b"], help="layer shape of --profile-steps")
    ap.add_argument("--workload", default="decode", choices=["decode", "mix14b", "long32b"],
                    help="decode (the default line) or one of the two other workloads of the benchmark record")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "7QiC/ccInfer is a CMake/C++23 project with no setup.py or pyproject.toml (pip: 'not "
                          "installable'); it needs boost, spdlog, fmt and real bfloat16 Qwen3 weights, none of "
                          "which are on this machine, and has no random-weights mode"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "ccinfer_b200 is a one-GPU engine: run with --gpus 1", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.profile_steps:
        return run_profile_steps(args)
    if args.workload != "decode":
        return run_workload(args)

    import numpy as np
    import torch
    from ccinfer_b200 import kernels
    from ccinfer_b200.config import Qwen3Config
    from ccinfer_b200.engine.engine import Engine, EngineOptions, StepEntry
    from ccinfer_b200.engine.scheduler import Scheduler
    from ccinfer_b200.sampling import SamplingParams

    peaks = load_peaks()
    cfg_json = dict(QWEN3_8B)
    layers_full = cfg_json["num_hidden_layers"]
    layers = args.layers or layers_full
    cfg_json["num_hidden_layers"] = layers
    cfg = Qwen3Config.from_json(cfg_json)
    weight_bytes, kv_per_token, prefill_flops = model_numbers(cfg_json, layers)
    batches = [args.batch] + [int(b) for b in args.points.split(",") if b]
    long_ctx = [int(c) for c in args.long_points.split(",") if c]
    prefill_lens = [] if args.no_prefill else [int(c) for c in args.prefill_points.split(",") if c]
    ctx, K, W, RUNS = args.context, args.steps, args.warmup, max(1, args.runs)
    E2E_STEPS = max(K, 256)
    page = 16
    chunk = 2048   # prompts longer than this are fed in steps of this many tokens, as the scheduler cuts them

    def tokens_held(c, steps):
        return -(-(c + steps + 2) // page) * page

    per_req = tokens_held(ctx, max(W + RUNS * K, W + E2E_STEPS))
    kv_tokens = max([max(batches) * per_req] + [args.batch * tokens_held(c, W + RUNS * K) for c in long_ctx]
                    + [tokens_held(t, 0) for t in prefill_lens])
    max_context = max([per_req] + [tokens_held(c, W + RUNS * K) for c in long_ctx] + [tokens_held(t, 0) for t in prefill_lens])
    opt = EngineOptions(dtype="bfloat16", page_size=page, kv_tokens=kv_tokens,
                        max_requests=max(batches), max_tokens_per_step=max(chunk, ctx), max_context=max_context,
                        use_pdl=args.pdl)
    t0 = time.time()
    engine = Engine.from_random(cfg, seed=42, std=0.02, options=opt)
    torch.cuda.synchronize()
    print(f"[bench] model on the device in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    rng = np.random.RandomState(0)
    V = cfg.vocab_size
    sampler = ClockSampler()
    sampler.start()

    # ---- prefill: one prompt, in steps of up to 2,048 tokens; timed from the first step's launch to the last one's end
    def time_prefill(Tp, reps):
        times = []
        for i in range(W + reps if Tp <= chunk else 1 + reps):
            toks = rng.randint(0, V, size=Tp).tolist()
            engine.open_request("p")
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for at in range(0, Tp, chunk):
                part = toks[at:at + chunk]
                engine.step([StepEntry("p", part, [len(part) - 1] if at + chunk >= Tp else [])])
            e1.record()
            torch.cuda.synchronize()
            engine.close_request("p")
            times.append(e0.elapsed_time(e1))
        times = times[-reps:]
        ms = statistics.median(times)
        return {"value": round(Tp / ms * 1e3, 1), "tokens": Tp, "ms": round(ms, 3),
                "frac": round(prefill_flops(Tp) / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}

    prefill = None
    prefill_points = {}
    if not args.no_prefill:
        prefill = time_prefill(2048, 5)
        print(f"[bench] prefill {prefill}", file=sys.stderr, flush=True)
        for Tp in prefill_lens:
            prefill_points[Tp] = time_prefill(Tp, 3)
            print(f"[bench] prefill {prefill_points[Tp]}", file=sys.stderr, flush=True)

    # ---- decode ----
    def fill(B, c, sched=None, steps=0):
        """Opens B requests and brings each to ``c`` cached tokens (prompts in steps of up to 2,048 tokens)."""
        prompts = [rng.randint(0, V, size=c).tolist() for _ in range(B)]
        if sched is not None:
            for b, p in enumerate(prompts):
                sched.submit(f"d{b}", p, SamplingParams(max_tokens=steps + 1))
            return prompts
        last = []
        for b, p in enumerate(prompts):
            engine.open_request(f"d{b}")
            for at in range(0, c, chunk):
                part = p[at:at + chunk]
                lg = engine.step([StepEntry(f"d{b}", part, [len(part) - 1] if at + chunk >= c else [])])
            last.append(engine.sample(lg, [SamplingParams()], [0])[0])
        return last

    def decode_device(B, c):
        """RUNS runs of K decode steps of B requests after c-token prompts, each step timed by its own pair of
        CUDA events; returns the runs' times in ms (each the sum of its K steps) and the launches of one run."""
        tokens = fill(B, c)
        run_ms, launches = [], None
        for i in range(W):
            lg = engine.step([StepEntry(f"d{b}", [tokens[b]], [0]) for b in range(B)])
            out = engine._sample_tokens[:B]
            kernels.sample_rows(lg, out)
            tokens = out.tolist()
        for r in range(RUNS):
            torch.cuda.synchronize()
            launches0 = (kernels.counters.own, kernels.counters.library)
            evs = []
            for i in range(K):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                lg = engine.step([StepEntry(f"d{b}", [tokens[b]], [0]) for b in range(B)])
                out = engine._sample_tokens[:B]
                kernels.sample_rows(lg, out)
                e1.record()
                tokens = out.tolist()  # waits for the step
                evs.append((e0, e1))
            torch.cuda.synchronize()
            launches = (kernels.counters.own - launches0[0], kernels.counters.library - launches0[1])
            run_ms.append(sum(a.elapsed_time(b) for a, b in evs))
        for b in range(B):
            engine.close_request(f"d{b}")
        engine.check()
        return run_ms, launches

    def decode_e2e(B):
        """E2E_STEPS steps through the scheduler: host token lists in, sampled host tokens out, wall clock."""
        sched = Scheduler(engine, prefill_chunk_size=0, max_tokens_per_step=opt.max_tokens_per_step, max_running=B,
                          run_ahead=True)
        fill(B, ctx, sched, steps=W + E2E_STEPS)
        while sched.counts()["prefilling"] or sched.counts()["waiting"]:
            sched.step()
        for _ in range(W):
            sched.step()
        torch.cuda.synchronize()
        t = time.perf_counter()
        produced = 0
        for _ in range(E2E_STEPS):  # each call launches a step and returns the host tokens of the step before it
            produced += sum(1 for ev in sched.step() if ev.token is not None)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t
        for rid in sched.active_ids():
            sched.cancel(rid)
        return produced / wall, produced

    def summarise(B, c, run_ms, launches):
        med = statistics.median(run_ms)
        return {"tok_s": B * K / med * 1e3, "ms_per_step": med / K, "launches": launches, "context": c,
                "runs_ms_per_step": [round(x / K, 4) for x in run_ms]}

    results = {}
    for B in batches:
        results[B] = summarise(B, ctx, *decode_device(B, ctx))
        print(f"[bench] decode batch {B}: {results[B]}", file=sys.stderr, flush=True)
    long_results = {}
    for c in long_ctx:
        long_results[c] = summarise(args.batch, c, *decode_device(args.batch, c))
        print(f"[bench] decode batch {args.batch} after {c}-token prompts: {long_results[c]}", file=sys.stderr, flush=True)
    e2e = None
    if not args.no_e2e:
        tok_s, produced = decode_e2e(args.batch)
        e2e = {"value": round(tok_s, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": int(engine.last_h2d_bytes), "d2h_bytes_per_step": int(args.batch * 4)}
        print(f"[bench] e2e {e2e} ({produced} tokens in {E2E_STEPS} steps)", file=sys.stderr, flush=True)
    sampler.stop()

    def roofline_frac(B, r):
        """Bytes a decode step of B requests must read (weights once + the live cache at the middle of the runs)
        over its time, as a fraction of the measured copy bandwidth."""
        mid = r["context"] + W + (RUNS * K + 1) / 2.0
        return (weight_bytes + B * mid * kv_per_token) / (r["ms_per_step"] * 1e-3) / 1e9 / peaks["hbm_gbs"]

    main_r = results[args.batch]
    mean_ctx = ctx + W + (RUNS * K + 1) / 2.0   # the runs follow one another: the median run sits near the middle
    step_bytes = weight_bytes + args.batch * mean_ctx * kv_per_token
    achieved = step_bytes / (main_r["ms_per_step"] * 1e-3) / 1e9
    line = {
        "metric": f"decode tokens/s (Qwen3-8B shape, batch {args.batch}, after {ctx:,}-token prompts)",
        "value": round(main_r["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(main_r["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: uniform random token ids, random weights (seed 42, N(0, 0.02))",
        "config": {"model": "Qwen3-8B shape", "layers": layers, "layers_full": layers_full, "hidden": cfg.hidden_size,
                   "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": args.batch,
                   "seq_len": ctx, "page_size": page, "prefill_tokens": 2048, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (15 GB of weights per step)", "decode": "CUDA graph per batch size",
                   "peaks": peaks["source"], "decode_runs": RUNS, "e2e_steps": E2E_STEPS},
        "e2e": e2e,
        "gpu_launches": int(main_r["launches"][0]),
        "library_launches": int(main_r["launches"][1]),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": {**{f"decode_b{B}": round(results[B]["tok_s"], 1) for B in batches if B != args.batch},
                   **{f"decode_b{args.batch}_ctx{c}": round(r["tok_s"], 1) for c, r in long_results.items()},
                   **{f"prefill_{t}": p["value"] for t, p in prefill_points.items()}},
        "points_frac": {**{f"decode_b{B}": round(roofline_frac(B, results[B]), 4) for B in batches if B != args.batch},
                        **{f"decode_b{args.batch}_ctx{c}": round(roofline_frac(args.batch, r), 4)
                           for c, r in long_results.items()},
                        **{f"prefill_{t}": p["frac"] for t, p in prefill_points.items()}},
        "runs_ms_per_step": main_r["runs_ms_per_step"],
        "clocks": sampler.summary(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
