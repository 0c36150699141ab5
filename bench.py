#!/usr/bin/env python3
"""Decode and prefill throughput at the Qwen3-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  The default run: 36 layers,
hidden 4096, 32 q heads, 8 kv heads, head size 128, intermediate 12288,
vocabulary 151936, bfloat16, a batch of 8 requests decoding after 2,048-token
prompts.  It prints ONE JSON line:

  value      decoded tokens a second, from CUDA events around each of the K timed steps
  e2e        the same through the Python entry point's scheduler, by wall clock: host prompts in, every
             step one copy of the step's arrays from pinned memory and one read of the sampled token
             ids into host lists.  The scheduler runs one step ahead: a step is launched before the
             tokens of the step before it are read (the embedding takes them from the device)
  prefill    one 2,048-token prompt in one step: tokens a second and the fraction of the bf16 peak
  roofline   the decode step's bytes (every weight once + the cache of the live requests) / its time
  points     decode at batch 1 and 64
  clocks     SM clock and throttle reasons sampled during the timed regions

Every timed decode step reads 15 GB of weights, far more than the 126 MB L2, so no flush is needed
between iterations.  With --gpus N > 1 it prints one line that says so and exits with 2.

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
        decode_only = all(r.prefill_done for r in sched.active.values()) and not sched.waiting
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
    ctx, K, W = args.context, args.steps, args.warmup
    page = 16
    per_req = -(-(ctx + W + K + 2) // page) * page
    opt = EngineOptions(dtype="bfloat16", page_size=page, kv_tokens=max(batches) * per_req,
                        max_requests=max(batches), max_tokens_per_step=max(2048, ctx), max_context=per_req,
                        use_pdl=args.pdl)
    t0 = time.time()
    engine = Engine.from_random(cfg, seed=42, std=0.02, options=opt)
    torch.cuda.synchronize()
    print(f"[bench] model on the device in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    rng = np.random.RandomState(0)
    V = cfg.vocab_size
    sampler = ClockSampler()
    sampler.start()

    # ---- prefill: one 2,048-token prompt in one step ----
    prefill = None
    if not args.no_prefill:
        Tp = 2048
        times = []
        for i in range(W + 5):
            toks = rng.randint(0, V, size=Tp).tolist()
            engine.open_request("p")
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            engine.step([StepEntry("p", toks, [Tp - 1])])
            e1.record()
            torch.cuda.synchronize()
            engine.close_request("p")
            if i >= W:
                times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        prefill = {"value": round(Tp / ms * 1e3, 1), "tokens": Tp, "ms": round(ms, 3),
                   "frac": round(prefill_flops(Tp) / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}
        print(f"[bench] prefill {prefill}", file=sys.stderr, flush=True)

    # ---- decode ----
    def fill(B, sched=None):
        """Opens B requests and brings each to ``ctx`` cached tokens (prompts in steps of up to 2,048 tokens)."""
        prompts = [rng.randint(0, V, size=ctx).tolist() for _ in range(B)]
        if sched is not None:
            for b, p in enumerate(prompts):
                sched.submit(f"d{b}", p, SamplingParams(max_tokens=W + K + 1))
            return prompts
        last = []
        for b, p in enumerate(prompts):
            engine.open_request(f"d{b}")
            lg = engine.step([StepEntry(f"d{b}", p, [ctx - 1])])
            last.append(engine.sample(lg, [SamplingParams()], [0])[0])
        return last

    def decode_device(B):
        """K decode steps of B requests, each step timed by its own pair of CUDA events."""
        tokens = fill(B)
        greedy = [SamplingParams()] * B
        evs = []
        launches0 = None
        for i in range(W + K):
            if i == W:
                torch.cuda.synchronize()
                launches0 = (kernels.counters.own, kernels.counters.library)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            lg = engine.step([StepEntry(f"d{b}", [tokens[b]], [0]) for b in range(B)])
            out = engine._sample_tokens[:B]
            kernels.sample_rows(lg, out)
            e1.record()
            tokens = out.tolist()  # waits for the step
            if i >= W:
                evs.append((e0, e1))
        torch.cuda.synchronize()
        launches = (kernels.counters.own - launches0[0], kernels.counters.library - launches0[1])
        ms = [a.elapsed_time(b) for a, b in evs]
        for b in range(B):
            engine.close_request(f"d{b}")
        engine.check()
        return sum(ms), launches

    def decode_e2e(B):
        """The same K steps through the scheduler: host token lists in, sampled host tokens out, wall clock."""
        sched = Scheduler(engine, prefill_chunk_size=0, max_tokens_per_step=opt.max_tokens_per_step, max_running=B,
                          run_ahead=True)
        fill(B, sched)
        while any(not r.prefill_done for r in sched.active.values()) or sched.waiting:
            sched.step()
        for _ in range(W):
            sched.step()
        torch.cuda.synchronize()
        t = time.perf_counter()
        produced = 0
        for _ in range(K):  # each call launches a step and returns the host tokens of the step before it
            produced += sum(1 for ev in sched.step() if ev.token is not None)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t
        for rid in list(sched.active):
            sched.cancel(rid)
        return produced / wall, produced

    results = {}
    for B in batches:
        total_ms, launches = decode_device(B)
        results[B] = {"tok_s": B * K / total_ms * 1e3, "ms_per_step": total_ms / K, "launches": launches}
        print(f"[bench] decode batch {B}: {results[B]}", file=sys.stderr, flush=True)
    e2e = None
    if not args.no_e2e:
        tok_s, produced = decode_e2e(args.batch)
        e2e = {"value": round(tok_s, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": int(engine.layout.size * 4), "d2h_bytes_per_step": int(args.batch * 4)}
        print(f"[bench] e2e {e2e} ({produced} tokens)", file=sys.stderr, flush=True)
    sampler.stop()

    main_r = results[args.batch]
    mean_ctx = ctx + W + (K + 1) / 2.0
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
                   "peaks": peaks["source"]},
        "e2e": e2e,
        "gpu_launches": int(main_r["launches"][0]),
        "library_launches": int(main_r["launches"][1]),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": {f"decode_b{B}": round(results[B]["tok_s"], 1) for B in batches if B != args.batch},
        "clocks": sampler.summary(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
