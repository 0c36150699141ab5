"""Command line: ``ccinfer --model-path PATH [--prefill-chunk-size N] --prompt-ids 1,2,3 ...``.

``--model-path`` and ``--prefill-chunk-size`` are 7QiC/ccInfer's own flags (src/main.cpp:33-61, default
chunk 512, 0 = no chunking); ``--max-tokens``, ``--temperature``, ``--top-k``, ``--top-p`` carry the
names of its request fields (src/http/http_server.cpp:529-555) and ``--seed`` that of its
SamplingParams.  The server's ``--port`` has no meaning here.  Prompts are token ids.
``--random-config FILE --weights-seed N`` runs a model of that configuration with random weights drawn on the
device (the model that ``--write-random-model`` would write for the same seed), ``--dump-config`` prints the
typed configuration and exits.
"""
from __future__ import annotations

import argparse
import json
import sys


def _parse_prompts(args) -> list:
    prompts = []
    for spec in args.prompt_ids or []:
        prompts.append([int(t) for t in spec.replace(" ", "").split(",") if t])
    if args.prompt_file:
        with open(args.prompt_file) as f:
            for line in f:
                line = line.strip()
                if line:
                    prompts.append(json.loads(line) if line.startswith("[") else
                                   [int(t) for t in line.replace(",", " ").split()])
    if args.random_prompts:
        import numpy as np
        cfg = _config(args)
        rng = np.random.RandomState(args.prompt_seed)
        for n in args.random_prompts.split(","):
            prompts.append(rng.randint(0, cfg.vocab_size, size=int(n)).tolist())
    return prompts


def _config(args):
    """The typed configuration of --random-config or of the folder of --model-path."""
    from .config.registry import architecture_of, load_config
    if args.random_config:
        with open(args.random_config) as f:
            cj = json.load(f)
        return architecture_of(cj).parse_config(cj)
    return load_config(args.model_path)[1]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ccinfer", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-path", help="folder with config.json and model.safetensors")
    ap.add_argument("--prefill-chunk-size", type=int, default=512, help="0 = whole prompts")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--prompt-ids", action="append", help="comma-separated token ids; may be repeated")
    ap.add_argument("--prompt-file", help="one prompt a line: a JSON list or ids separated by blanks or commas")
    ap.add_argument("--random-prompts", help="lengths of random prompts, e.g. 5,11,17")
    ap.add_argument("--prompt-seed", type=int, default=0)
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0, help="0 = off; applies with a temperature above 0")
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--kv-tokens", type=int, default=None, help="tokens the cache pool holds (default 16384)")
    ap.add_argument("--kv-memory-fraction", type=float, default=None,
                    help="instead of --kv-tokens: share of the free device memory that goes to the cache pool")
    ap.add_argument("--max-requests", type=int, default=64)
    ap.add_argument("--max-running", type=int, default=16)
    ap.add_argument("--max-tokens-per-step", type=int, default=4096)
    ap.add_argument("--max-context", type=int, default=None)
    ap.add_argument("--eos-token-id", type=int, default=None)
    ap.add_argument("--warm-up", action="store_true", help="capture the decode graphs before the first request")
    ap.add_argument("--stats", action="store_true", help="print cache and scheduler figures to stderr")
    ap.add_argument("--write-random-model", metavar="CONFIG_JSON",
                    help="write a random model folder to --model-path from this config.json and exit")
    ap.add_argument("--random-config", metavar="CONFIG_JSON",
                    help="instead of --model-path: a model of this config.json with random weights (--weights-seed, "
                         "--weights-std) drawn on the device")
    ap.add_argument("--dump-config", action="store_true", help="print the typed configuration as JSON and exit")
    ap.add_argument("--weights-seed", type=int, default=0)
    ap.add_argument("--weights-std", type=float, default=0.02)
    args = ap.parse_args(argv)

    if not args.model_path and not args.random_config:
        ap.print_usage(sys.stderr)
        print("Error: --model-path (or --random-config) is required", file=sys.stderr)
        return 1
    if args.write_random_model and not args.model_path:
        print("Error: --write-random-model writes to --model-path", file=sys.stderr)
        return 1
    from .errors import CcinferError
    try:
        if args.write_random_model:
            from .config.registry import architecture_of
            from .weights.loader import write_random_model
            with open(args.write_random_model) as f:
                cj = json.load(f)
            cfg = architecture_of(cj).parse_config(cj)
            write_random_model(args.model_path, cfg, args.weights_seed, args.weights_std)
            print(f"wrote {args.model_path}", file=sys.stderr)
            return 0
        if args.dump_config:
            print(json.dumps(_config(args).to_json(), indent=1, sort_keys=True))
            return 0
        prompts = _parse_prompts(args)
        if not prompts:
            print("Error: no prompts (--prompt-ids, --prompt-file or --random-prompts)", file=sys.stderr)
            return 1
        from .engine.scheduler import SamplingParams
        from .llm import LLM
        options = dict(dtype=args.dtype, prefill_chunk_size=args.prefill_chunk_size, page_size=args.page_size,
                       kv_tokens=args.kv_tokens, kv_memory_fraction=args.kv_memory_fraction,
                       max_requests=args.max_requests, max_tokens_per_step=args.max_tokens_per_step,
                       max_context=args.max_context, max_running=args.max_running, eos_token_id=args.eos_token_id,
                       warm_up=args.warm_up)
        if args.random_config:
            llm = LLM.from_random(_config(args), args.weights_seed, args.weights_std, **options)
        else:
            llm = LLM(args.model_path, **options)
        sp = SamplingParams(max_tokens=args.max_tokens, top_k=args.top_k, top_p=args.top_p,
                            temperature=args.temperature, seed=args.seed)
        for i, toks in enumerate(llm.generate(prompts, sp)):
            print(json.dumps({"request": i, "prompt_tokens": len(prompts[i]), "token_ids": toks}))
        if args.stats:
            print(json.dumps(llm.stats()), file=sys.stderr)
    except CcinferError as e:
        print(f"Error [{e.code}]: {e}", file=sys.stderr)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
