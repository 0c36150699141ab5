"""Random configurations of the architecture against the plain implementation.

Every size and option of a configuration is drawn at random within what config.json allows: head sizes in
steps of 16 (one of them beyond 128), any number of heads and groups, widths and vocabularies that are no
power of two (odd ones too), the number of layers, the norms' eps, the rotation base, a tied or an untied
head, a window on some layers, the cache's page size.  Each model runs a mixed trace (up to four live
requests, portions beside decoded tokens, so few pages that they are used again) in 32-bit and in bfloat16
with and without CUDA graphs.  What the five fixed tiny configurations of the other tests do not happen to
hit, these may.  Sixteen configurations by default; CCB_FUZZ_SEEDS=N draws N (120 passed).
"""
import json
import os

import numpy as np
import pytest
import torch

import helpers
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


def _draw(seed):
    rng = np.random.RandomState(1000 + seed)
    hd = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 160]))
    nkv = int(rng.choice([1, 2, 3, 4]))
    group = int(rng.choice([1, 2, 3, 4, 5, 8]))
    nq = nkv * group
    layers = int(rng.randint(1, 5))
    cfg = {
        "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": layers,
        "hidden_size": int(rng.choice([24, 36, 50, 56, 72, 100, 136, 200, 264])),
        "num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": hd,
        "intermediate_size": int(rng.choice([48, 64, 70, 88, 128, 192, 200, 320])),
        "vocab_size": int(rng.choice([97, 128, 301, 500, 1001])),
        "rope_theta": float(rng.choice([1e4, 5e4, 1e6])), "rms_norm_eps": float(rng.choice([1e-6, 3e-6, 1e-5])),
        "tie_word_embeddings": bool(rng.randint(0, 2)), "max_position_embeddings": 512, "torch_dtype": "bfloat16",
    }
    if layers > 1 and rng.rand() < 0.5:
        cfg.update({"use_sliding_window": True, "sliding_window": int(rng.choice([9, 24, 40, 70])),
                    "max_window_layers": int(rng.randint(0, layers))})
    page = int(rng.choice([4, 8, 16, 32]))
    std = float(rng.choice([0.03, 0.05]))
    lengths = [int(x) for x in rng.randint(1, 260, size=5)]
    return cfg, page, std, lengths


@pytest.mark.parametrize("seed", range(int(os.environ.get("CCB_FUZZ_SEEDS", "16"))))
def test_random_configuration_matches_plain(tmp_path, seed):
    from safetensors.torch import save_file
    from ccinfer_b200.engine.engine import Engine, EngineOptions
    cfg, page, std, lengths = _draw(seed)
    w = {k: v.to(torch.bfloat16) for k, v in plain.random_weights(cfg, seed, std).items()}
    d = str(tmp_path)
    save_file(w, os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    weights = {k: v.to(torch.float32) for k, v in w.items()}
    rng = np.random.RandomState(seed)
    reqs = {f"r{i}": rng.randint(0, cfg["vocab_size"], size=n).tolist() for i, n in enumerate(lengths)}
    ref = {rid: helpers.plain_logits(cfg, weights, toks) for rid, toks in reqs.items()}
    what = {k: cfg[k] for k in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                                "head_dim", "intermediate_size", "vocab_size")}
    what.update(page=page, window=cfg.get("sliding_window"), window_from=cfg.get("max_window_layers"))
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 2e-2)):   # seen: 1.6e-6 and 8.6e-3
        for graphs in (False, True):
            steps = helpers.trace_mixed(reqs, max_live=4, seed=seed + (7 if graphs else 0),
                                        portion_choices=(2, 3, 5, 16, 70, 130))
            pool = helpers.max_live_tokens(steps, round_to=max(64, page))
            eng = Engine.from_model_dir(d, EngineOptions(
                dtype=dtype, page_size=page, kv_tokens=pool, max_requests=8, max_tokens_per_step=max(pool, 8),
                max_context=pool, use_graphs=graphs))
            rows = helpers.replay(eng, steps)
            worst = helpers.compare(rows, ref, tol, f"random configuration {seed} {what} {dtype} graphs={graphs}")
            print(f"[worst] random configuration {seed} {what}, {dtype}, graphs {graphs}: {worst:.3e}")
            eng.cache.check_consistency()
            assert all(p.used_pages == 0 for p in eng.cache.pools)
            del eng
    torch.cuda.empty_cache()
