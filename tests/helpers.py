"""Shared helpers of the GPU tests: model folders, replay of traces, comparison with the plain implementation."""
import json
import os

import numpy as np
import torch

import plain_qwen3 as plain
import tiny_configs


def make_model_dir(path, name, store="bfloat16", sharpen=None):
    """Writes a tiny random model with the tests' own writer (safetensors library, plain weights).

    Values are rounded to bfloat16 once so that the 32-bit and the bfloat16 run
    see the same weights; ``store`` chooses how the file holds them.  ``sharpen``: the query norms' weights
    are multiplied by it, so that scores are that much larger and a query's attention sits on a few keys
    anywhere in its context: a key that the engine dropped or misplaced then changes the logits visibly, which
    the flat attention of small random weights would hide."""
    from safetensors.torch import save_file
    cfg, seed, std, page = tiny_configs.get(name)
    w = plain.random_weights(cfg, seed, std)
    if sharpen:
        for k in w:
            if k.endswith("self_attn.q_norm.weight"):
                w[k] = w[k] * sharpen
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    if store == "float32":
        stored = {k: v.to(torch.float32) for k, v in w.items()}
    else:
        stored = w
    cfg["torch_dtype"] = store
    os.makedirs(path, exist_ok=True)
    save_file(stored, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    return cfg, {k: v.to(torch.float32) for k, v in w.items()}, page


def plain_logits(cfg, weights, tokens):
    return plain.forward(cfg, weights, tokens).numpy()


# ---------------------------------------------------------------------------------------------
# traces: lists of steps {"entries": [{"id", "tokens", "want"}], "end": [...]}
# ---------------------------------------------------------------------------------------------
def trace_whole(reqs):
    """Each request alone and whole: one step, all rows."""
    steps = []
    for rid, toks in reqs.items():
        steps.append({"entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def trace_prefill_then_decode(reqs, tail=32):
    """Most of it in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in reqs.items():
        n = len(toks)
        head = max(1, n - tail)
        steps.append({"entries": [{"id": rid, "tokens": list(toks[:head]), "want": list(range(head))}], "end": []})
        for i in range(head, n):
            steps.append({"entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def trace_portions(reqs, sizes=(7, 2, 13, 3, 2, 5, 16, 2, 9)):
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in reqs.items():
        i, k = 0, 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            steps.append({"entries": [{"id": rid, "tokens": list(toks[i:i + n]), "want": list(range(n))}], "end": []})
            i += n
            k += 1
        steps[-1]["end"] = [rid]
    return steps


def trace_mixed(reqs, max_live=4, seed=0, prefill_frac=0.6, portion_choices=(2, 3, 5, 7, 11, 16)):
    """Up to ``max_live`` live requests; portions of some beside decoded tokens of others in one step.

    A request is first fed in portions of random size up to ``prefill_frac`` of its
    length and then one token per step; requests start as others end, so pages
    are handed from finished requests to later ones."""
    rng = np.random.RandomState(seed)
    pending = list(reqs.items())
    live = {}  # rid -> [tokens, cursor, prefill_end]
    steps = []
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending.pop(0)
            live[rid] = [list(toks), 0, max(1, int(len(toks) * prefill_frac))]
        entries, end = [], []
        for rid in list(live):
            toks, cur, pend = live[rid]
            if rng.rand() < 0.15 and len(live) > 1:
                continue  # left out of this step, goes on later
            if cur < pend:
                n = min(int(rng.choice(list(portion_choices))), pend - cur)
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[cur:cur + n], "want": list(range(n))})
            live[rid][1] = cur + n
            if cur + n >= len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def trace_many_decoders(reqs, decode_steps=6, per_prefill_step=5):
    """All requests live at once: their prompts a few requests per step, then ``decode_steps`` steps in which
    every request brings one token (steps of as many single-token rows as there are requests)."""
    steps = []
    rids = list(reqs)
    for i in range(0, len(rids), per_prefill_step):
        entries = []
        for rid in rids[i:i + per_prefill_step]:
            head = max(1, len(reqs[rid]) - decode_steps)
            entries.append({"id": rid, "tokens": list(reqs[rid][:head]), "want": list(range(head))})
        steps.append({"entries": entries, "end": []})
    cursor = {rid: max(1, len(reqs[rid]) - decode_steps) for rid in rids}
    while any(cursor[rid] < len(reqs[rid]) for rid in rids):
        entries = []
        for rid in rids:
            if cursor[rid] < len(reqs[rid]):
                entries.append({"id": rid, "tokens": [reqs[rid][cursor[rid]]], "want": [0]})
                cursor[rid] += 1
        steps.append({"entries": entries, "end": []})
    steps[-1]["end"] = rids
    return steps


def max_live_tokens(steps, round_to=64):
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held, worst = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return worst


def replay(engine, steps):
    """Runs a trace on an Engine in this process; returns {(rid, position): logits row}."""
    from ccinfer_b200.engine.engine import StepEntry
    out = {}
    live = {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            if e["id"] not in live:
                engine.open_request(e["id"])
                live[e["id"]] = 0
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = engine.step(entries).cpu().numpy()
        engine.check()
        r = 0
        for e in st["entries"]:
            for w in e["want"]:
                out[(e["id"], live[e["id"]] + w)] = logits[r].copy()
                r += 1
            live[e["id"]] += len(e["tokens"])
        assert r == logits.shape[0]
        for rid in st["end"]:
            engine.close_request(rid)
            del live[rid]
    return out


def compare(rows, ref_by_req, rel_tol, what):
    """Every replayed row against the plain logits of its request; error relative to the largest logit."""
    worst = (0.0, None)
    for (rid, pos), row in rows.items():
        ref = ref_by_req[rid][pos]
        scale = max(1e-6, float(np.abs(ref_by_req[rid]).max()))
        err = float(np.abs(row - ref).max()) / scale
        if not np.isfinite(row).all():
            err = float("inf")
        if err > worst[0]:
            worst = (err, (rid, pos))
    assert worst[0] <= rel_tol, f"{what}: relative error {worst[0]:.3e} at (request, position) {worst[1]} > {rel_tol:.1e}"
    return worst[0]
