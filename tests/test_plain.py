"""The plain implementation checked against independent restatements of the same formulas (no GPU)."""
import math

import numpy as np
import torch

import plain_qwen3 as plain
import tiny_configs


def test_philox_known_answers():
    # Random123's known-answer vectors of Philox4x32-10
    z = np.zeros(1, dtype=np.uint64)
    r = plain.philox4x32([z, z, z, z], [z, z])
    assert [int(x[0]) for x in r] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    f = z + np.uint64(0xFFFFFFFF)
    r = plain.philox4x32([f, f, f, f], [f, f])
    assert [int(x[0]) for x in r] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]


def test_gumbel_draws_follow_softmax():
    logits = torch.tensor([0.0, 1.0, 2.0, -1.0], dtype=torch.float64)
    n, T = 4000, 0.7
    counts = np.zeros(4)
    for i in range(n):
        counts[plain.sample_temperature(logits, T, seed=11, out_index=i)] += 1
    p = torch.softmax(logits / T, 0).numpy()
    assert float(((counts - n * p) ** 2 / (n * p)).sum()) < 20.0
    assert plain.sample_temperature(logits, 0.0, 1, 0) == 2
    assert plain.greedy(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1  # ties to the lowest id


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = plain.rms_norm(x, w, 0.0)
    r = math.sqrt((9 + 16) / 2)
    assert torch.allclose(y, torch.tensor([[3 / r * 2, 4 / r * 0.5]], dtype=torch.float64))


def test_rope_is_a_rotation_by_pos_times_inv_freq():
    hd, theta = 8, 10000.0
    inv = plain.rope_inv_freq(hd, theta)
    assert torch.allclose(inv.double(), torch.tensor([theta ** (-2 * i / hd) for i in range(hd // 2)]).double(),
                          rtol=1e-7)
    x = torch.randn(5, 2, hd, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    pos = torch.tensor([0, 1, 2, 50, 1000])
    y = plain.apply_rope(x, pos, inv)
    z = torch.complex(x[..., :hd // 2], x[..., hd // 2:])
    ang = (pos.float()[:, None] * inv[None, :]).double()
    zr = z * torch.polar(torch.ones_like(ang), ang)[:, None, :]
    assert torch.allclose(y[..., :hd // 2], zr.real) and torch.allclose(y[..., hd // 2:], zr.imag)
    assert torch.equal(y[0], x[0])  # position 0 is the identity
    # the score of a rotated pair depends on the distance only
    q, k = x[0:1, 0:1], x[1:2, 0:1]
    s1 = (plain.apply_rope(q, torch.tensor([7]), inv) * plain.apply_rope(k, torch.tensor([3]), inv)).sum()
    s2 = (plain.apply_rope(q, torch.tensor([104]), inv) * plain.apply_rope(k, torch.tensor([100]), inv)).sum()
    assert abs(float(s1 - s2)) < 1e-4


def test_attention_by_loops():
    g = torch.Generator().manual_seed(1)
    T, nq, nkv, hd, W = 9, 4, 2, 6, 4
    q, k, v = (torch.randn(T, n, hd, dtype=torch.float64, generator=g) for n in (nq, nkv, nkv))
    for window in (None, W):
        out = plain.causal_attention(q, k, v, window)
        for t in range(T):
            for h in range(nq):
                kh = h // (nq // nkv)
                js = [j for j in range(t + 1) if window is None or t - j < window]
                s = np.array([float(q[t, h] @ k[j, kh]) / math.sqrt(hd) for j in js])
                p = np.exp(s - s.max())
                p /= p.sum()
                ref = sum(pj * v[j, kh].numpy() for pj, j in zip(p, js))
                assert np.allclose(out[t, h].numpy(), ref)


def test_a_token_does_not_see_the_future_and_window_layers_forget():
    cfg, seed, std, _ = tiny_configs.get("C")
    w = plain.random_weights(cfg, seed, std)
    toks = list(range(3, 63))
    full = plain.forward(cfg, w, toks)
    assert torch.allclose(plain.forward(cfg, w, toks[:40]), full[:40], atol=1e-12)
    assert [plain.layer_window(cfg, l) for l in range(4)] == [None, 24, 24, 24]
    cfg2 = dict(cfg, use_sliding_window=False)
    assert not torch.allclose(plain.forward(cfg2, w, toks)[-1], full[-1], atol=1e-6)
    assert torch.allclose(plain.forward(cfg2, w, toks)[:24], full[:24], atol=1e-12)  # inside the window: same


def test_tied_head_and_shapes():
    cfg, seed, std, _ = tiny_configs.get("A")
    w = plain.random_weights(cfg, seed, std)
    assert "lm_head.weight" not in w
    lg = plain.forward(cfg, w, [1, 2, 3])
    assert lg.shape == (3, cfg["vocab_size"])
    out = plain.generate(cfg, w, [5, 6, 7], 4)
    assert len(out) == 4 and out[0] == plain.greedy(plain.forward(cfg, w, [5, 6, 7])[-1])



def test_filtered_draws_stay_in_their_set_and_follow_the_renormalised_distribution():
    """top-k / top-p: every draw is one of the allowed tokens, top_k = 1 is the argmax, and the draws
    follow softmax over the allowed set."""
    import numpy as np
    import torch
    logits = torch.tensor([2.0, 1.5, 1.4, 0.2, -0.5, -1.0, -3.0, 0.9])
    T = 0.8
    assert all(plain.sample_filtered(logits, T, 1, i, top_k=1)[0] == 0 for i in range(20))
    n = 6000
    draws = [plain.sample_filtered(logits, T, 9, i, top_k=5, top_p=0.9)[0] for i in range(n)]
    p_all = torch.softmax(logits.double() / T, dim=0)
    top5 = torch.topk(logits, 5).indices.tolist()
    p5 = p_all[top5] / p_all[top5].sum()
    keep, acc = [], 0.0
    for j, t in enumerate(top5):           # topk returns them in descending order
        keep.append(t)
        acc += float(p5[j])
        if acc >= 0.9:
            break
    assert set(draws) <= set(keep)
    pk = (p_all[keep] / p_all[keep].sum()).numpy()
    counts = np.array([draws.count(t) for t in keep])
    chi2 = float(((counts - n * pk) ** 2 / (n * pk)).sum())
    assert chi2 < 30.0, chi2


# ---------------------------------------------------------------------------------------------
# The plain functions against what 7QiC/ccInfer's own CPU functions computed (tests/golden/parts_golden.npz,
# made by tests/golden/make_parts_golden.py from the function bodies of the reference's kernel tests).
# The reference computes in float and rounds its outputs to bfloat16; the plain functions compute in float64.
# ---------------------------------------------------------------------------------------------
import os

import pytest

BF16_ROUNDING = 2.0 ** -8     # half a unit in the last place of a bfloat16 value, relative, with room for float sums


@pytest.fixture(scope="module")
def golden():
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "parts_golden.npz"))
    return {k: g[k] for k in g.files}


def _close_to_bf16(got: torch.Tensor, ref: np.ndarray):
    ref = torch.from_numpy(ref).double().view(got.shape)
    return bool(((got.double() - ref).abs() <= BF16_ROUNDING * ref.abs() + 1e-6).all())


def test_rms_norm_matches_the_references_cpu_function(golden):
    g = golden
    y = plain.rms_norm(torch.from_numpy(g["norm_x"]).double(), torch.from_numpy(g["norm_w"]).double(),
                       float(g["size_NORM_EPS"]))
    assert _close_to_bf16(y, g["norm_out"])


def test_inverse_frequencies_match_the_references_evaluation(golden):
    """1.0f / std::pow(theta, float(2i) / float(dim)) as src/model/rope/rope_cache.cpp:31-35 evaluates it:
    equal in all but a few entries (1 of 432), where the reference's powf is one unit off the correctly rounded power."""
    ref = golden["inv_freq"]
    at = differ = 0
    for theta in (1e4, 5e4, 1e6):
        for dim in (16, 32, 48, 64, 128):
            mine = plain.rope_inv_freq(dim, theta).numpy()
            theirs = ref[at:at + dim // 2]
            at += dim // 2
            differ += int((mine != theirs).sum())
            assert np.all(np.abs(mine - theirs) <= 2 * np.spacing(theirs))   # one unit of the power: two of 1 / power
    assert at == ref.size and differ <= 2, differ


def test_rotation_matches_the_references_cpu_function(golden):
    g = golden
    T, nq, nkv, hd = (int(g["size_ROPE_" + k]) for k in ("T", "NQ", "NKV", "HD"))
    inv = plain.rope_inv_freq(hd, float(g["size_ROPE_THETA"]))
    pos = torch.from_numpy(g["rope_pos"].astype(np.int64))
    q = plain.apply_rope(torch.from_numpy(g["rope_q"]).double().view(T, nq, hd), pos, inv)
    k = plain.apply_rope(torch.from_numpy(g["rope_k"]).double().view(T, nkv, hd), pos, inv)
    assert _close_to_bf16(q, g["rope_q_out"]) and _close_to_bf16(k, g["rope_k_out"])


def test_silu_mul_matches_the_references_cpu_function(golden):
    g = golden
    gate, up = torch.from_numpy(g["silu_g"]).double(), torch.from_numpy(g["silu_u"]).double()
    # the activation of plain.swiglu, with identity projections around it
    eye = torch.eye(gate.numel(), dtype=torch.float64)
    act = plain.swiglu(torch.ones(1, 1, dtype=torch.float64), gate[:, None], up[:, None], eye)
    assert _close_to_bf16(act.view(-1), g["silu_out"])


def test_causal_attention_matches_the_references_cpu_function(golden):
    g = golden
    T, nq, nkv, hd = (int(g["size_ATT_" + k]) for k in ("T", "NQ", "NKV", "HD"))
    o = plain.causal_attention(torch.from_numpy(g["att_q"]).double().view(T, nq, hd),
                               torch.from_numpy(g["att_k"]).double().view(T, nkv, hd),
                               torch.from_numpy(g["att_v"]).double().view(T, nkv, hd))
    assert _close_to_bf16(o, g["att_out"])


def test_attention_over_pages_matches_the_references_cpu_function(golden):
    """One query per request over the keys that a block table names (the reference's cache layout:
    [page * page_size + offset][kv head][head size]); the reference's function returns float."""
    g = golden
    B, nq, nkv, hd, P, stride = (int(g["size_DEC_" + k]) for k in ("B", "NQ", "NKV", "HD", "P", "STRIDE"))
    kc = torch.from_numpy(g["dec_k"]).double().view(-1, P, nkv, hd)
    vc = torch.from_numpy(g["dec_v"]).double().view(-1, P, nkv, hd)
    q = torch.from_numpy(g["dec_q"]).double().view(B, nq, hd)
    bt = g["dec_bt"].reshape(B, stride)
    ref = torch.from_numpy(g["dec_out"]).double().view(B, nq, hd)
    for b in range(B):
        L = int(g["dec_ctx"][b])
        pages = torch.from_numpy(bt[b, :-(-L // P)].astype(np.int64))
        k = kc[pages].reshape(-1, nkv, hd)[:L]
        v = vc[pages].reshape(-1, nkv, hd)[:L]
        q_all = torch.zeros((L, nq, hd), dtype=torch.float64)
        q_all[-1] = q[b]
        o = plain.causal_attention(q_all, k, v)[-1]
        assert float((o - ref[b]).abs().max()) <= 2e-6 * float(ref[b].abs().max()) + 1e-6
