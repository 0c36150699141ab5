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
