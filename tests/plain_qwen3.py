"""Plain, slow Qwen3-dense implementation used as the oracle of the test-suite.

It rests on the formulas of 7QiC/ccInfer's kernels and model code (cited per
function as ``path:line`` within that project); the reference's own model code
cannot run without a GPU, boost and real weights, so nothing here was compared
with it live (the one part of it that does run on a CPU, its config.json
parser, is compared in tests/golden/).  Whole sequences, no cache, one function per part, CPU only, and
no code shared with the ``ccinfer_b200`` package: this file imports nothing
from it.  Everything is computed in float64 by default so that the error of
the engine's 32-bit path is visible down to 32-bit round-off.
"""
from __future__ import annotations

import math

import numpy as np
import torch

F64 = torch.float64

_PHILOX_M0 = 0xD2511F53
_PHILOX_M1 = 0xCD9E8D57
_PHILOX_W0 = 0x9E3779B9
_PHILOX_W1 = 0xBB67AE85


# ----------------------------------------------------------------------------
# weights
# ----------------------------------------------------------------------------
def tensor_shapes(cfg: dict) -> dict:
    """HF tensor names and shapes of a Qwen3 dense model.

    Names as loaded by src/model/qwen3/qwen3_weights.cpp:74-152.
    """
    D = cfg["hidden_size"]
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nq)
    hd = cfg.get("head_dim", D // nq)
    F = cfg["intermediate_size"]
    V = cfg["vocab_size"]
    shapes = {"model.embed_tokens.weight": (V, D), "model.norm.weight": (D,)}
    if not cfg.get("tie_word_embeddings", False):
        shapes["lm_head.weight"] = (V, D)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        shapes[p + "input_layernorm.weight"] = (D,)
        shapes[p + "post_attention_layernorm.weight"] = (D,)
        shapes[p + "self_attn.q_proj.weight"] = (nq * hd, D)
        shapes[p + "self_attn.k_proj.weight"] = (nkv * hd, D)
        shapes[p + "self_attn.v_proj.weight"] = (nkv * hd, D)
        shapes[p + "self_attn.o_proj.weight"] = (D, nq * hd)
        shapes[p + "self_attn.q_norm.weight"] = (hd,)
        shapes[p + "self_attn.k_norm.weight"] = (hd,)
        shapes[p + "mlp.gate_proj.weight"] = (F, D)
        shapes[p + "mlp.up_proj.weight"] = (F, D)
        shapes[p + "mlp.down_proj.weight"] = (D, F)
    return shapes


def random_weights(cfg: dict, seed: int, std: float = 0.02) -> dict:
    """Embedding and linears ~ N(0, std); norm weights = 1 + N(0, std)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        w = torch.randn(shape, generator=g, dtype=torch.float32) * std
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            w = w + 1.0
        out[name] = w
    return out


def _mulhilo32(a: int, b: torch.Tensor):
    """High and low 32 bits of a * b for a 32-bit constant a and 32-bit values b held in int64."""
    bl, bh = b & 0xFFFF, b >> 16
    lo_part = a * bl                       # < 2^48
    mid = a * bh + (lo_part >> 16)         # < 2^49
    hi = mid >> 16
    lo = ((mid & 0xFFFF) << 16) | (lo_part & 0xFFFF)
    return hi, lo


def philox4x32_torch(c, k):
    """Philox4x32-10 on int64 tensors holding 32-bit words; c = four counters, k = two keys (Python ints)."""
    k0, k1 = k
    c = list(c)
    for _ in range(10):
        hi0, lo0 = _mulhilo32(_PHILOX_M0, c[0])
        hi1, lo1 = _mulhilo32(_PHILOX_M1, c[2])
        c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
        k0, k1 = (k0 + _PHILOX_W0) & 0xFFFFFFFF, (k1 + _PHILOX_W1) & 0xFFFFFFFF
    return c


def _box_muller_f32(wa: torch.Tensor, wb: torch.Tensor):
    """Two standard normal values from two 32-bit words, in single float operations only.

    The engine's random-weights mode (7QiC/ccInfer has none: src/model/qwen3/qwen3_weights.cpp:49-51 loads
    checkpoints only) defines its stream so that it can be restated anywhere:
    u = ((wa >> 9) + 0.5) / 2^23; ln u = e ln 2 + ln m with u = m 2^e, m in (sqrt(1/2), sqrt 2],
    ln m = 2 s (1 + s^2/3 + s^4/5 + s^6/7 + s^8/9 + s^10/11), s = (m - 1) / (m + 1); r = sqrt(-2 ln u);
    the direction from the top 24 bits of wb: 3 bits of octant, 21 bits (+ 0.5) of x / (pi / 4), sine and
    cosine of x by their Taylor polynomials, placed on the circle by the octant.
    """
    F = torch.float32
    one = torch.tensor(1.0, dtype=F, device=wa.device)
    u = ((wa >> 9).to(F) + 0.5) * (1.0 / 8388608.0)
    bits = u.view(torch.int32)
    e = (bits >> 23) - 127
    m = ((bits & 0x7FFFFF) | 0x3F800000).view(F)
    big = m > torch.tensor(1.41421354, dtype=F, device=wa.device)
    m = torch.where(big, m * 0.5, m)
    e = e + big.to(torch.int32)
    s = (m - 1.0) / (m + 1.0)
    s2 = s * s
    poly = one / 11.0
    for d in (9.0, 7.0, 5.0, 3.0):
        poly = poly * s2 + one / d
    poly = poly * s2
    two_s = 2.0 * s
    ln_u = e.to(F) * torch.tensor(0.693147182, dtype=F, device=wa.device) + (two_s + two_s * poly)
    # the correctly rounded float square root: through float64, since torch's vectorised float sqrt on a
    # CPU is not (a float64 root, even one unit off, rounds to the right float)
    r = torch.sqrt((-2.0 * ln_u).double()).float()
    k = wb >> 8
    octant = k >> 21
    x = ((k & 0x1FFFFF).to(F) + 0.5) * (1.0 / 2097152.0) * torch.tensor(0.785398185, dtype=F, device=wa.device)
    x2 = x * x
    ps = one / 362880.0
    for num, d in ((-1.0, 5040.0), (1.0, 120.0), (-1.0, 6.0)):
        ps = ps * x2 + (num * one) / d
    sn = x + (x * x2) * ps
    pc = -one / 3628800.0
    for num, d in ((1.0, 40320.0), (-1.0, 720.0), (1.0, 24.0), (-1.0, 2.0)):
        pc = pc * x2 + (num * one) / d
    cs = 1.0 + x2 * pc
    swap = (((octant + 1) >> 1) & 1).bool()
    c = torch.where(swap, sn, cs)
    sv = torch.where(swap, cs, sn)
    c = torch.where((octant >= 2) & (octant <= 5), -c, c)
    sv = torch.where(octant >= 4, -sv, sv)
    return r * c, r * sv


def stream_normal(numel: int, seed: int, name: str, std: float, add_one: bool, device="cpu",
                  chunk: int = 1 << 22) -> torch.Tensor:
    """float32 [numel] of the random-weights stream of (seed, tensor name): element i takes word i % 4 of
    Philox4x32-10(counter = (i // 4 as two words, first 8 bytes of sha256(name) as two words),
    key = seed as two words); words 0, 1 make elements 0, 1 of a group and words 2, 3 elements 2, 3."""
    import hashlib
    key = int.from_bytes(hashlib.sha256(name.encode()).digest()[:8], "little")
    groups = (numel + 3) // 4
    out = torch.empty(groups * 4, dtype=torch.float32, device=device)
    for g0 in range(0, groups, chunk):
        g = torch.arange(g0, min(groups, g0 + chunk), dtype=torch.int64, device=device)
        n = g.numel()
        full = lambda v: torch.full((n,), v, dtype=torch.int64, device=device)
        w = philox4x32_torch([g & 0xFFFFFFFF, g >> 32, full(key & 0xFFFFFFFF), full(key >> 32)],
                             (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
        z0, z1 = _box_muller_f32(w[0], w[1])
        z2, z3 = _box_muller_f32(w[2], w[3])
        block = torch.stack([z0, z1, z2, z3], dim=1).reshape(-1) * torch.tensor(std, dtype=torch.float32, device=device)
        if add_one:
            block = block + 1.0
        out[4 * g0:4 * g0 + block.numel()] = block
    return out[:numel]


def stream_weights(cfg: dict, seed: int, std: float = 0.02, device="cpu") -> dict:
    """The random model that a seed names in the engine's random-weights mode: every tensor from its own
    stream (``stream_normal``), norm weights 1 + N(0, std), all in float32."""
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        n = 1
        for d in shape:
            n *= d
        norm = name.endswith("norm.weight") or name.endswith("layernorm.weight")
        out[name] = stream_normal(n, seed, name, std, norm, device).view(shape)
    return out


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------
def embed(table: torch.Tensor, ids) -> torch.Tensor:
    """out[t, :] = table[ids[t], :]  (src/kernel/elementwise/elementwise.cu:67-78)."""
    return table[torch.as_tensor(ids, dtype=torch.long, device=table.device)]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last axis.

    src/kernel/norm/rms_norm.cu:24-60 (the weight multiplies directly, not
    1 + w); the plain sum of squares of tests/kernel/test_rms_norm.cu:13-30 is
    used, not the kernel's bfloat16-rounded running sum.
    """
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * w


def rope_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """inv_freq[i] = 1.0f / powf(theta, float(2i) / float(head_dim)), i < head_dim / 2, in 32-bit steps as
    src/model/rope/rope_cache.cpp:31-35 (and tests/kernel/test_rope.cu:15-28) evaluate it.

    The power is taken in float64 and rounded to float32 (the correctly rounded powf); compared with the
    reference's own evaluation in tests/golden/parts_golden.npz.
    """
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / torch.tensor(float(head_dim), dtype=torch.float32)
    power = torch.pow(torch.tensor(float(theta), dtype=torch.float32).double(), exponent.double()).float()
    return torch.tensor(1.0, dtype=torch.float32) / power


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE over the whole head; x is [T, H, hd].

    angle = float32(pos) * inv_freq (32-bit product, as
    src/model/rope/rope_cache.cpp:38-45), pairs (i, i + hd/2), x0' = x0 c - x1 s,
    x1' = x1 c + x0 s (src/kernel/pos/rope.cu:41-46).
    """
    half = x.shape[-1] // 2
    angle = (positions.to(torch.float32)[:, None] * inv_freq.to(positions.device)[None, :]).to(x.dtype)  # [T, half]
    c = torch.cos(angle)[:, None, :]
    s = torch.sin(angle)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x1 * c + x0 * s], dim=-1)


def causal_attention(q, k, v, window=None) -> torch.Tensor:
    """Causal GQA attention of one whole sequence; q [T, nq, hd], k/v [T, nkv, hd].

    q head h uses kv head h // (nq / nkv); score = q.k / sqrt(hd); query p sees
    keys j <= p (src/kernel/attention/prefill_attn.cu:98-110, 145-241;
    tests/kernel/test_naive_attn.cu:16-65).  With ``window`` W a query also
    sees only keys with p - j < W.
    """
    T, nq, hd = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = 1.0 / math.sqrt(hd)
    pos = torch.arange(T, device=q.device)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= (pos[:, None] - pos[None, :]) < window
    out = torch.empty_like(q)
    for h in range(nq):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def attention_block(x, w, prefix, cfg, positions, window=None):
    """QKV projection, per-head q/k RMSNorm, RoPE, attention, output projection.

    src/model/qwen3/qwen3_model.cpp:158-298 in that order: the head norms come
    before RoPE and v is untouched.
    """
    D = cfg["hidden_size"]
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nq)
    hd = cfg.get("head_dim", D // nq)
    eps = cfg.get("rms_norm_eps", 1e-6)
    T = x.shape[0]
    q = (x @ w[prefix + "q_proj.weight"].T).view(T, nq, hd)
    k = (x @ w[prefix + "k_proj.weight"].T).view(T, nkv, hd)
    v = (x @ w[prefix + "v_proj.weight"].T).view(T, nkv, hd)
    q = rms_norm(q, w[prefix + "q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "k_norm.weight"], eps)
    inv_freq = rope_inv_freq(hd, cfg.get("rope_theta", 10000.0))
    q = apply_rope(q, positions, inv_freq)
    k = apply_rope(k, positions, inv_freq)
    o = causal_attention(q, k, v, window)
    return o.reshape(T, nq * hd) @ w[prefix + "o_proj.weight"].T


def swiglu(x, w_gate, w_up, w_down):
    """(silu(x Wg^T) * (x Wu^T)) Wd^T, silu(g) = g / (1 + exp(-g)).

    src/model/qwen3/qwen3_model.cpp:325-384; src/kernel/mlp/silu_mul.cu:24-28.
    """
    g = x @ w_gate.T
    u = x @ w_up.T
    return (g / (1.0 + torch.exp(-g)) * u) @ w_down.T


def layer_window(cfg: dict, layer: int):
    """Window of a layer from the architecture's own keys, or None.

    ``use_sliding_window`` switches it on; layers with index >=
    ``max_window_layers`` use ``sliding_window`` keys, the others all keys.
    (The reference reads none of these keys: src/model/config.h:55-133.)
    """
    if cfg.get("layer_types") is not None:  # a per-layer list, where the file has one, wins
        return int(cfg["sliding_window"]) if cfg["layer_types"][layer] == "sliding_attention" else None
    if not cfg.get("use_sliding_window", False) or cfg.get("sliding_window") is None:
        return None
    if layer >= cfg.get("max_window_layers", cfg["num_hidden_layers"]):
        return int(cfg["sliding_window"])
    return None


def forward(cfg: dict, weights: dict, tokens, dtype=F64) -> torch.Tensor:
    """Logits [T, V] of one whole sequence, pre-norm blocks.

    h += Attn(norm1(h)); h += MLP(norm2(h)); logits = norm_f(h) W_lm^T
    (src/model/qwen3/qwen3_model.cpp:141-426).  A tied model uses the embedding
    table as W_lm.
    """
    w = {k: v.to(dtype) for k, v in weights.items()}
    device = w["model.embed_tokens.weight"].device   # the weights decide where it runs (a GPU for large shapes)
    eps = cfg.get("rms_norm_eps", 1e-6)
    T = len(tokens)
    positions = torch.arange(T, device=device)
    h = embed(w["model.embed_tokens.weight"], torch.as_tensor(tokens, dtype=torch.long, device=device))
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        x = rms_norm(h, w[p + "input_layernorm.weight"], eps)
        h = h + attention_block(x, w, p + "self_attn.", cfg, positions, layer_window(cfg, l))
        x = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + swiglu(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                       w[p + "mlp.down_proj.weight"])
    x = rms_norm(h, w["model.norm.weight"], eps)
    w_lm = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return x @ w_lm.T


# ----------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------
def greedy(logits_row: torch.Tensor) -> int:
    """argmax, ties to the lowest id (src/kernel/sampling/sample.cu:32, 51-52)."""
    m = logits_row.max()
    return int(torch.nonzero(logits_row == m)[0, 0])


def philox4x32(counter, key):
    """Philox4x32-10 on numpy uint64 lanes; counter [4, n], key [2, n] -> [4, n]."""
    c = [np.asarray(x, dtype=np.uint64) & 0xFFFFFFFF for x in counter]
    k = [np.asarray(x, dtype=np.uint64) & 0xFFFFFFFF for x in key]
    for _ in range(10):
        p0 = _PHILOX_M0 * c[0]
        p1 = _PHILOX_M1 * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & 0xFFFFFFFF
        hi1, lo1 = p1 >> np.uint64(32), p1 & 0xFFFFFFFF
        c = [hi1 ^ c[1] ^ k[0], lo1, hi0 ^ c[3] ^ k[1], lo0]
        k = [(k[0] + _PHILOX_W0) & 0xFFFFFFFF, (k[1] + _PHILOX_W1) & 0xFFFFFFFF]
    return c


def gumbel_noise(seed: int, out_index: int, vocab: int) -> np.ndarray:
    """G_v = -log(-log u_v), u_v from word v % 4 of Philox(counter=(v // 4, out_index, 0, 0), key=(seed, 0)):
    one call of the generator serves four consecutive token ids.

    u = (top 23 bits of the word + 0.5) / 2^23, so 0 < u < 1 and u is exact in 32-bit floating point.
    """
    groups = (vocab + 3) // 4
    g = np.arange(groups, dtype=np.uint64)
    z = np.zeros(groups, dtype=np.uint64)
    r = philox4x32([g, z + np.uint64(out_index), z, z], [z + np.uint64(seed & 0xFFFFFFFF), z])
    words = np.stack(r, axis=1).reshape(-1)[:vocab]
    u = ((words >> np.uint64(9)).astype(np.float64) + 0.5) / float(1 << 23)
    return -np.log(-np.log(u))


def sample_temperature(logits_row: torch.Tensor, temperature: float, seed: int, out_index: int) -> int:
    """Gumbel-max draw from softmax(logits / T): argmax_v(logit_v / T + G_v).

    The reference carries temperature and seed (src/base/types.h:54-60) but
    implements greedy only; temperature <= 0 means greedy there and here.
    """
    if temperature <= 0:
        return greedy(logits_row)
    g = gumbel_noise(seed, out_index, logits_row.numel())
    z = logits_row.to(F64) / temperature + torch.from_numpy(g)
    return greedy(z)


def sample_filtered(logits_row: torch.Tensor, temperature: float, seed: int, out_index: int, top_k: int = 0,
                    top_p: float = 1.0):
    """A temperature draw restricted to the top-k logits and, within those, to the smallest set of most
    probable tokens whose probabilities at this temperature add up to top_p (ties at either threshold are
    kept).  The reference names both in its SamplingParams (src/base/types.h:54-60) and refuses them
    (src/model/model_runner.h:96-100).  Returns (token, margin): margin is how far the cumulative
    probability at the top-p cut is from top_p (a test skips rows where float rounding could move the cut).
    """
    if temperature <= 0:
        return greedy(logits_row), 1.0
    l = logits_row.to(F64)
    allowed = torch.ones_like(l, dtype=torch.bool)
    V = l.numel()
    if 0 < top_k < V:
        kth = torch.sort(l, descending=True).values[top_k - 1]
        allowed &= l >= kth
    margin = 1.0
    if top_p < 1.0:
        z = torch.where(allowed, torch.exp((l - l.max()) / temperature), torch.zeros_like(l))
        order = torch.argsort(l, descending=True, stable=True)
        cum = torch.cumsum(z[order], dim=0) / z.sum()
        first = int((cum >= top_p).nonzero()[0])          # the prefix up to here reaches top_p
        cut = l[order[first]]
        allowed &= l >= cut
        below = float(cum[first - 1]) if first > 0 else 0.0
        margin = min(float(cum[first]) - top_p, top_p - below)
    g = gumbel_noise(seed, out_index, V)
    zz = l / temperature + torch.from_numpy(g)
    zz = torch.where(allowed, zz, torch.full_like(zz, -float("inf")))
    return greedy(zz), margin


def generate(cfg, weights, prompt, max_tokens, temperature=0.0, seed=42, dtype=F64):
    """Whole-sequence recomputation per token; returns the new token ids."""
    toks = list(prompt)
    out = []
    for i in range(max_tokens):
        logits = forward(cfg, weights, toks, dtype)[-1]
        t = sample_temperature(logits, temperature, seed, i)
        out.append(t)
        toks.append(t)
    return out
