"""Each part alone against its plain function, the order of layers as data, and a toy architecture whose
mixer keeps state of its own, registered, built and stepped without a change to the package's files."""
import dataclasses
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def _rel(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert torch.isfinite(got).all()
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-9))


def _weights(specs, seed, std=0.1):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for s in specs:
        w = torch.randn(s.shape, generator=g) * std
        if s.init == "one_plus_normal":
            w = w + 1
        out[s.name] = w.to(torch.bfloat16).float()  # the same values in both compute types
    return out


def _fetch(weights, specs, dtype):
    by = {s.name: s for s in specs}

    def fetch(name):
        return weights[name].to("cuda", dtype=torch.float32 if by[name].role == "vector" else dtype).contiguous()
    return fetch


def _engine(plan, weights, dtype, page=8, tokens=256):
    from ccinfer_b200.engine.engine import Engine, EngineOptions
    return Engine(plan, _fetch(weights, plan.tensor_specs(), DT[dtype]),
                  EngineOptions(dtype=dtype, page_size=page, kv_tokens=tokens, max_requests=4,
                                max_tokens_per_step=tokens, use_graphs=False))


def _qwen_plan(hidden=48, heads=4, kv=2, hd=16, inter=72, vocab=97, layers=1, window=None, eps=1e-5, theta=1e4):
    from ccinfer_b200.config import Qwen3Config
    from ccinfer_b200.architectures.qwen3 import build_plan
    cfg = {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": layers, "hidden_size": hidden,
           "num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": hd, "intermediate_size": inter,
           "vocab_size": vocab, "rope_theta": theta, "rms_norm_eps": eps, "max_position_embeddings": 512}
    if window:
        cfg.update(use_sliding_window=True, sliding_window=window, max_window_layers=0)
    return cfg, build_plan(Qwen3Config.from_json(cfg))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parts_alone(dtype):
    """Norm, position encoding, feed-forward, embedding, head, mixer and block, each called by itself."""
    from ccinfer_b200.engine.engine import StepEntry
    from ccinfer_b200.parts import Residual
    cfg, plan = _qwen_plan(window=20)
    w = _weights(plan.tensor_specs(), 1)
    eng = _engine(plan, w, dtype)
    T = 45
    toks = list(range(3, 3 + T))
    eng.open_request("a")

    def run(step):
        block = plan.layers[0]
        g = torch.Generator().manual_seed(2)
        x_ref = torch.randn(T, 48, generator=g).to(DT[dtype]).double()
        x = x_ref.to("cuda", DT[dtype])
        p = "model.layers.0."
        wd = {k: v.double() for k, v in w.items()}
        # embedding
        stream = plan.embedding.forward(step)
        assert torch.equal(stream.h.cpu().double(), plain.embed(wd["model.embed_tokens.weight"], toks))
        # the embedding with the norm that folds it first: one kernel writes both
        s0 = plan.embedding.forward(step, block.norm1)
        assert torch.equal(s0.h, stream.h) and s0.ready is not None
        y0 = block.norm1.fold(s0)
        assert s0.ready is None
        assert _rel(y0, plain.rms_norm(stream.h.cpu().double(), wd[p + "input_layernorm.weight"], 1e-5)) <= TOL[dtype]
        s0 = plan.embedding.forward(step, block.norm1)          # another norm than announced: it norms the stream itself
        assert _rel(block.norm2.fold(s0), plain.rms_norm(stream.h.cpu().double(),
                                                         wd[p + "post_attention_layernorm.weight"], 1e-5)) <= TOL[dtype]
        # norm: plain apply, fold of a pending delta, fold on picked rows
        assert _rel(block.norm1.apply(x), plain.rms_norm(x_ref, wd[p + "input_layernorm.weight"], 1e-5)) <= TOL[dtype]
        h0 = stream.h.clone()
        stream.pending = x
        y = block.norm1.fold(stream)
        assert stream.pending is None and _rel(stream.h, h0.cpu().double() + x_ref) <= 1e-6
        assert _rel(y, plain.rms_norm(h0.cpu().double() + x_ref, wd[p + "input_layernorm.weight"], 1e-5)) <= TOL[dtype]
        rows = plan.final_norm.fold(stream, rows=step.logit_rows, n_rows=2)
        ref_rows = plain.rms_norm(stream.h.cpu().double(), wd["model.norm.weight"], 1e-5)[[0, T - 1]]
        assert _rel(rows, ref_rows) <= TOL[dtype]
        # head
        assert _rel(plan.head.forward(rows), rows.cpu().double() @ wd["lm_head.weight"].T) <= TOL[dtype]
        # position encoding by itself
        xq = x.view(T, 3, 16).contiguous()
        rot = block.mixer.position.apply(xq, step.positions)
        assert _rel(rot, plain.apply_rope(x_ref.view(T, 3, 16), torch.arange(T), plain.rope_inv_freq(16, 1e4))) <= TOL[dtype]
        # feed-forward
        ff = block.ffn.forward(x, step)
        assert _rel(ff, plain.swiglu(x_ref, wd[p + "mlp.gate_proj.weight"], wd[p + "mlp.up_proj.weight"],
                                     wd[p + "mlp.down_proj.weight"])) <= TOL[dtype]
        # mixer (windowed attention over the paged cache)
        from ccinfer_b200.engine.step import LayerCache
        cache = LayerCache(eng._cache[0], step.groups[0], True)
        att = block.mixer.forward(x, step, cache, None)
        ref_att = plain.attention_block(x_ref, wd, p + "self_attn.", cfg, torch.arange(T), window=20)
        assert _rel(att, ref_att) <= TOL[dtype]
        # the block: h += Attn(norm1(h)); pending = MLP(norm2(h))
        s2 = Residual(h0.clone())
        block.forward(s2, step, cache, None)
        hh = h0.cpu().double()
        hh = hh + plain.attention_block(plain.rms_norm(hh, wd[p + "input_layernorm.weight"], 1e-5), wd,
                                        p + "self_attn.", cfg, torch.arange(T), window=20)
        assert _rel(s2.h, hh) <= TOL[dtype]
        mlp = plain.swiglu(plain.rms_norm(hh, wd[p + "post_attention_layernorm.weight"], 1e-5),
                           wd[p + "mlp.gate_proj.weight"], wd[p + "mlp.up_proj.weight"], wd[p + "mlp.down_proj.weight"])
        assert _rel(s2.pending, mlp) <= TOL[dtype] * 2

    # a real step is laid out for the parts to run in (pages taken, arrays on the device); nothing is committed
    eng.try_step([StepEntry("a", toks, [0, T - 1])], run)
    assert eng.context_len("a") == 0 and all(p.used_pages == 0 for p in eng.cache.pools)
    eng.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_product_that_adds_into_the_stream_and_the_norm_after_it(dtype):
    """With few rows the last product of a part may take the sum and the norm after it apart
    (``ResidualSink`` / ``UnscaledRows``): whatever the part after the norm is, the rows it gets are
    norm(h + x W^T): as unscaled rows that the next product finishes, as a plain tensor for a part that takes no
    such rows, for another norm than the one that was announced, and for picked rows.  In 32-bit nothing is
    taken apart and the same calls give the same values."""
    from ccinfer_b200.engine.runtime import Runtime
    from ccinfer_b200.parts import Residual, RMSNorm
    from ccinfer_b200.parts.base import ResidualSink, UnscaledRows
    M, D, K, N2 = 7, 1040, 2304, 520
    rt = Runtime("cuda:0", DT[dtype], max_tokens=32, max_entries=8)
    g = torch.Generator().manual_seed(5)
    x_ref = torch.randn(M, K, generator=g).to(DT[dtype]).double()
    w_ref = (torch.randn(D, K, generator=g) * 0.05).to(DT[dtype]).double()
    w2_ref = (torch.randn(N2, D, generator=g) * 0.05).to(DT[dtype]).double()
    h_ref = torch.randn(M, D, generator=g).float().double()
    x, w, w2 = (t.to("cuda", DT[dtype]) for t in (x_ref, w_ref, w2_ref))
    weights = {"n.weight": 1 + 0.1 * torch.randn(D, generator=g), "m.weight": 1 + 0.1 * torch.randn(D, generator=g)}
    norm, other = RMSNorm(D, 1e-5, "n.weight"), RMSNorm(D, 2e-5, "m.weight", scratch_key="normed_other")
    for n in (norm, other):
        n.bind(rt, lambda name: weights[name].float().cuda())
    h_want = h_ref + x_ref @ w_ref.T
    want = plain.rms_norm(h_want, weights["n.weight"].double(), 1e-5)

    def produce():
        stream = Residual(h_ref.float().cuda())
        out = torch.empty((M, D), dtype=DT[dtype], device="cuda")
        stream.pending = rt.linear(out, x, w, sink=ResidualSink(stream, norm))
        return stream

    # the part after the norm takes unscaled rows: a product finishes them
    stream = produce()
    taken_apart = stream.unscaled is not None
    assert taken_apart == (dtype == "bfloat16") and (stream.pending is None) == taken_apart
    stream.takes_unscaled = True
    rows = norm.fold(stream)
    assert isinstance(rows, UnscaledRows) == taken_apart and stream.unscaled is None
    assert _rel(stream.h, h_want) <= 2e-5
    y = torch.empty((M, N2), dtype=DT[dtype], device="cuda")
    rt.linear(y, rows, w2)
    assert _rel(y, want @ w2_ref.T) <= TOL[dtype]
    assert _rel(rt.rows(rows), want) <= TOL[dtype]
    # it takes none: the norm finishes them itself
    stream = produce()
    stream.takes_unscaled = False
    y = norm.fold(stream)
    assert torch.is_tensor(y) and _rel(y, want) <= TOL[dtype] and _rel(stream.h, h_want) <= 2e-5
    # another norm than the one announced, and picked rows: the stream is complete, they norm it themselves
    stream = produce()
    stream.takes_unscaled = True
    y = other.fold(stream)
    assert torch.is_tensor(y) and stream.unscaled is None
    assert _rel(y, plain.rms_norm(h_want, weights["m.weight"].double(), 2e-5)) <= TOL[dtype]
    stream = produce()
    picked = torch.tensor([M - 1, 0], dtype=torch.int32, device="cuda")
    y = norm.fold(stream, rows=picked, n_rows=2)
    assert _rel(y, want[[M - 1, 0]]) <= TOL[dtype]
    rt.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_order_of_layers_is_data(dtype):
    """A layer named twice (two caches) and a layer that reads another run's cache, against plain parts."""
    from ccinfer_b200.engine.engine import StepEntry
    from ccinfer_b200.engine.plan import ModelPlan, RunEntry
    from ccinfer_b200.parts import (GroupedQueryAttention, OutputHead, PreNormBlock, RMSNorm, RotaryHalf, SwiGLU,
                                    TokenEmbedding)
    D, nq, nkv, hd, F, V, eps, theta = 32, 4, 2, 16, 40, 61, 1e-6, 1e4

    def block(name, own_kv):
        n = {k: f"{name}.attn.{k}" for k in ("q", "k", "v", "o", "q_norm", "k_norm")}
        return PreNormBlock(
            RMSNorm(D, eps, f"{name}.n1"),
            GroupedQueryAttention(D, nq, nkv, hd, RotaryHalf(hd, theta), n, qk_norm_eps=eps, own_kv=own_kv),
            RMSNorm(D, eps, f"{name}.n2"),
            SwiGLU(D, F, {k: f"{name}.ffn.{k}" for k in ("gate", "up", "down")}))

    plan = ModelPlan(TokenEmbedding(V, D, "emb"), [block("L0", True), block("L1", False)],
                     [RunEntry(0), RunEntry(1, cache_of=0), RunEntry(0)], RMSNorm(D, eps, "nf"),
                     OutputHead(D, V, "emb"), V, 256)
    assert plan.shared_tensor_names() == {"emb"}
    w = _weights(plan.tensor_specs(), 3, std=0.15)
    assert "L1.attn.k" not in w and "L1.attn.k_norm" not in w  # the borrowing layer has no k/v projections
    eng = _engine(plan, w, dtype)
    toks = [5, 9, 60, 1, 33, 7, 7, 12, 50, 2, 18, 41, 3]
    eng.open_request("r")
    got = torch.cat([eng.step([StepEntry("r", toks[:6], list(range(6)))]),
                     eng.step([StepEntry("r", toks[6:8], [0, 1])]),
                     eng.step([StepEntry("r", toks[8:], list(range(5)))])]).cpu()
    eng.check()
    assert len(eng._cache) == 2  # runs 0 and 2 own a cache, run 1 borrows

    wd = {k: v.double() for k, v in w.items()}
    T = len(toks)
    pos = torch.arange(T)
    inv = plain.rope_inv_freq(hd, theta)

    def qkv(x, name, with_kv=True):
        q = plain.apply_rope(plain.rms_norm((x @ wd[f"{name}.attn.q"].T).view(T, nq, hd), wd[f"{name}.attn.q_norm"], eps), pos, inv)
        if not with_kv:
            return q, None, None
        k = plain.apply_rope(plain.rms_norm((x @ wd[f"{name}.attn.k"].T).view(T, nkv, hd), wd[f"{name}.attn.k_norm"], eps), pos, inv)
        return q, k, (x @ wd[f"{name}.attn.v"].T).view(T, nkv, hd)

    def ffn(h, name):
        x = plain.rms_norm(h, wd[f"{name}.n2"], eps)
        return h + plain.swiglu(x, wd[f"{name}.ffn.gate"], wd[f"{name}.ffn.up"], wd[f"{name}.ffn.down"])

    h = plain.embed(wd["emb"], toks)
    q, k0, v0 = qkv(plain.rms_norm(h, wd["L0.n1"], eps), "L0")
    h = ffn(h + plain.causal_attention(q, k0, v0).reshape(T, -1) @ wd["L0.attn.o"].T, "L0")
    q, _, _ = qkv(plain.rms_norm(h, wd["L1.n1"], eps), "L1", with_kv=False)
    h = ffn(h + plain.causal_attention(q, k0, v0).reshape(T, -1) @ wd["L1.attn.o"].T, "L1")  # run 0's keys
    q, k2, v2 = qkv(plain.rms_norm(h, wd["L0.n1"], eps), "L0")
    h = ffn(h + plain.causal_attention(q, k2, v2).reshape(T, -1) @ wd["L0.attn.o"].T, "L0")
    ref = plain.rms_norm(h, wd["nf"], eps) @ wd["emb"].T
    assert _rel(got, ref) <= TOL[dtype]


# ---------------------------------------------------------------------------------------------
# a toy architecture, defined here: its mixer keeps a running sum per request in a state slot
# ---------------------------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    eps: float

    @classmethod
    def from_json(cls, j):
        return cls(j["vocab_size"], j["hidden_size"], j["intermediate_size"], j["eps"])

    def to_json(self):
        return {"architectures": ["ToyRunningMeanLM"], "torch_dtype": "float32", **dataclasses.asdict(self)}


def _toy_parts():
    from ccinfer_b200.parts.base import Mixer, StateNeed, TensorSpec

    class RunningMean(Mixer):
        """y_t = W mean(x_0 .. x_t): the sum and the count live in the request's state slot."""
        graph_safe = False  # it reads the step's host arrays

        def __init__(self, dim, name):
            self.dim, self.name = dim, name

        def tensor_specs(self):
            return [TensorSpec(self.name, (self.dim, self.dim))]

        def state_need(self):
            return StateNeed((self.dim + 1,), torch.float32)

        def bind(self, rt, fetch):
            self.w = fetch(self.name)

        def forward(self, x, step, cache, state):
            out = torch.empty_like(x)
            cu, slots = step.host.cu_q, step.host.state_slot
            for b in range(step.n_entries):
                if slots[b] < 0:
                    continue
                st = state[int(slots[b])]
                xs = x[int(cu[b]):int(cu[b + 1])].float()
                sums = st[:self.dim] + torch.cumsum(xs, 0)
                counts = st[self.dim] + torch.arange(1, xs.shape[0] + 1, device=x.device)
                out[int(cu[b]):int(cu[b + 1])] = ((sums / counts[:, None]) @ self.w.float().T).to(x.dtype)
                st[:self.dim] = sums[-1]
                st[self.dim] = counts[-1]
            return out

    return RunningMean


def _toy_plan(cfg: ToyConfig):
    from ccinfer_b200.engine.plan import ModelPlan, RunEntry
    from ccinfer_b200.parts import OutputHead, PreNormBlock, RMSNorm, SwiGLU, TokenEmbedding
    RunningMean = _toy_parts()
    D = cfg.hidden_size
    blocks = [PreNormBlock(RMSNorm(D, cfg.eps, f"b{i}.n1"), RunningMean(D, f"b{i}.mix"), RMSNorm(D, cfg.eps, f"b{i}.n2"),
                           SwiGLU(D, cfg.intermediate_size, {k: f"b{i}.{k}" for k in ("gate", "up", "down")}))
              for i in range(2)]
    return ModelPlan(TokenEmbedding(cfg.vocab_size, D, "emb"), blocks, [RunEntry(0), RunEntry(1)],
                     RMSNorm(D, cfg.eps, "nf"), OutputHead(D, cfg.vocab_size, "head"), cfg.vocab_size, None)


def _toy_plain(w, cfg, toks):
    w = {k: v.double() for k, v in w.items()}
    h = plain.embed(w["emb"], toks)
    n = torch.arange(1, len(toks) + 1, dtype=torch.float64)[:, None]
    for i in range(2):
        x = plain.rms_norm(h, w[f"b{i}.n1"], cfg.eps)
        h = h + (torch.cumsum(x, 0) / n) @ w[f"b{i}.mix"].T
        h = h + plain.swiglu(plain.rms_norm(h, w[f"b{i}.n2"], cfg.eps), w[f"b{i}.gate"], w[f"b{i}.up"], w[f"b{i}.down"])
    return plain.rms_norm(h, w["nf"], cfg.eps) @ w["head"].T


def test_toy_mixer_with_state_of_its_own(tmp_path):
    from ccinfer_b200.config import register_architecture
    from ccinfer_b200.engine.engine import Engine, EngineOptions, StepEntry
    from ccinfer_b200.weights import SafetensorsFile, write_random_model
    register_architecture("ToyRunningMeanLM", ToyConfig.from_json, _toy_plan, replace=True)
    cfg = ToyConfig(vocab_size=53, hidden_size=24, intermediate_size=40, eps=1e-6)
    d = write_random_model(str(tmp_path / "toy"), cfg, seed=9, std=0.3, store_dtype="float32")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    w = {n: f.tensor(n).clone() for n in f.entries}
    eng = Engine.from_model_dir(d, EngineOptions(dtype="float32", max_requests=2, max_tokens_per_step=64))
    assert not eng.graph_safe and len(eng.cache.groups) == 0 and len(eng._state) == 2
    rng = np.random.RandomState(0)
    a, b, c = (rng.randint(0, 53, size=n).tolist() for n in (19, 7, 11))
    eng.open_request("a")
    eng.open_request("b")
    rows = {"a": [], "b": [], "c": []}
    rows["a"].append(eng.step([StepEntry("a", a[:5], range(5))]))
    out = eng.step([StepEntry("b", b[:3], range(3)), StepEntry("a", a[5:6], [0])])   # a portion beside a single token
    rows["b"].append(out[:3]); rows["a"].append(out[3:])
    out = eng.step([StepEntry("a", a[6:17], range(11)), StepEntry("b", b[3:], range(4))])
    rows["a"].append(out[:11]); rows["b"].append(out[11:])
    eng.close_request("b")
    eng.open_request("c")  # takes b's slot: its state starts from zero again
    assert eng.cache.get("c").slot != eng.cache.get("a").slot
    out = eng.step([StepEntry("c", c, range(11)), StepEntry("a", a[17:], range(2))])
    rows["c"].append(out[:11]); rows["a"].append(out[11:])
    for rid, toks in (("a", a), ("b", b), ("c", c)):
        assert _rel(torch.cat(rows[rid]), _toy_plain(w, cfg, toks)) <= 2e-5, rid


# ---------------------------------------------------------------------------------------------
# more toy parts defined here: a feed-forward with routing, and other position encodings
# ---------------------------------------------------------------------------------------------
def _toy_routed_ffn():
    from ccinfer_b200.parts.base import FeedForward, TensorSpec

    class Top1Experts(FeedForward):
        """Router logits in float, one expert per token (ties to the lowest id), y = p_e * (x W_e^T)."""

        def __init__(self, dim, n_experts, prefix):
            self.dim, self.n, self.prefix = dim, n_experts, prefix

        def tensor_specs(self):
            return [TensorSpec(f"{self.prefix}.router", (self.n, self.dim))] + \
                   [TensorSpec(f"{self.prefix}.expert{e}", (self.dim, self.dim)) for e in range(self.n)]

        def bind(self, rt, fetch):
            self.router = fetch(f"{self.prefix}.router")
            self.experts = torch.stack([fetch(f"{self.prefix}.expert{e}") for e in range(self.n)])

        def forward(self, x, step):
            logits = x.float() @ self.router.float().T
            p = torch.softmax(logits, dim=-1)
            e = torch.argmax(logits, dim=-1)  # first maximum
            y = torch.einsum("td,tod->to", x.float(), self.experts[e].float())
            return (y * p.gather(1, e[:, None])).to(x.dtype)

    return Top1Experts


@pytest.mark.parametrize("pos_kind", ["scaled", "none"])
def test_toy_routed_feed_forward_and_other_position_encodings(pos_kind):
    """A block of the package's attention with a position encoding defined here (interpolated rotary, or none
    at all) and a routed feed-forward defined here, against the plain functions."""
    from ccinfer_b200.engine.engine import StepEntry
    from ccinfer_b200.engine.plan import ModelPlan, RunEntry
    from ccinfer_b200.parts import (GroupedQueryAttention, NoPosition, OutputHead, PreNormBlock, RMSNorm, RotaryHalf,
                                    TokenEmbedding)
    Top1Experts = _toy_routed_ffn()
    D, nq, nkv, hd, V, eps, theta, factor = 48, 3, 1, 16, 71, 1e-6, 1e4, 4.0

    class InterpolatedRotary(RotaryHalf):
        """Positions divided by a factor: the same kernel, another table."""

        def bind(self, rt, fetch):
            super().bind(rt, fetch)
            self.inv_freq = (self.inv_freq.double() / factor).float()

    position = InterpolatedRotary(hd, theta) if pos_kind == "scaled" else NoPosition()
    names = {k: f"a.{k}" for k in ("q", "k", "v", "o", "q_norm", "k_norm")}
    block = PreNormBlock(RMSNorm(D, eps, "n1"), GroupedQueryAttention(D, nq, nkv, hd, position, names, qk_norm_eps=eps),
                         RMSNorm(D, eps, "n2"), Top1Experts(D, 4, "moe"))
    plan = ModelPlan(TokenEmbedding(V, D, "emb"), [block], [RunEntry(0)], RMSNorm(D, eps, "nf"),
                     OutputHead(D, V, "head"), V, 256)
    w = _weights(plan.tensor_specs(), 11, std=0.2)
    eng = _engine(plan, w, "float32")
    assert not hasattr(block.ffn, "rt")  # the toy part is not one of the package's
    toks = list(np.random.RandomState(3).randint(0, V, size=37))
    eng.open_request("r")
    got = torch.cat([eng.step([StepEntry("r", toks[:20], range(20))]), eng.step([StepEntry("r", toks[20:22], [0, 1])]),
                     eng.step([StepEntry("r", toks[22:], range(15))])]).cpu()
    eng.check()

    wd = {k: v.double() for k, v in w.items()}
    T = len(toks)
    pos = torch.arange(T)
    h = plain.embed(wd["emb"], toks)
    x = plain.rms_norm(h, wd["n1"], eps)
    q = plain.rms_norm((x @ wd["a.q"].T).view(T, nq, hd), wd["a.q_norm"], eps)
    k = plain.rms_norm((x @ wd["a.k"].T).view(T, nkv, hd), wd["a.k_norm"], eps)
    v = (x @ wd["a.v"].T).view(T, nkv, hd)
    if pos_kind == "scaled":
        inv = (plain.rope_inv_freq(hd, theta).double() / factor).float()
        q, k = plain.apply_rope(q, pos, inv), plain.apply_rope(k, pos, inv)
    h = h + plain.causal_attention(q, k, v).reshape(T, -1) @ wd["a.o"].T
    x = plain.rms_norm(h, wd["n2"], eps)
    logits = x @ wd["moe.router"].T
    p = torch.softmax(logits, -1)
    e = torch.argmax(logits, -1)
    y = torch.stack([x[t] @ wd[f"moe.expert{int(e[t])}"].T * p[t, e[t]] for t in range(T)])
    ref = plain.rms_norm(h + y, wd["nf"], eps) @ wd["head"].T
    assert _rel(got, ref) <= 2e-5


def test_scratch_that_follows_the_step_is_refused_once_a_graph_holds_it():
    """A part that sizes its scratch by the step, not by its largest shape: after a decode step has been
    captured, the step that would move the buffer from under the graph raises instead."""
    from ccinfer_b200.engine.engine import Engine, EngineOptions, StepEntry
    from ccinfer_b200.engine.plan import ModelPlan, RunEntry
    from ccinfer_b200.errors import ScratchMoved
    from ccinfer_b200.parts import OutputHead, PreNormBlock, RMSNorm, SwiGLU, TokenEmbedding
    from ccinfer_b200.parts.base import Mixer, TensorSpec

    class Careless(Mixer):
        def __init__(self, dim):
            self.dim = dim

        def bind(self, rt, fetch):
            self.rt = rt

        def forward(self, x, step, cache, state):
            out = self.rt.scratch.get("careless_out", tuple(x.shape), x.dtype)   # the step's shape: the fault
            out.copy_(x)
            return out

    D, V, eps = 32, 41, 1e-6
    block = PreNormBlock(RMSNorm(D, eps, "n1"), Careless(D), RMSNorm(D, eps, "n2"),
                         SwiGLU(D, 64, {k: f"f.{k}" for k in ("gate", "up", "down")}))
    plan = ModelPlan(TokenEmbedding(V, D, "emb"), [block], [RunEntry(0)], RMSNorm(D, eps, "nf"),
                     OutputHead(D, V, "head"), V, 64)
    w = _weights(plan.tensor_specs(), 2)
    eng = Engine(plan, _fetch(w, plan.tensor_specs(), torch.float32),
                 EngineOptions(dtype="float32", page_size=8, kv_tokens=64, max_requests=4, max_tokens_per_step=32))
    eng.open_request("a")
    eng.open_request("b")
    eng.step([StepEntry("a", [1], [0])])          # a decode step of one row: captured, the pool is frozen
    assert eng.graph_replays == 1 and eng.rt.scratch.frozen
    eng.step([StepEntry("a", [2], [0])])          # the same shape: fine
    with pytest.raises(ScratchMoved, match="careless_out"):
        eng.step([StepEntry("a", [3], [0]), StepEntry("b", [4], [0])])
    assert eng.context_len("a") == 2 and eng.context_len("b") == 0   # the refused step changed nothing
    eng.cache.check_consistency()


# ---------------------------------------------------------------------------------------------
# a toy mixer that caches ONE vector per token (not keys and values), defined here
# ---------------------------------------------------------------------------------------------
def _toy_latent_mixer():
    from ccinfer_b200.parts.base import CachedTensor, CacheNeed, Mixer, TensorSpec

    class LatentMean(Mixer):
        """c_t = A x_t (r numbers) is cached in pages; y_t = B mean(c_j, j <= t, within the window if any)."""
        graph_safe = False   # it walks the step's host arrays

        def __init__(self, dim, r, prefix, window=None):
            self.dim, self.r, self.prefix, self.window = dim, r, prefix, window

        def tensor_specs(self):
            return [TensorSpec(f"{self.prefix}.down", (self.r, self.dim)), TensorSpec(f"{self.prefix}.up", (self.dim, self.r))]

        def cache_need(self):
            return CacheNeed((CachedTensor("latent", (self.r,), token_axis=0, dtype=torch.float32),), self.window)

        def bind(self, rt, fetch):
            self.a, self.b = fetch(f"{self.prefix}.down"), fetch(f"{self.prefix}.up")

        def forward(self, x, step, cache, state):
            g = cache.group
            pool = cache.tensors["latent"]                      # [pages, page_size, r]
            flat = pool.view(-1, self.r)
            c = x.float() @ self.a.float().T
            flat[g.slot_map.long()] = c                         # slot = page * page_size + offset
            out = torch.empty_like(x)
            P = g.page_size
            for b in range(step.n_entries):
                lo, hi = int(step.host.cu_q[b]), int(step.host.cu_q[b + 1])
                table = g.host_block_table[b]
                for t in range(lo, hi):
                    p = int(step.host.positions[t])
                    first = 0 if self.window is None else max(0, p - self.window + 1)
                    slots = [int(table[j // P]) * P + j % P for j in range(first, p + 1)]
                    assert min(slots) >= 0, "a page of the window was given back too early"
                    out[t] = (flat[torch.tensor(slots, device=x.device)].mean(0) @ self.b.float().T).to(x.dtype)
            return out

    return LatentMean


@pytest.mark.parametrize("window", [None, 11])
def test_toy_mixer_that_caches_one_vector_per_token(window):
    """The cache need of a mixer is a list of named tensors of its own shapes and types: here one float vector
    of 6 numbers per token in [pages, page_size, 6], beside an attention layer's keys and values in another
    group, with so few pages that they are used again."""
    from ccinfer_b200.engine.engine import Engine, EngineOptions, StepEntry
    from ccinfer_b200.engine.plan import ModelPlan, RunEntry
    from ccinfer_b200.parts import (GroupedQueryAttention, OutputHead, PreNormBlock, RMSNorm, RotaryHalf, SwiGLU,
                                    TokenEmbedding)
    LatentMean = _toy_latent_mixer()
    D, V, eps, r, hd = 32, 61, 1e-6, 6, 16
    names = {k: f"a.{k}" for k in ("q", "k", "v", "o", "q_norm", "k_norm")}
    blocks = [PreNormBlock(RMSNorm(D, eps, "b0.n1"), LatentMean(D, r, "b0.mix", window), RMSNorm(D, eps, "b0.n2"),
                           SwiGLU(D, 48, {k: f"b0.{k}" for k in ("gate", "up", "down")})),
              PreNormBlock(RMSNorm(D, eps, "b1.n1"), GroupedQueryAttention(D, 2, 1, hd, RotaryHalf(hd, 1e4), names),
                           RMSNorm(D, eps, "b1.n2"), SwiGLU(D, 48, {k: f"b1.{k}" for k in ("gate", "up", "down")}))]
    plan = ModelPlan(TokenEmbedding(V, D, "emb"), blocks, [RunEntry(0), RunEntry(1)], RMSNorm(D, eps, "nf"),
                     OutputHead(D, V, "head"), V, 256)
    w = _weights(plan.tensor_specs(), 21, std=0.2)
    opts = EngineOptions(dtype="float32", page_size=4, kv_tokens=128, max_requests=2, max_tokens_per_step=32,
                         use_graphs=False)
    eng = Engine(plan, _fetch(w, plan.tensor_specs(), torch.float32), opts)
    groups = {g.key: g for g in eng.cache.groups}
    if window is None:
        assert len(groups) == 1 and eng._cache[0]["latent"].shape == (32, 4, r) and eng._cache[0]["latent"].dtype == torch.float32
        assert eng._cache[1]["k"].shape == (32, 1, 4, hd)
    else:   # two groups; the window group's pool is as small as two requests can ever need
        assert groups[("window", 11)].num_pages == 2 * (11 // 4 + 2) + 32 // 4 < groups[("all",)].num_pages
    rng = np.random.RandomState(5)
    a, b = (rng.randint(0, V, size=n).tolist() for n in (41, 23))
    eng.open_request("a")
    eng.open_request("b")
    got = {"a": [], "b": []}
    ia = ib = 0
    for na, nb in ((5, 0), (1, 7), (9, 2), (1, 1), (13, 6), (2, 7), (10, 0)):
        entries = []
        if na:
            entries.append(StepEntry("a", a[ia:ia + na], range(na)))
        if nb:
            entries.append(StepEntry("b", b[ib:ib + nb], range(nb)))
        out = eng.step(entries).cpu()
        # rows come in the order of the entries
        if na:
            got["a"].append(out[:na])
        if nb:
            got["b"].append(out[na:])
        ia, ib = ia + na, ib + nb
        eng.cache.check_consistency()
    assert ia == len(a) and ib == len(b)
    eng.check()

    def plain_forward(toks):
        wd = {k: v.double() for k, v in w.items()}
        T = len(toks)
        h = plain.embed(wd["emb"], toks)
        c = plain.rms_norm(h, wd["b0.n1"], eps) @ wd["b0.mix.down"].T
        mean = torch.stack([c[max(0, t - window + 1) if window else 0:t + 1].mean(0) for t in range(T)])
        h = h + mean @ wd["b0.mix.up"].T
        h = h + plain.swiglu(plain.rms_norm(h, wd["b0.n2"], eps), wd["b0.gate"], wd["b0.up"], wd["b0.down"])
        x = plain.rms_norm(h, wd["b1.n1"], eps)
        pos = torch.arange(T)
        inv = plain.rope_inv_freq(hd, 1e4)
        q = plain.apply_rope((x @ wd["a.q"].T).view(T, 2, hd), pos, inv)
        k = plain.apply_rope((x @ wd["a.k"].T).view(T, 1, hd), pos, inv)
        h = h + plain.causal_attention(q, k, (x @ wd["a.v"].T).view(T, 1, hd)).reshape(T, -1) @ wd["a.o"].T
        h = h + plain.swiglu(plain.rms_norm(h, wd["b1.n2"], eps), wd["b1.gate"], wd["b1.up"], wd["b1.down"])
        return plain.rms_norm(h, wd["nf"], eps) @ wd["head"].T

    for rid, toks in (("a", a), ("b", b)):
        assert _rel(torch.cat(got[rid]), plain_forward(toks)) <= 2e-5, rid
    if window is not None:   # the window group really gave pages back while the requests ran
        pool = eng.cache.pools[list(groups).index(("window", 11))]
        assert pool.high_water < (41 + 23) // 4


# ---------------------------------------------------------------------------------------------
# position encodings with another pairing of coordinates: one defined here, and the package's options
# ---------------------------------------------------------------------------------------------
def _plain_partial_rope(x, positions, rotary_dim, theta, interleaved=False):
    """The first ``rotary_dim`` coordinates of every head turned, pairs (i, i + rotary_dim / 2) or (2i, 2i + 1)."""
    inv = plain.rope_inv_freq(rotary_dim, theta).double()
    ang = positions.double()[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2]
        out[..., 0:rotary_dim:2], out[..., 1:rotary_dim:2] = a * c - b * s, b * c + a * s
    else:
        a, b = x[..., :rotary_dim // 2], x[..., rotary_dim // 2:rotary_dim]
        out[..., :rotary_dim // 2], out[..., rotary_dim // 2:rotary_dim] = a * c - b * s, b * c + a * s
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["toy partial", "package partial", "package interleaved"])
def test_position_encodings_with_other_pairings(kind, dtype):
    """Partial rotation and interleaved pairs need no kernel of their own: the encoding states a permutation of
    the head's coordinates and a table with zeros, the attention mixer permutes its projections.  One such
    encoding is defined here (no file of the package changes), two are options of the package's RotaryHalf."""
    from ccinfer_b200.engine.engine import StepEntry
    from ccinfer_b200.engine.plan import ModelPlan, RunEntry
    from ccinfer_b200.parts import (GroupedQueryAttention, OutputHead, PositionEncoding, PreNormBlock, RMSNorm,
                                    RotaryHalf, SwiGLU, TokenEmbedding)
    D, nq, nkv, hd, V, eps, theta, rd = 64, 4, 2, 64, 83, 1e-6, 1e4, 24

    class ToyPartialRotary(PositionEncoding):
        """Rotates the first rd coordinates, pairs (i, i + rd / 2); written without the package's helper."""

        def bind(self, rt, fetch):
            table = torch.zeros(hd // 2)
            table[:rd // 2] = plain.rope_inv_freq(rd, theta)
            self.table = table.to(rt.device)

        def rotary_table(self):
            return self.table

        def head_permutation(self):
            rest = list(range(rd, hd))
            return (list(range(rd // 2)) + rest[:len(rest) // 2]) + (list(range(rd // 2, rd)) + rest[len(rest) // 2:])

    interleaved = kind == "package interleaved"
    position = {"toy partial": ToyPartialRotary(), "package partial": RotaryHalf(hd, theta, rotary_dim=rd),
                "package interleaved": RotaryHalf(hd, theta, rotary_dim=rd, interleaved=True)}[kind]
    names = {k: f"a.{k}" for k in ("q", "k", "v", "o", "q_norm", "k_norm")}
    block = PreNormBlock(RMSNorm(D, eps, "n1"), GroupedQueryAttention(D, nq, nkv, hd, position, names, qk_norm_eps=eps),
                         RMSNorm(D, eps, "n2"), SwiGLU(D, 96, {k: f"f.{k}" for k in ("gate", "up", "down")}))
    plan = ModelPlan(TokenEmbedding(V, D, "emb"), [block], [RunEntry(0)], RMSNorm(D, eps, "nf"),
                     OutputHead(D, V, "head"), V, 512)
    w = _weights(plan.tensor_specs(), 31, std=0.15)
    eng = _engine(plan, w, dtype, page=16, tokens=256)
    toks = list(np.random.RandomState(4).randint(0, V, size=150))
    eng.open_request("r")
    # a long portion (tensor-core prefill in bfloat16), short ones, and single tokens (the fused decode kernel)
    cuts = [0, 90, 97, 99] + list(range(100, 151))
    got = torch.cat([eng.step([StepEntry("r", toks[a:b], range(b - a))]).cpu() for a, b in zip(cuts, cuts[1:])])
    eng.check()

    wd = {k: v.double() for k, v in w.items()}
    T = len(toks)
    pos = torch.arange(T)
    h = plain.embed(wd["emb"], toks)
    x = plain.rms_norm(h, wd["n1"], eps)
    q = plain.rms_norm((x @ wd["a.q"].T).view(T, nq, hd), wd["a.q_norm"], eps)
    k = plain.rms_norm((x @ wd["a.k"].T).view(T, nkv, hd), wd["a.k_norm"], eps)
    q, k = (_plain_partial_rope(t, pos, rd, theta, interleaved) for t in (q, k))
    h = h + plain.causal_attention(q, k, (x @ wd["a.v"].T).view(T, nkv, hd)).reshape(T, -1) @ wd["a.o"].T
    h = h + plain.swiglu(plain.rms_norm(h, wd["n2"], eps), wd["f.gate"], wd["f.up"], wd["f.down"])
    ref = plain.rms_norm(h, wd["nf"], eps) @ wd["head"].T
    assert _rel(got, ref) <= TOL[dtype]
    if kind != "toy partial":   # the encoding alone
        xq = torch.randn((7, 3, hd), generator=torch.Generator().manual_seed(1)).to(DT[dtype])
        p7 = torch.tensor([0, 1, 5, 63, 64, 200, 511], dtype=torch.int32)
        rot = position.apply(xq.cuda(), p7.cuda())
        assert _rel(rot, _plain_partial_rope(xq.double(), p7, rd, theta, interleaved)) <= (1e-6 if dtype == "float32" else 8e-3)


def test_what_the_attention_mixer_cannot_do_is_refused():
    from ccinfer_b200.engine.plan import ModelPlan, RunEntry
    from ccinfer_b200.errors import Unsupported
    from ccinfer_b200.parts import (GroupedQueryAttention, OutputHead, PositionEncoding, PreNormBlock, RMSNorm, SwiGLU,
                                    TokenEmbedding)
    D, hd, V, eps = 32, 16, 19, 1e-6

    class DistanceBias(PositionEncoding):
        def rotary_table(self):
            return None

        def score_bias(self):
            return "slopes"

    class ShortTable(PositionEncoding):
        def bind(self, rt, fetch):
            self.t = torch.ones(3, device=rt.device)

        def rotary_table(self):
            return self.t

    for position in (DistanceBias(), ShortTable()):
        names = {k: f"a.{k}" for k in ("q", "k", "v", "o")}
        block = PreNormBlock(RMSNorm(D, eps, "n1"), GroupedQueryAttention(D, 2, 1, hd, position, names),
                             RMSNorm(D, eps, "n2"), SwiGLU(D, 48, {k: f"f.{k}" for k in ("gate", "up", "down")}))
        plan = ModelPlan(TokenEmbedding(V, D, "emb"), [block], [RunEntry(0)], RMSNorm(D, eps, "nf"),
                         OutputHead(D, V, "head"), V, 64)
        with pytest.raises(Unsupported):
            _engine(plan, _weights(plan.tensor_specs(), 1), "float32")
    with pytest.raises(Unsupported, match="multiples of 16"):
        GroupedQueryAttention(D, 2, 1, 120, DistanceBias(), {})
