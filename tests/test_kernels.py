"""Each kernel alone against the plain function of the same op, at sizes other than the engine tests'."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# error relative to the largest reference value
TOL = {"float32": 3e-6, "bfloat16": 1.2e-2}


def _k():
    from ccinfer_b200 import kernels
    return kernels


def _rel(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert torch.isfinite(got).all()
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-9))


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(shape, generator=g) * scale).to(dtype)
    return x.cuda(), x.double()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,D,V", [(1, 80, 11), (37, 1000, 301), (5, 4096, 64)])
def test_embed_gather(dtype, T, D, V):
    table, ref = _rand((V, D), DT[dtype], 1)
    ids = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    h = torch.empty((T, D), dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _k().embed_gather(h, table, ids.cuda(), status)
    assert torch.equal(h.cpu().double(), plain.embed(ref, ids.tolist()))
    assert int(status.item()) == 0
    bad = ids.clone()
    bad[0] = V
    _k().embed_gather(h, table, bad.cuda(), status)
    assert int(status.item()) == _k().ST_BAD_TOKEN
    assert float(h[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,D,V,eps", [(1, 80, 11, 1e-6), (37, 1000, 301, 1e-5), (5, 4096, 64, 3e-6), (4, 67, 9, 1e-6),
                                       (3, 8200, 5, 1e-6)])
def test_embed_rmsnorm(dtype, T, D, V, eps):
    """The gather and the first norm in one pass: the stream as embed_gather writes it, the normed rows as the
    plain formula gives them; widths that take the vector path, an odd one and one beyond it; a pending token;
    a bad id is reported and its rows are zero."""
    k = _k()
    table, ref = _rand((V, D), DT[dtype], 1)
    w, w_ref = _rand((D,), torch.float32, 6)
    w, w_ref = (w + 1).contiguous(), w_ref + 1
    ids = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    pending = torch.tensor([0, int(ids[-1])], dtype=torch.int32, device="cuda")
    sent = ids.clone()
    sent[-1] = -1 - 1                       # "the token last sampled for slot 1"
    h = torch.full((T, D), float("nan"), dtype=torch.float32, device="cuda")
    y = torch.full((T, D), float("nan"), dtype=DT[dtype], device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.embed_rmsnorm(y, h, table, sent.cuda(), w, eps, status=status, pending=pending)
    want = plain.embed(ref, ids.tolist())
    assert torch.equal(h.cpu().double(), want) and int(status.item()) == 0
    assert _rel(y, plain.rms_norm(want, w_ref, eps)) <= (2e-6 if dtype == "float32" else 8e-3)
    bad = ids.clone()
    bad[0] = V
    k.embed_rmsnorm(y, h, table, bad.cuda(), w, eps, status=status)
    assert int(status.item()) == k.ST_BAD_TOKEN
    assert float(h[0].abs().max()) == 0.0 == float(y[0].float().abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,D,eps", [(3, 80, 1e-6), (17, 1000, 1e-5), (2, 5120, 3e-6)])
def test_residual_rmsnorm(dtype, T, D, eps):
    k = _k()
    h0, h_ref = _rand((T, D), torch.float32, 3, 2.0)
    delta, d_ref = _rand((T, D), DT[dtype], 4)
    w, w_ref = _rand((D,), torch.float32, 5)
    w_ref = w_ref + 1
    w = (w + 1).contiguous()
    # fused with the residual sum
    h = h0.clone()
    y = torch.empty((T, D), dtype=DT[dtype], device="cuda")
    k.residual_rmsnorm(y, h, delta, w, eps)
    ref_h = h_ref + d_ref
    assert _rel(h, ref_h) <= 3e-7
    assert _rel(y, plain.rms_norm(ref_h, w_ref, eps)) <= TOL[dtype]
    # without a delta, h untouched
    h = h0.clone()
    k.residual_rmsnorm(y, h, None, w, eps)
    assert torch.equal(h, h0)
    assert _rel(y, plain.rms_norm(h_ref, w_ref, eps)) <= TOL[dtype]
    # picked rows: h untouched, delta added on the fly
    rows = torch.tensor([T - 1, 0, T - 1], dtype=torch.int32, device="cuda")
    h = h0.clone()
    yr = torch.empty((3, D), dtype=DT[dtype], device="cuda")
    k.residual_rmsnorm(yr, h, delta, w, eps, row_idx=rows)
    assert torch.equal(h, h0)
    assert _rel(yr, plain.rms_norm(ref_h, w_ref, eps)[[T - 1, 0, T - 1]]) <= TOL[dtype]
    # plain norm of a typed tensor
    x, x_ref = _rand((T, 3, D), DT[dtype], 6)
    y3 = torch.empty_like(x)
    k.rmsnorm(y3, x, w, eps)
    assert _rel(y3, plain.rms_norm(x_ref, w_ref, eps)) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,F", [(1, 7), (9, 208), (3, 12288)])
def test_silu_mul(dtype, T, F):
    gu, ref = _rand((T, 2 * F), DT[dtype], 7, 3.0)
    act = torch.empty((T, F), dtype=DT[dtype], device="cuda")
    _k().silu_mul(act, gu)
    g, u = ref[:, :F], ref[:, F:]
    assert _rel(act, g / (1 + torch.exp(-g)) * u) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,F,block", [(3, 64, 64), (9, 192, 64), (2, 12288, 64), (5, 30, 6), (4, 21, 7)])
def test_silu_mul_blocked_layout(dtype, T, F, block):
    """Gate and up columns in blocks: `block` of gate, then the `block` of up for the same channels."""
    k = _k()
    gu, ref = _rand((T, 2 * F), DT[dtype], 7, 3.0)
    g, u = ref[:, :F], ref[:, F:]
    blocked = k.interleave_gate_up(gu[:, :F].T.contiguous(), gu[:, F:].T.contiguous(), block).T.contiguous()
    act = torch.empty((T, F), dtype=DT[dtype], device="cuda")
    k.silu_mul(act, blocked, block)
    assert _rel(act, g / (1 + torch.exp(-g)) * u) <= TOL[dtype]
    from ccinfer_b200.errors import Unsupported
    with pytest.raises(Unsupported):
        k.silu_mul(act, blocked, F + 1)


@pytest.mark.parametrize("M,F,K", [(1, 64, 64), (8, 192, 512), (16, 12288, 256), (5, 640, 4096), (13, 128, 96)])
def test_gemm_tc_swiglu(M, F, K):
    """silu(a Wg^T) * (a Wu^T) as the epilogue of the tensor-core product, against the plain formula."""
    from ccinfer_b200.errors import Unsupported
    k = _k()
    a, a_ref = _rand((M, K), torch.bfloat16, 34)
    wg, wg_ref = _rand((F, K), torch.bfloat16, 35)
    wu, wu_ref = _rand((F, K), torch.bfloat16, 36)
    w = k.interleave_gate_up(wg, wu, k.SWIGLU_BLOCK)
    act = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.gemm_tc_swiglu_bf16(act, a, w, status)
    assert int(status.item()) == 0
    g, u = a_ref @ wg_ref.T, a_ref @ wu_ref.T
    assert _rel(act, g / (1 + torch.exp(-g)) * u) <= 8e-3
    with pytest.raises(Unsupported):  # more rows than the kernel takes
        k.gemm_tc_swiglu_bf16(torch.empty((17, F), dtype=torch.bfloat16, device="cuda"),
                              torch.zeros((17, K), dtype=torch.bfloat16, device="cuda"), w, status)


@pytest.mark.parametrize("M,N,K", [(1, 17, 33), (5, 301, 80), (33, 130, 257), (70, 64, 12), (130, 500, 96)])
def test_gemm_f32(M, N, K):
    a, a_ref = _rand((M, K), torch.float32, 8)
    w, w_ref = _rand((N, K), torch.float32, 9)
    c = torch.empty((M, N), dtype=torch.float32, device="cuda")
    _k().gemm_f32(c, a, w)
    assert _rel(c, a_ref @ w_ref.T) <= 2e-6
    # a row's result does not depend on the other rows of the batch
    c1 = torch.empty((1, N), dtype=torch.float32, device="cuda")
    _k().gemm_f32(c1, a[M - 1:M].contiguous(), w)
    assert torch.equal(c1[0], c[M - 1])


@pytest.mark.parametrize("M,N,K", [(3, 6144, 4096), (70, 4096, 12288), (2, 151936, 4096)])
def test_gemm_f32_at_the_sizes_of_a_large_model(M, N, K):
    """The sums of the 8B layer shape: 4,096 and 12,288 terms, the vocabulary's 151,936 features (a sample
    of them is compared in float64 on the GPU)."""
    g = torch.Generator(device="cuda").manual_seed(M + K)
    a = torch.randn((M, K), generator=g, device="cuda")
    w = torch.randn((N, K), generator=g, device="cuda") * 0.02
    c = torch.empty((M, N), dtype=torch.float32, device="cuda")
    _k().gemm_f32(c, a, w)
    cols = torch.randperm(N, generator=g, device="cuda")[:4096]
    ref = a.double() @ w[cols].double().T
    assert _rel(c[:, cols], ref) <= 1e-5   # float accumulation over up to 12,288 terms against float64
    assert _rel(c[:, N - 1:], a.double() @ w[N - 1:].double().T) <= 1e-5   # the last feature of a ragged tile
    c1 = torch.empty((1, N), dtype=torch.float32, device="cuda")
    _k().gemm_f32(c1, a[M - 1:M].contiguous(), w)
    assert torch.equal(c1[0], c[M - 1])


@pytest.mark.parametrize("out", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 24, 40), (7, 304, 80), (64, 1000, 256), (200, 96, 512)])
def test_gemm_bf16(out, M, N, K):
    k = _k()
    handle = k.CublasHandle(torch.device("cuda:0"))
    a, a_ref = _rand((M, K), torch.bfloat16, 10)
    w, w_ref = _rand((N, K), torch.bfloat16, 11)
    c = torch.empty((M, N), dtype=DT[out], device="cuda")
    handle.gemm_bf16(c, a, w)
    assert _rel(c, a_ref @ w_ref.T) <= (1e-5 if out == "float32" else 8e-3)
    handle.close()


@pytest.mark.parametrize("out", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 24, 64), (3, 301, 96), (8, 1000, 4096), (9, 500, 160), (16, 40, 12288),
                                   (17, 130, 256), (32, 6144, 512)])
def test_gemm_skinny(out, M, N, K):
    k = _k()
    a, a_ref = _rand((M, K), torch.bfloat16, 20)
    w, w_ref = _rand((N, K), torch.bfloat16, 21)
    c = torch.full((M, N), float("nan"), dtype=DT[out], device="cuda")
    k.gemm_skinny_bf16(c, a, w)
    assert _rel(c, a_ref @ w_ref.T) <= (2e-5 if out == "float32" else 8e-3)
    # a row's result does not depend on the other rows of the batch
    c1 = torch.empty((1, N), dtype=DT[out], device="cuda")
    k.gemm_skinny_bf16(c1, a[M - 1:M].contiguous(), w)
    assert torch.equal(c1[0], c[M - 1])
    # rows of a wider buffer (row stride > K) as the engine passes them
    wide = torch.zeros((M, K + 64), dtype=torch.bfloat16, device="cuda")
    wide[:, :K] = a
    c2 = torch.empty_like(c)
    k.gemm_skinny_bf16(c2, wide[:, :K], w)
    assert torch.equal(c2, c)


@pytest.mark.parametrize("out", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (200, 520, 192), (65, 96, 4096), (300, 301 * 8, 96),
                                   (2048, 1024, 1024)])
def test_gemm_tc_normal(out, M, N, K):
    k = _k()
    a, a_ref = _rand((M, K), torch.bfloat16, 30)
    w, w_ref = _rand((N, K), torch.bfloat16, 31)
    c = torch.full((M, N), float("nan"), dtype=DT[out], device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.gemm_tc_bf16(c, a, w, status=status)
    assert int(status.item()) == 0
    assert _rel(c, a_ref @ w_ref.T) <= (2e-5 if out == "float32" else 8e-3)


@pytest.mark.parametrize("out", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (200, 520, 192), (65, 96, 4096), (300, 301 * 8, 96), (1000, 2048, 1024),
                                   (2048, 6144, 512), (129, 257 * 8, 8 * 33), (5000, 768, 128), (257, 24576, 64)])
def test_gemm_tc_pair(out, M, N, K):
    """Two SMs on every tile, one cluster per pair of SMs over many tiles, two accumulators: ragged edges included."""
    k = _k()
    a, a_ref = _rand((M, K), torch.bfloat16, 21)
    w, w_ref = _rand((N, K), torch.bfloat16, 22, scale=0.1)
    c = torch.full((M, N), 7.0, dtype=DT[out], device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.gemm_tc_pair_bf16(c, a, w, status=status)
    assert int(status.item()) == 0
    assert _rel(c, a_ref @ w_ref.T) <= (2e-5 if out == "float32" else 6e-3)


@pytest.mark.parametrize("M,F,K", [(128, 64, 64), (300, 192, 512), (2048, 1024, 256), (77, 64 * 37, 320)])
def test_gemm_tc_pair_swiglu(M, F, K):
    k = _k()
    a, a_ref = _rand((M, K), torch.bfloat16, 23)
    gate, g_ref = _rand((F, K), torch.bfloat16, 24, scale=0.1)
    up, u_ref = _rand((F, K), torch.bfloat16, 25, scale=0.1)
    w = k.interleave_gate_up(gate, up, k.SWIGLU_BLOCK)
    act = torch.full((M, F), 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.gemm_tc_pair_bf16(act, a, w, swiglu=True, status=status)
    assert int(status.item()) == 0
    g, u = a_ref @ g_ref.T, a_ref @ u_ref.T
    assert _rel(act, g / (1 + torch.exp(-g)) * u) <= 8e-3


@pytest.mark.parametrize("out", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K,splits", [(1, 128, 64, 1), (8, 256, 512, 1), (8, 384, 4096, 4), (16, 130, 192, 3),
                                          (17, 1000, 256, 2), (33, 520, 12288, 5), (64, 6144, 4096, 3),
                                          (5, 301 * 8, 96, 1)])
def test_gemm_tc_swapped(out, M, N, K, splits):
    k = _k()
    a, a_ref = _rand((M, K), torch.bfloat16, 32)
    w, w_ref = _rand((N, K), torch.bfloat16, 33)
    c = torch.full((M, N), float("nan"), dtype=DT[out], device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    partial = torch.empty(splits * M * N, dtype=torch.float32, device="cuda")
    counters = torch.zeros(-(-N // 128), dtype=torch.int32, device="cuda")
    for _ in range(2):  # the counters are left at zero for the next launch
        c.fill_(float("nan"))
        k.gemm_tc_bf16(c, a, w, splits, partial, counters, status)
        assert int(status.item()) == 0
        assert _rel(c, a_ref @ w_ref.T) <= (2e-5 if out == "float32" else 8e-3)
    assert int(counters.abs().sum().item()) == 0
    assert k.gemm_tc_splits(M, N, K) >= 1


@pytest.mark.parametrize("out", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 16, 8), (1, 24, 64), (3, 301, 96), (8, 1000, 4096), (9, 500, 160), (16, 40, 12288),
                                   (8, 4096, 4096), (16, 6144, 520), (5, 130, 2048 + 72)])
def test_gemm_fewrows(out, M, N, K):
    """The TMA-ring few-rows product: ragged edges of N (blocks of 16 features) and of K (stages of 256),
    more stages than the ring holds, one to 16 tokens."""
    k = _k()
    a, a_ref = _rand((M, K), torch.bfloat16, 50)
    w, w_ref = _rand((N, K), torch.bfloat16, 51)
    c = torch.full((M, N), float("nan"), dtype=DT[out], device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.gemm_fewrows_bf16(c, a, w, status=status)
    assert int(status.item()) == 0
    assert _rel(c, a_ref @ w_ref.T) <= (2e-5 if out == "float32" else 8e-3)
    # a row's result does not depend on the other rows of the batch
    c1 = torch.empty((1, N), dtype=DT[out], device="cuda")
    k.gemm_fewrows_bf16(c1, a[M - 1:M].contiguous(), w, status=status)
    assert torch.equal(c1[0], c[M - 1])
    # rows of a wider buffer (row stride > K, output stride > N) as the engine passes them
    wide = torch.zeros((M, K + 64), dtype=torch.bfloat16, device="cuda")
    wide[:, :K] = a
    cw = torch.full((M, N + 24), float("nan"), dtype=DT[out], device="cuda")
    k.gemm_fewrows_bf16(cw[:, :N], wide[:, :K], w, status=status)
    assert torch.equal(cw[:, :N], c) and bool(torch.isnan(cw[:, N:].float()).all())
    assert int(status.item()) == 0


@pytest.mark.parametrize("M,F,K", [(1, 64, 64), (8, 192, 512), (8, 12288, 1024), (16, 64 * 75, 320), (5, 64 * 3, 4096 + 8)])
def test_gemm_fewrows_swiglu(M, F, K):
    """silu(a Wg^T) * (a Wu^T) as the epilogue: a block holds 8 gate rows and the 8 up rows of the same channels."""
    from ccinfer_b200.errors import Unsupported
    k = _k()
    a, a_ref = _rand((M, K), torch.bfloat16, 54)
    wg, wg_ref = _rand((F, K), torch.bfloat16, 55)
    wu, wu_ref = _rand((F, K), torch.bfloat16, 56)
    w = k.interleave_gate_up(wg, wu, k.SWIGLU_BLOCK)
    act = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.gemm_fewrows_bf16(act, a, w, swiglu=True, status=status)
    assert int(status.item()) == 0
    g, u = a_ref @ wg_ref.T, a_ref @ wu_ref.T
    assert _rel(act, g / (1 + torch.exp(-g)) * u) <= 8e-3
    with pytest.raises(Unsupported):  # more rows than the kernel takes
        k.gemm_fewrows_bf16(torch.empty((17, F), dtype=torch.bfloat16, device="cuda"),
                            torch.zeros((17, K), dtype=torch.bfloat16, device="cuda"), w, swiglu=True, status=status)


@pytest.mark.parametrize("M,D,K,N2,F", [(1, 48, 64, 40, 64), (5, 1000, 520, 301, 192), (8, 4096, 4096, 6144, 12288),
                                        (13, 2560, 9728, 4096, 64 * 151), (16, 136, 2048 + 72, 130, 64 * 3)])
def test_products_that_take_a_norm_apart(M, D, K, N2, F):
    """h += a Wo^T, then RMSNorm(h) feeding a plain product and a gated one, with no kernel for the norm: the
    first product's epilogue adds into h and leaves bf16(h * w_norm) and partial sums of h^2, the products after
    it multiply their results by each token's factor (before the activation).  Against the plain formulas in
    64-bit; the 16-feature blocks of the first product and D, N2 ragged against every tile."""
    k = _k()
    a, a_ref = _rand((M, K), torch.bfloat16, 70)
    wo, wo_ref = _rand((D, K), torch.bfloat16, 71, scale=0.05)
    h, h_ref = _rand((M, D), torch.float32, 72)
    h[min(M - 1, 2)] *= 30.0    # rows of very different size: each needs its own factor
    h_ref = h.double().cpu()
    nw, nw_ref = _rand((D,), torch.float32, 73)
    eps = 1e-5
    parts = k.gemm_fewrows_blocks(D)
    ssq = torch.full((16, parts), float("nan"), dtype=torch.float32, device="cuda")
    xw = torch.full((M, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.gemm_fewrows_norm_bf16(xw, a, wo, into=(h, nw, ssq), status=status)
    h_want = h_ref + a_ref @ wo_ref.T
    assert _rel(h, h_want) <= 2e-5
    assert _rel(xw, h_want * nw_ref) <= 8e-3
    assert _rel(ssq[:M].sum(1), (h_want ** 2).sum(1)) <= 2e-5
    normed = h_want * torch.rsqrt((h_want ** 2).mean(1, keepdim=True) + eps) * nw_ref
    # a plain product of those rows
    w2, w2_ref = _rand((N2, D), torch.bfloat16, 74, scale=0.05)
    for out in (torch.float32, torch.bfloat16):
        c = torch.full((M, N2), float("nan"), dtype=out, device="cuda")
        k.gemm_fewrows_norm_bf16(c, xw, w2, scale=(ssq, parts, D, eps), status=status)
        assert _rel(c, normed @ w2_ref.T) <= 8e-3
    # the gated product, both kernels that take such rows
    wg, wg_ref = _rand((F, D), torch.bfloat16, 75, scale=0.05)
    wu, wu_ref = _rand((F, D), torch.bfloat16, 76, scale=0.05)
    w = k.interleave_gate_up(wg, wu, k.SWIGLU_BLOCK)
    g, u = normed @ wg_ref.T, normed @ wu_ref.T
    want = g / (1 + torch.exp(-g)) * u
    act = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    k.gemm_fewrows_norm_bf16(act, xw, w, swiglu=True, scale=(ssq, parts, D, eps), status=status)
    assert _rel(act, want) <= 8e-3
    if k.gemm_tc_fits(D, xw, w):
        act2 = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
        k.gemm_tc_swiglu_scaled_bf16(act2, xw, w, ssq, parts, D, eps, status=status)
        assert _rel(act2, want) <= 8e-3
    assert int(status.item()) == 0
    # the same factor as the norm kernel's: the two ways to the normed rows differ by bfloat16 rounding only
    y = torch.empty((M, D), dtype=torch.bfloat16, device="cuda")
    k.residual_rmsnorm(y, h, None, nw, eps, status=status)
    assert _rel(y, normed) <= 8e-3


@pytest.mark.parametrize("M,N,K", [(8, 6144, 4096), (16, 6144, 4096), (3, 10240, 5120), (8, 16384, 2048), (12, 12288, 2560)])
def test_gemm_fewrows_many_blocks_per_sm(M, N, K):
    """Shapes with three to seven blocks resident per SM and more stages than the ring holds: the ring's
    stages are rewritten by TMA under the eyes of many readers.  (Without the proxy fence before the
    producer's copies these shapes gave wrong features in random blocks, a few hundred of 6,144.)"""
    k = _k()
    a, a_ref = _rand((M, K), torch.bfloat16, 57)
    w, w_ref = _rand((N, K), torch.bfloat16, 58, scale=0.05)
    want = a_ref @ w_ref.T
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    first = None
    for rep in range(8):
        c = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        k.gemm_fewrows_bf16(c, a, w, status=status)
        assert _rel(c, want) <= 2e-5, rep
        first = c if first is None else first
        assert torch.equal(c, first), rep
    assert int(status.item()) == 0


def test_gemm_skinny_refuses():
    from ccinfer_b200.errors import Unsupported
    k = _k()
    for M, K in ((33, 64), (4, 80)):
        a = torch.zeros((M, K), dtype=torch.bfloat16, device="cuda")
        w = torch.zeros((16, K), dtype=torch.bfloat16, device="cuda")
        c = torch.zeros((M, 16), dtype=torch.bfloat16, device="cuda")
        assert not k.gemm_skinny_fits(M, K, a, w)
        with pytest.raises(Unsupported):
            k.gemm_skinny_bf16(c, a, w)


def _paged_case(dtype, lens_ctx, lens_new, nq, nkv, hd, P, seed, window=None, peak=None):
    """Random keys in a shuffled page pool; returns inputs of the attention kernel and the plain result.

    ``peak`` = (entry, key position): that key and the entry's last query are scaled so that this one
    score stands out, which shows whether a far key or a key on a page's edge is really read."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens_ctx)
    total_pages = sum(-(-(c + n) // P) for c, n in zip(lens_ctx, lens_new)) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    stride = max(-(-(c + n) // P) for c, n in zip(lens_ctx, lens_new)) + 1
    k_cache = torch.zeros((total_pages, nkv, P, hd))
    v_cache = torch.zeros((total_pages, nkv, P, hd))
    # stale data everywhere: what is not a visible key must not matter
    k_cache.normal_(generator=g).mul_(5)
    v_cache.normal_(generator=g).mul_(5)
    bt = torch.full((B, stride), -1, dtype=torch.int32)
    qs, pos, eot, refs = [], [], [], []
    for b, (c, n) in enumerate(zip(lens_ctx, lens_new)):
        L = c + n
        k = torch.randn((L, nkv, hd), generator=g)
        v = torch.randn((L, nkv, hd), generator=g)
        q = torch.randn((L, nq, hd), generator=g)
        if peak is not None and peak[0] == b:
            k[peak[1]] *= 6.0
            q[L - 1] = k[peak[1]].repeat_interleave(nq // nkv, dim=0) * 1.0
        k, v, q = (t.to(DT[dtype]).float() for t in (k, v, q))
        for lp in range(-(-L // P)):
            page = perm.pop()
            bt[b, lp] = page
            lo, hi = lp * P, min(L, lp * P + P)
            k_cache[page, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            v_cache[page, :, :hi - lo] = v[lo:hi].transpose(0, 1)
        ref = plain.causal_attention(q.double(), k.double(), v.double(), window)
        refs.append(ref[c:])
        qs.append(q[c:])
        pos += list(range(c, L))
        eot += [b] * n
    dev = lambda t, dt=None: (t.to(dt) if dt else t).cuda().contiguous()
    return (dev(torch.cat(qs), DT[dtype]), dev(k_cache, DT[dtype]), dev(v_cache, DT[dtype]),
            dev(torch.tensor(pos, dtype=torch.int32)), dev(torch.tensor(eot, dtype=torch.int32)), dev(bt),
            torch.cat(refs))


ATTN_CASES = [
    # ctx, new, nq, nkv, hd, page, window
    ([0], [1], 2, 1, 16, 4, None),
    ([0, 5, 31], [9, 1, 2], 6, 3, 48, 8, None),
    ([100, 0, 63], [1, 70, 1], 8, 2, 64, 16, None),
    ([0, 40, 129], [33, 3, 1], 4, 4, 80, 16, 24),
    ([300], [1], 16, 2, 128, 16, None),
    ([17, 250], [40, 1], 5, 1, 256, 32, 100),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ATTN_CASES)
def test_paged_attention_generic(dtype, case):
    ctx, new, nq, nkv, hd, P, window = case
    q, kc, vc, pos, eot, bt, ref = _paged_case(dtype, ctx, new, nq, nkv, hd, P, seed=hd + len(ctx), window=window)
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _k().paged_attention_generic(q, kc, vc, out, pos, eot, bt, len(ctx), window or 0, 1 / math.sqrt(hd), status)
    assert int(status.item()) == 0
    assert _rel(out, ref) <= (1e-5 if dtype == "float32" else 1.5e-2)


def _run_split(q, kc, vc, pos, eot, bt, n_entries, window, hd, splits, row0=0, n_rows=None, fn=None):
    k = _k()
    fn = fn or k.attention_split
    T, nq, _ = q.shape
    n_rows = T - row0 if n_rows is None else n_rows
    out = torch.zeros_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    part_acc = torch.empty(max(1, n_rows * nq * splits * hd), dtype=torch.float32, device="cuda")
    part_ml = torch.empty(max(1, n_rows * nq * splits * 2), dtype=torch.float32, device="cuda")
    fn(q, kc, vc, out, part_acc, part_ml, pos, eot, bt, n_entries, row0, n_rows, window or 0,
       1 / math.sqrt(hd), splits, status)
    assert int(status.item()) == 0
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("splits", [1, 3, 32])
@pytest.mark.parametrize("case", ATTN_CASES + [([700, 33], [1, 1], 32, 8, 128, 16, None),
                                                ([90], [2], 12, 2, 96, 8, 50), ([64], [1], 7, 7, 32, 16, None)])
def test_attention_split(dtype, case, splits):
    ctx, new, nq, nkv, hd, P, window = case
    q, kc, vc, pos, eot, bt, ref = _paged_case(dtype, ctx, new, nq, nkv, hd, P, seed=hd + len(ctx), window=window)
    out = _run_split(q, kc, vc, pos, eot, bt, len(ctx), window, hd, splits)
    assert _rel(out, ref) <= (1e-5 if dtype == "float32" else 1.5e-2)
    if q.shape[0] > 2:  # a range of rows only: the others stay untouched
        part = _run_split(q, kc, vc, pos, eot, bt, len(ctx), window, hd, splits, row0=1, n_rows=q.shape[0] - 2)
        assert torch.equal(part[1:-1], out[1:-1]) and float(part[0].abs().max()) == 0 == float(part[-1].abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far_key", [0, 15, 16, 255, 256, 257, 511])
def test_attention_split_reads_far_key(dtype, far_key):
    nq, nkv, hd, P = 8, 2, 128, 16
    L = 600
    q, kc, vc, pos, eot, bt, ref = _paged_case(dtype, [L - 1], [1], nq, nkv, hd, P, seed=far_key,
                                               peak=(0, far_key))
    for splits in (1, 5):
        out = _run_split(q, kc, vc, pos, eot, bt, 1, None, hd, splits)
        assert _rel(out, ref) <= (1e-5 if dtype == "float32" else 1.5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("edge", [-1, 0, 1])
def test_attention_split_window_edge(dtype, edge):
    nq, nkv, hd, P, W = 2, 1, 32, 8, 40
    L = 200
    key = (L - 1) - W + 1 + edge
    q, kc, vc, pos, eot, bt, ref = _paged_case(dtype, [L - 1], [1], nq, nkv, hd, P, seed=7, window=W,
                                               peak=(0, key))
    for splits in (1, 4):
        out = _run_split(q, kc, vc, pos, eot, bt, 1, W, hd, splits)
        assert _rel(out, ref) <= (1e-5 if dtype == "float32" else 1.5e-2)


MMA_CASES = [
    # ctx, new, nq, nkv, hd, page, window
    ([0], [1], 4, 1, 64, 16, None),
    ([700, 33, 64, 63], [1, 1, 1, 1], 32, 8, 128, 16, None),
    ([100, 0, 63], [1, 70, 1], 8, 2, 64, 8, None),
    ([300, 129], [5, 1], 12, 2, 128, 4, 100),
    ([511], [1], 40, 2, 128, 32, None),       # groups of 20 q heads: two head chunks per kv head
    ([90], [2], 3, 3, 64, 16, 50),
]


@pytest.mark.parametrize("splits", [1, 3, 32])
@pytest.mark.parametrize("case", MMA_CASES)
def test_attention_decode_mma(case, splits):
    ctx, new, nq, nkv, hd, P, window = case
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", ctx, new, nq, nkv, hd, P, seed=hd + len(ctx),
                                               window=window)
    out = _run_split(q, kc, vc, pos, eot, bt, len(ctx), window, hd, splits, fn=_k().attention_decode_mma)
    assert _rel(out, ref) <= 1.5e-2
    if q.shape[0] > 2:
        part = _run_split(q, kc, vc, pos, eot, bt, len(ctx), window, hd, splits, row0=1, n_rows=q.shape[0] - 2,
                          fn=_k().attention_decode_mma)
        assert torch.equal(part[1:-1], out[1:-1]) and float(part[0].abs().max()) == 0 == float(part[-1].abs().max())


@pytest.mark.parametrize("splits", [1, 3, 32])
@pytest.mark.parametrize("case", [c for c in MMA_CASES if c[5] >= 8])
def test_attention_decode_tma(case, splits):
    ctx, new, nq, nkv, hd, P, window = case
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", ctx, new, nq, nkv, hd, P, seed=hd + len(ctx),
                                               window=window)
    out = _run_split(q, kc, vc, pos, eot, bt, len(ctx), window, hd, splits, fn=_k().attention_decode_tma)
    assert _rel(out, ref) <= 1.5e-2
    if q.shape[0] > 2:
        part = _run_split(q, kc, vc, pos, eot, bt, len(ctx), window, hd, splits, row0=1, n_rows=q.shape[0] - 2,
                          fn=_k().attention_decode_tma)
        assert torch.equal(part[1:-1], out[1:-1]) and float(part[0].abs().max()) == 0 == float(part[-1].abs().max())


@pytest.mark.parametrize("splits", [2, 5, 64])
@pytest.mark.parametrize("case", [c for c in MMA_CASES if c[5] >= 8])
def test_attention_decode_tma_merges_in_the_last_block(case, splits):
    """With counters the attention kernel merges its own splits: same numbers as the second kernel's, twice
    in a row (the counters are left at zero)."""
    import functools
    ctx, new, nq, nkv, hd, P, window = case
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", ctx, new, nq, nkv, hd, P, seed=hd + len(ctx),
                                               window=window)
    two = _run_split(q, kc, vc, pos, eot, bt, len(ctx), window, hd, splits, fn=_k().attention_decode_tma)
    counters = torch.zeros(q.shape[0] * nq, dtype=torch.int32, device="cuda")
    own0 = _k().counters.own
    for _ in range(2):
        one = _run_split(q, kc, vc, pos, eot, bt, len(ctx), window, hd, splits,
                         fn=functools.partial(_k().attention_decode_tma, merge_counters=counters))
        assert _rel(one, ref) <= 1.5e-2
        assert _rel(one, two.double()) <= 1e-2   # the merge's arithmetic differs only in its rounding
        assert int(counters.abs().sum().item()) == 0
    assert _k().counters.own - own0 == 2  # one launch each


FUSED_CASES = [
    # cached tokens per row (the new token's position), nq, nkv, hd, page, window, entries that are padding
    ([0, 1, 15, 16, 63, 64, 65, 700], 32, 8, 128, 16, None, ()),
    ([5, 127, 128, 300], 8, 8, 64, 8, None, (2,)),          # groups of one head, page 8, a padded row
    ([511, 512, 40], 16, 2, 128, 32, None, ()),             # groups of 8
    ([200, 64, 0], 40, 2, 128, 64, 70, ()),                 # groups of 20 (two head chunks), a window
    ([90, 31], 6, 3, 64, 16, 50, ()),
]


@pytest.mark.parametrize("splits", [1, 3, 16])
@pytest.mark.parametrize("plain_keys", [False, True])
@pytest.mark.parametrize("case", FUSED_CASES)
def test_attention_decode_tma_fused(case, splits, plain_keys):
    """The decode attention fed with the rows of the q|k|v product does what qk_norm_rope_kv_write followed
    by the attention does: same output, same key and value in the same place of the cache, nothing else
    touched.  plain_keys: without norm weights and rotation."""
    k = _k()
    ctx, nq, nkv, hd, P, window, padding = case
    B = len(ctx)
    g = torch.Generator().manual_seed(hd + B + splits)
    pages_per = [c // P + 1 for c in ctx]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=g)
    stride = max(pages_per)
    bt = torch.full((B, stride), -1, dtype=torch.int32)
    at = 0
    for b in range(B):
        bt[b, :pages_per[b]] = perm[at:at + pages_per[b]].to(torch.int32)
        at += pages_per[b]
    kc0 = (torch.randn((num_pages, nkv, P, hd), generator=g) * 0.7).bfloat16().cuda()
    vc0 = torch.randn((num_pages, nkv, P, hd), generator=g).bfloat16().cuda()
    qkv = torch.randn((B, (nq + 2 * nkv) * hd), generator=g).bfloat16().cuda()
    qw = None if plain_keys else (1 + 0.1 * torch.randn(hd, generator=g)).cuda()
    kw = None if plain_keys else (1 + 0.1 * torch.randn(hd, generator=g)).cuda()
    inv_freq = None if plain_keys else plain.rope_inv_freq(hd, 1e6).float().cuda()
    eps = 1e-6
    pos = torch.tensor(ctx, dtype=torch.int32)
    eot = torch.arange(B, dtype=torch.int32)
    slots = torch.tensor([int(bt[b, ctx[b] // P]) * P + ctx[b] % P for b in range(B)], dtype=torch.int32)
    for b in padding:
        eot[b] = -1
        slots[b] = -1
    pos, eot, slots, btd = pos.cuda(), eot.cuda(), slots.cuda(), bt.cuda()
    scale = 1 / math.sqrt(hd)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    acc = torch.empty(B * nq * splits * hd, dtype=torch.float32, device="cuda")
    ml = torch.empty(B * nq * splits * 2, dtype=torch.float32, device="cuda")
    # two kernels
    kc2, vc2 = kc0.clone(), vc0.clone()
    q = torch.zeros((B, nq, hd), dtype=torch.bfloat16, device="cuda")
    k.qk_norm_rope_kv_write(qkv, q, kc2, vc2, pos, slots, inv_freq, qw, kw, eps, nq, nkv, hd, P, status)
    want = torch.zeros_like(q)
    k.attention_decode_tma(q, kc2, vc2, want, acc, ml, pos, eot, btd, B, 0, B, window or 0, scale, splits, status)
    # one kernel
    kc1, vc1 = kc0.clone(), vc0.clone()
    got = torch.zeros_like(q)
    counters = torch.zeros(B * nq, dtype=torch.int32, device="cuda")
    k.attention_decode_tma_fused(qkv, kc1, vc1, got, acc, ml, pos, eot, btd, B, 0, B, nq, window or 0, scale, splits,
                                 qw, kw, eps, inv_freq, status=status,
                                 merge_counters=counters if splits == 16 else None)
    assert int(status.item()) == 0 and int(counters.abs().sum().item()) == 0
    live = [b for b in range(B) if b not in padding]
    assert _rel(got[live], want[live].double().cpu()) <= 1e-2
    # and what the plain functions make of the same rows: norm, rotation, the cached keys of the request's
    # pages followed by the new one, causal (windowed) attention of the last position
    for b in live:
        L = ctx[b] + 1
        row = qkv[b].double().cpu()
        qn = row[:nq * hd].view(1, nq, hd)
        kn = row[nq * hd:(nq + nkv) * hd].view(1, nkv, hd)
        vn = row[(nq + nkv) * hd:].view(1, nkv, hd)
        if not plain_keys:
            here = torch.tensor([ctx[b]])
            qn = plain.apply_rope(plain.rms_norm(qn, qw.double().cpu(), eps), here, inv_freq.cpu())
            kn = plain.apply_rope(plain.rms_norm(kn, kw.double().cpu(), eps), here, inv_freq.cpu())
        pages = bt[b, :L // P + 1].long()
        k_old = kc0.double().cpu()[pages].permute(0, 2, 1, 3).reshape(-1, nkv, hd)[:ctx[b]]
        v_old = vc0.double().cpu()[pages].permute(0, 2, 1, 3).reshape(-1, nkv, hd)[:ctx[b]]
        q_all = torch.zeros((L, nq, hd), dtype=torch.float64)
        q_all[-1] = qn[0]
        ref = plain.causal_attention(q_all, torch.cat([k_old, kn]), torch.cat([v_old, vn]), window)[-1]
        assert _rel(got[b], ref) <= 1.5e-2, b
    assert float(got[list(padding)].abs().max()) == 0 if padding else True
    assert torch.equal(vc1, vc2)                                  # values are copied
    assert _rel(kc1, kc2.double().cpu()) <= 8e-3                   # keys: the same up to the rounding of the norm
    changed = (kc1 != kc0).any(dim=-1)
    assert int(changed.sum().item()) <= len(live) * nkv           # only the new tokens' rows
    # a layer that reads another layer's cache: queries only, the position is already there
    got2 = torch.zeros_like(q)
    k.attention_decode_tma_fused(qkv, kc2, vc2, got2, acc, ml, pos, eot, btd, B, 0, B, nq, window or 0, scale,
                                 splits, qw, None, eps, inv_freq, write_kv=False, status=status)
    assert int(status.item()) == 0
    assert _rel(got2[live], want[live].double().cpu()) <= 1e-2


@pytest.mark.parametrize("far_key", [0, 15, 16, 63, 64, 255, 256, 257, 511, 598])
def test_attention_decode_tma_reads_far_key(far_key):
    nq, nkv, hd, P = 8, 2, 128, 16
    L = 600
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", [L - 1], [1], nq, nkv, hd, P, seed=far_key,
                                               peak=(0, far_key))
    for splits in (1, 5):
        out = _run_split(q, kc, vc, pos, eot, bt, 1, None, hd, splits, fn=_k().attention_decode_tma)
        assert _rel(out, ref) <= 1.5e-2


@pytest.mark.parametrize("edge", [-1, 0, 1])
def test_attention_decode_tma_window_edge(edge):
    nq, nkv, hd, P, W = 4, 1, 64, 8, 40
    L = 200
    key = (L - 1) - W + 1 + edge
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", [L - 1], [1], nq, nkv, hd, P, seed=7, window=W,
                                               peak=(0, key))
    for splits in (1, 4):
        out = _run_split(q, kc, vc, pos, eot, bt, 1, W, hd, splits, fn=_k().attention_decode_tma)
        assert _rel(out, ref) <= 1.5e-2


def test_attention_decode_tma_padding_rows():
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", [40, 9], [1, 1], 4, 2, 64, 16, seed=3)
    eot2 = eot.clone()
    eot2[1] = -1
    out = _run_split(q, kc, vc, pos, eot2, bt, 2, None, 64, 4, fn=_k().attention_decode_tma)
    assert float(out[1].abs().max()) == 0.0 and _rel(out[:1], ref[:1]) <= 1.5e-2


@pytest.mark.parametrize("far_key", [0, 15, 16, 63, 64, 255, 256, 257, 511, 598])
def test_attention_decode_mma_reads_far_key(far_key):
    nq, nkv, hd, P = 8, 2, 128, 16
    L = 600
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", [L - 1], [1], nq, nkv, hd, P, seed=far_key,
                                               peak=(0, far_key))
    for splits in (1, 5):
        out = _run_split(q, kc, vc, pos, eot, bt, 1, None, hd, splits, fn=_k().attention_decode_mma)
        assert _rel(out, ref) <= 1.5e-2


@pytest.mark.parametrize("edge", [-1, 0, 1])
def test_attention_decode_mma_window_edge(edge):
    nq, nkv, hd, P, W = 4, 1, 64, 8, 40
    L = 200
    key = (L - 1) - W + 1 + edge
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", [L - 1], [1], nq, nkv, hd, P, seed=7, window=W,
                                               peak=(0, key))
    for splits in (1, 4):
        out = _run_split(q, kc, vc, pos, eot, bt, 1, W, hd, splits, fn=_k().attention_decode_mma)
        assert _rel(out, ref) <= 1.5e-2


@pytest.mark.parametrize("kernel", ["split", "decode_mma", "decode_tma", "prefill_mma", "prefill_tc"])
def test_attention_reports_a_missing_page_with_a_visible_key(kernel):
    """A block-table entry of -1 where a query reads keys: the status word says so (the TMA kernels stand a
    page that certainly exists in for pages that a tile reaches but no query reads, never for a needed one).
    The same entry behind a window is no fault and changes nothing."""
    k = _k()
    nq, nkv, hd, P, W = 4, 2, 128, 16, 100
    prefill = kernel.startswith("prefill")
    ctx, new = ([300], [70]) if prefill else ([299], [1])

    def run(window, dead_page):
        q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", ctx, new, nq, nkv, hd, P, seed=3, window=window)
        bt = bt.clone()
        bt[0, dead_page] = -1
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = torch.zeros_like(q)
        scale = 1 / math.sqrt(hd)
        if prefill:
            cu = torch.tensor([0, new[0]], dtype=torch.int32, device="cuda")
            pos0 = torch.tensor(ctx, dtype=torch.int32, device="cuda")
            getattr(k, "attention_" + kernel)(q, kc, vc, out, cu, pos0, bt, 0, 1, new[0], window or 0, scale, status)
        else:
            acc = torch.empty(nq * 4 * hd, dtype=torch.float32, device="cuda")
            ml = torch.empty(nq * 4 * 2, dtype=torch.float32, device="cuda")
            getattr(k, "attention_" + kernel)(q, kc, vc, out, acc, ml, pos, eot, bt, 1, 0, 1, window or 0, scale, 4,
                                              status)
        return int(status.item()), out, ref

    word, _, _ = run(None, 3)             # keys 48..63 are read by every query
    assert word == k.ST_BAD_PAGE
    word, _, _ = run(W, 18)               # inside the window of the last queries
    assert word == k.ST_BAD_PAGE
    word, out, ref = run(W, 3)            # long before the window of the first query (position 300 - 99 = 201)
    assert word == 0
    assert _rel(out, ref) <= 1.5e-2


PREFILL_CASES = [
    # ctx, new, nq, nkv, hd, page, window
    ([0], [1], 2, 1, 64, 16, None),
    ([0], [64], 4, 2, 128, 16, None),
    ([0, 5, 31], [70, 2, 130], 6, 3, 64, 8, None),
    ([100, 0, 63], [1, 200, 65], 8, 2, 128, 16, None),
    ([0, 40, 129], [150, 3, 64], 4, 4, 64, 4, 24),
    ([17, 250], [300, 1], 5, 1, 128, 32, 100),
]


@pytest.mark.parametrize("case", PREFILL_CASES)
def test_attention_prefill_mma(case):
    ctx, new, nq, nkv, hd, P, window = case
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", ctx, new, nq, nkv, hd, P, seed=hd + len(ctx),
                                               window=window)
    cu = torch.tensor([0] + list(np.cumsum(new)), dtype=torch.int32, device="cuda")
    pos0 = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q)
    _k().attention_prefill_mma(q, kc, vc, out, cu, pos0, bt, 0, len(ctx), max(new), window or 0,
                               1 / math.sqrt(hd), status)
    assert int(status.item()) == 0
    assert _rel(out, ref) <= 1.5e-2
    if len(ctx) > 1:  # only the requests from the second on: the first one's rows stay untouched
        part = torch.zeros_like(q)
        _k().attention_prefill_mma(q, kc, vc, part, cu, pos0, bt, 1, len(ctx) - 1, max(new[1:]), window or 0,
                                   1 / math.sqrt(hd), status)
        assert torch.equal(part[new[0]:], out[new[0]:]) and float(part[:new[0]].abs().max()) == 0.0


TC_PREFILL_CASES = [
    # ctx, new, nq, nkv, hd, page, window
    ([0], [1], 2, 1, 64, 16, None),
    ([0], [128], 4, 2, 128, 16, None),
    ([0, 5, 31], [70, 2, 130], 6, 3, 64, 8, None),
    ([100, 0, 63], [1, 300, 65], 8, 2, 128, 16, None),
    ([0, 40, 129], [150, 3, 64], 4, 4, 64, 32, 24),
    ([17, 250], [300, 1], 5, 1, 128, 128, 100),
    ([1000], [200], 8, 2, 128, 64, None),
    ([0, 700], [700, 260], 32, 8, 128, 16, None),     # the 8B head layout, several query tiles, many key tiles
    ([130], [400], 16, 2, 64, 16, 200),               # groups of 8, head size 64, a window across tiles
]


@pytest.fixture(params=["two heads a block where the group is even", "one head a block"])
def tc_prefill_form(request):
    single = request.param == "one head a block"
    _k().attention_prefill_tc_single_head(single)
    yield request.param
    _k().attention_prefill_tc_single_head(False)


@pytest.mark.parametrize("case", TC_PREFILL_CASES)
def test_attention_prefill_tc(case, tc_prefill_form):
    ctx, new, nq, nkv, hd, P, window = case
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", ctx, new, nq, nkv, hd, P, seed=hd + len(ctx),
                                               window=window)
    cu = torch.tensor([0] + list(np.cumsum(new)), dtype=torch.int32, device="cuda")
    pos0 = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q)
    _k().attention_prefill_tc(q, kc, vc, out, cu, pos0, bt, 0, len(ctx), max(new), window or 0, 1 / math.sqrt(hd),
                              status)
    assert int(status.item()) == 0
    assert _rel(out, ref) <= 1.5e-2
    if len(ctx) > 1:
        part = torch.zeros_like(q)
        _k().attention_prefill_tc(q, kc, vc, part, cu, pos0, bt, 1, len(ctx) - 1, max(new[1:]), window or 0,
                                  1 / math.sqrt(hd), status)
        assert torch.equal(part[new[0]:], out[new[0]:]) and float(part[:new[0]].abs().max()) == 0.0


@pytest.mark.parametrize("far_key", [0, 63, 64, 127, 128, 400, 449])
def test_attention_prefill_tc_reads_far_key(far_key, tc_prefill_form):
    nq, nkv, hd, P = 4, 2, 128, 16
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", [450], [150], nq, nkv, hd, P, seed=far_key,
                                               peak=(0, far_key))
    cu = torch.tensor([0, 150], dtype=torch.int32, device="cuda")
    pos0 = torch.tensor([450], dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _k().attention_prefill_tc(q, kc, vc, out, cu, pos0, bt, 0, 1, 150, 0, 1 / math.sqrt(hd), status)
    assert int(status.item()) == 0
    assert _rel(out, ref) <= 1.5e-2 and _rel(out[-1:], ref[-1:]) <= 1.5e-2


@pytest.mark.parametrize("edge", [-1, 0, 1])
def test_attention_prefill_tc_window_edge(edge, tc_prefill_form):
    nq, nkv, hd, P, W = 2, 1, 64, 8, 40
    ctx, new = 130, 70
    L = ctx + new
    key = (L - 1) - W + 1 + edge
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", [ctx], [new], nq, nkv, hd, P, seed=7, window=W,
                                               peak=(0, key))
    cu = torch.tensor([0, new], dtype=torch.int32, device="cuda")
    pos0 = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q)
    _k().attention_prefill_tc(q, kc, vc, out, cu, pos0, bt, 0, 1, new, W, 1 / math.sqrt(hd))
    assert _rel(out, ref) <= 1.5e-2 and _rel(out[-1:], ref[-1:]) <= 1.5e-2


def test_attention_prefill_tc_refuses_small_pages():
    from ccinfer_b200.errors import Unsupported
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", [0], [20], 2, 1, 64, 4, seed=1)
    cu = torch.tensor([0, 20], dtype=torch.int32, device="cuda")
    pos0 = torch.tensor([0], dtype=torch.int32, device="cuda")
    assert not _k().attention_prefill_tc_fits(64, 4) and _k().attention_prefill_tc_fits(128, 16)
    with pytest.raises(Unsupported):
        _k().attention_prefill_tc(q, kc, vc, torch.zeros_like(q), cu, pos0, bt, 0, 1, 20, 0, 0.125)


@pytest.mark.parametrize("far_key", [0, 63, 64, 127, 128, 400, 449])
def test_attention_prefill_mma_reads_far_key(far_key):
    nq, nkv, hd, P = 4, 2, 128, 16
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", [450], [150], nq, nkv, hd, P, seed=far_key,
                                               peak=(0, far_key))
    cu = torch.tensor([0, 150], dtype=torch.int32, device="cuda")
    pos0 = torch.tensor([450], dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q)
    _k().attention_prefill_mma(q, kc, vc, out, cu, pos0, bt, 0, 1, 150, 0, 1 / math.sqrt(hd))
    assert _rel(out, ref) <= 1.5e-2
    assert _rel(out[-1:], ref[-1:]) <= 1.5e-2  # the row whose score stands out


@pytest.mark.parametrize("edge", [-1, 0, 1])
def test_attention_prefill_mma_window_edge(edge):
    nq, nkv, hd, P, W = 2, 1, 64, 8, 40
    ctx, new = 130, 70
    L = ctx + new
    key = (L - 1) - W + 1 + edge
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", [ctx], [new], nq, nkv, hd, P, seed=7, window=W,
                                               peak=(0, key))
    cu = torch.tensor([0, new], dtype=torch.int32, device="cuda")
    pos0 = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q)
    _k().attention_prefill_mma(q, kc, vc, out, cu, pos0, bt, 0, 1, new, W, 1 / math.sqrt(hd))
    assert _rel(out, ref) <= 1.5e-2 and _rel(out[-1:], ref[-1:]) <= 1.5e-2


def test_attention_decode_mma_refuses_other_head_sizes():
    from ccinfer_b200.errors import Unsupported
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", [10], [1], 2, 1, 48, 16, seed=1)
    with pytest.raises(Unsupported):
        _run_split(q, kc, vc, pos, eot, bt, 1, None, 48, 1, fn=_k().attention_decode_mma)


def test_attention_split_padding_rows():
    """Rows that belong to no request (padding of a replayed decode step) come out as zeros."""
    q, kc, vc, pos, eot, bt, ref = _paged_case("bfloat16", [40, 9], [1, 1], 4, 2, 64, 16, seed=3)
    eot2 = eot.clone()
    eot2[1] = -1
    out = _run_split(q, kc, vc, pos, eot2, bt, 2, None, 64, 4)
    assert float(out[1].abs().max()) == 0.0 and _rel(out[:1], ref[:1]) <= 1.5e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far_key", [0, 15, 16, 255, 256, 257, 511])
def test_attention_reads_far_key(dtype, far_key):
    """One key among hundreds carries the whole output: its value must come through."""
    nq, nkv, hd, P = 4, 2, 64, 16
    L = 600
    q, kc, vc, pos, eot, bt, ref = _paged_case(dtype, [L - 1], [1], nq, nkv, hd, P, seed=far_key,
                                               peak=(0, far_key))
    out = torch.empty_like(q)
    _k().paged_attention_generic(q, kc, vc, out, pos, eot, bt, 1, 0, 1 / math.sqrt(hd))
    assert _rel(out, ref) <= (1e-5 if dtype == "float32" else 1.5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("edge", [-1, 0, 1])
def test_attention_window_edge(dtype, edge):
    """The strongest key sits just outside, on, and just inside the window's edge."""
    nq, nkv, hd, P, W = 2, 1, 32, 8, 40
    L = 200
    key = (L - 1) - W + 1 + edge  # edge -1: the first key that is no longer seen
    q, kc, vc, pos, eot, bt, ref = _paged_case(dtype, [L - 1], [1], nq, nkv, hd, P, seed=7, window=W,
                                               peak=(0, key))
    out = torch.empty_like(q)
    _k().paged_attention_generic(q, kc, vc, out, pos, eot, bt, 1, W, 1 / math.sqrt(hd))
    assert _rel(out, ref) <= (1e-5 if dtype == "float32" else 1.5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [11, 150])   # many tokens: the 16-byte variant of the bfloat16 kernel
@pytest.mark.parametrize("nq,nkv,hd,P,theta", [(4, 2, 16, 4, 1e4), (6, 3, 48, 8, 5e4), (8, 2, 128, 16, 1e6),
                                                 (3, 1, 256, 16, 1e6), (5, 5, 64, 8, 1e4), (9, 3, 32, 16, 1e6),
                                                 (32, 8, 128, 16, 1e6)])
def test_qk_norm_rope_kv_write(dtype, nq, nkv, hd, P, theta, T):
    k = _k()
    eps = 1e-6
    pages = max(9, T // P + 3)
    qkv, ref = _rand((T, (nq + 2 * nkv) * hd), DT[dtype], 12)
    qw, qw_ref = _rand((hd,), torch.float32, 13)
    kw, kw_ref = _rand((hd,), torch.float32, 14)
    qw, kw, qw_ref, kw_ref = qw + 1, kw + 1, qw_ref + 1, kw_ref + 1
    positions = torch.tensor([0, 1, 2, 3, 900, 901, 17, 4000, 5, 6, 7], dtype=torch.int32)
    if T > 11:
        more = torch.randint(0, 5000, (T - 11,), generator=torch.Generator().manual_seed(16), dtype=torch.int32)
        positions = torch.cat([positions, more])
    slots = torch.randperm(pages * P, generator=torch.Generator().manual_seed(15))[:T].to(torch.int32)
    slots[3] = -1  # a padded row: nothing is cached for it
    inv_freq = plain.rope_inv_freq(hd, theta)
    q_out = torch.empty((T, nq, hd), dtype=DT[dtype], device="cuda")
    kc = torch.zeros((pages, nkv, P, hd), dtype=DT[dtype], device="cuda")
    vc = torch.zeros_like(kc)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.qk_norm_rope_kv_write(qkv, q_out, kc, vc, positions.cuda(), slots.cuda(), inv_freq.cuda(), qw, kw, eps,
                            nq, nkv, hd, P, status)
    assert int(status.item()) == 0
    q_ref = ref[:, :nq * hd].view(T, nq, hd)
    k_ref = ref[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd)
    v_ref = ref[:, (nq + nkv) * hd:].view(T, nkv, hd)
    q_ref = plain.apply_rope(plain.rms_norm(q_ref, qw_ref, eps), positions, inv_freq)
    k_ref = plain.apply_rope(plain.rms_norm(k_ref, kw_ref, eps), positions, inv_freq)
    tol = 2e-6 if dtype == "float32" else 1.2e-2
    assert _rel(q_out, q_ref) <= tol
    kc_h, vc_h = kc.cpu().double(), vc.cpu().double()
    written = torch.zeros(pages * P, dtype=torch.bool)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        written[s] = True
        assert float((kc_h[s // P, :, s % P] - k_ref[t]).abs().max()) <= tol * float(k_ref.abs().max())
        assert float((vc_h[s // P, :, s % P] - v_ref[t]).abs().max()) == 0.0  # v is copied as it is
    untouched = ~written
    assert float(kc_h.transpose(1, 2).reshape(pages * P, -1)[untouched].abs().max()) == 0.0


@pytest.mark.parametrize("V", [11, 500, 151936])
def test_sampling(V):
    k = _k()
    R = 5
    g = torch.Generator().manual_seed(16)
    logits = torch.randn((R, V), generator=g)
    logits[1, V // 2] = logits[1].max() + 1  # a clear winner
    logits[2, 3] = logits[2, V - 1] = logits[2].max() + 2  # a tie: the lowest id wins
    tokens = torch.zeros(R, dtype=torch.int32, device="cuda")
    k.sample_rows(logits.cuda(), tokens)
    want = [plain.greedy(logits[r]) for r in range(R)]
    assert tokens.tolist() == want and want[2] == 3
    temps = torch.tensor([0.0, 0.8, 1.5, 0.3, 1.0])
    seeds = torch.tensor([7, 7, 42, 123456789, -5], dtype=torch.int32)
    idx = torch.tensor([0, 3, 1, 250, 9], dtype=torch.int32)
    k.sample_rows(logits.cuda(), tokens, temps.cuda(), seeds.cuda(), idx.cuda())
    want = [plain.sample_temperature(logits[r], float(temps[r]), int(seeds[r]) & 0xFFFFFFFF, int(idx[r]))
            for r in range(R)]
    assert tokens.tolist() == want


@pytest.mark.parametrize("V", [97, 5000, 151936])
def test_sampling_top_k_top_p(V):
    """The draw restricted to the k largest logits and to the top-p share: the same token as the plain
    sort-based rule, never a token outside the allowed set, ties at the k-th logit kept."""
    k = _k()
    R = 12
    g = torch.Generator().manual_seed(21)
    logits = torch.randn((R, V), generator=g) * 2.0
    logits[3, 5] = logits[3, 11] = torch.sort(logits[3], descending=True).values[3]   # a tie at the 4th place
    temps = torch.tensor([0.7, 1.0, 1.3, 0.9, 0.0, 2.0, 0.5, 1.0, 1.0, 0.8, 1.1, 3.0])
    top_k = torch.tensor([1, 5, 0, 4, 3, 50, 0, V, 7, 2, 0, 40], dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 0.9, 1.0, 0.5, 0.8, 0.3, 0.95, 0.6, 1.0, 0.999, 0.05])
    seeds = torch.arange(R, dtype=torch.int32) * 77 + 5
    idx = torch.arange(R, dtype=torch.int32) * 3
    tokens = torch.zeros(R, dtype=torch.int32, device="cuda")
    k.sample_rows(logits.cuda(), tokens, temps.cuda(), seeds.cuda(), idx.cuda(), top_k=top_k.cuda(), top_p=top_p.cuda())
    got = tokens.tolist()
    checked = 0
    for r in range(R):
        want, margin = plain.sample_filtered(logits[r], float(temps[r]), int(seeds[r]), int(idx[r]), int(top_k[r]),
                                             float(top_p[r]))
        # With a large vocabulary the float sums may move the top-p cut by a few tokens of probability
        # 1e-6 each (margin: how close the plain rule's cut is to top_p); such a token is practically
        # never the winner, so the draw is the same unless the cut sits on a rounding edge.
        assert got[r] == want or margin < 1e-5, (r, margin)
        checked += got[r] == want
    assert checked >= R - 1
    assert got[0] == plain.greedy(logits[0])   # top_k = 1 is the argmax whatever the noise
    assert got[4] == plain.greedy(logits[4])   # temperature 0: greedy, the filters do not apply
    # many draws never leave the allowed set
    n = 400
    row = logits[1:2].expand(n, V).contiguous().cuda()
    toks = torch.zeros(n, dtype=torch.int32, device="cuda")
    k.sample_rows(row, toks, torch.full((n,), 1.5, device="cuda"), torch.full((n,), 3, dtype=torch.int32, device="cuda"),
                  torch.arange(n, dtype=torch.int32, device="cuda"), top_k=torch.full((n,), 5, dtype=torch.int32, device="cuda"),
                  top_p=torch.full((n,), 1.0, device="cuda"))
    top5 = set(torch.topk(logits[1], 5).indices.tolist())
    seen = set(toks.tolist())
    assert seen <= top5 and len(seen) >= 3


def test_sampling_distribution():
    """Temperature draws follow softmax(logits / T): chi-square over a 12-symbol vocabulary."""
    k = _k()
    V, n, T = 12, 20000, 0.7
    logits = torch.linspace(-1.5, 1.5, V)
    p = torch.softmax(logits.double() / T, dim=0).numpy()
    rows = logits[None, :].expand(n, V).contiguous().cuda()
    tokens = torch.zeros(n, dtype=torch.int32, device="cuda")
    temps = torch.full((n,), T, device="cuda")
    seeds = torch.full((n,), 99, dtype=torch.int32, device="cuda")
    idx = torch.arange(n, dtype=torch.int32, device="cuda")
    k.sample_rows(rows, tokens, temps, seeds, idx)
    counts = np.bincount(tokens.cpu().numpy(), minlength=V)
    chi2 = float(((counts - n * p) ** 2 / (n * p)).sum())
    assert chi2 < 40.0, chi2  # 11 degrees of freedom: 40 is far in the tail (p < 1e-4)
