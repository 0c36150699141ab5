"""The entry point that allocates nothing, called through its exported C symbol.

For users who cannot call cudaMalloc when they need attention (all device memory already handed to their
own pools, a decode loop in which a synchronising allocation is forbidden, a plug-in under a host
framework's allocator lock): ccb_attention_split_noalloc keeps the kernel's scratch in a fixed array of the
library.  Its output must equal that of ccb_attention_split with caller-owned scratch, on two calls in a
row (the array keeps the first call's contents), and sizes beyond the array must be refused.

This file is collected last, so a run that stops at the first failure has already run every other test.
"""
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 512 * 1024
REFUSE_TOO_LARGE = -5


def _symbol():
    from ccinfer_b200 import kernels
    fn = kernels.lib().ccb_attention_split_noalloc
    fn.argtypes = [c_void_p] * 7 + [c_int] * 10 + [c_float, c_int, c_int, c_void_p, c_void_p]
    fn.restype = c_int
    return fn


def _case(dtype, seed, B=3, ctx=(150, 40, 9), nq=8, nkv=2, hd=64, P=16):
    g = torch.Generator().manual_seed(seed)
    pages = sum(-(-(c + 1) // P) for c in ctx) + 2
    kc = torch.randn((pages, nkv, P, hd), generator=g).to(dtype).cuda()
    vc = torch.randn((pages, nkv, P, hd), generator=g).to(dtype).cuda()
    q = torch.randn((B, nq, hd), generator=g).to(dtype).cuda()
    perm = torch.randperm(pages, generator=g).tolist()
    stride = max(-(-(c + 1) // P) for c in ctx)
    bt = torch.full((B, stride), -1, dtype=torch.int32)
    for b, c in enumerate(ctx):
        for lp in range(-(-(c + 1) // P)):
            bt[b, lp] = perm.pop()
    pos = torch.tensor(list(ctx), dtype=torch.int32).cuda()
    eot = torch.arange(B, dtype=torch.int32).cuda()
    return q, kc, vc, pos, eot, bt.cuda()


def _plain_attention(q, kc, vc, pos, bt):
    """softmax(q k^T / sqrt(hd)) v in float64 for one query per request over its pages' first pos + 1 keys."""
    B, nq, hd = q.shape
    nkv, P = kc.shape[1], kc.shape[2]
    out = torch.zeros((B, nq, hd), dtype=torch.float64)
    for b in range(B):
        L = int(pos[b]) + 1
        pages = bt[b, :-(-L // P)].long().cpu()
        k = kc.double().cpu()[pages].permute(0, 2, 1, 3).reshape(-1, nkv, hd)[:L]
        v = vc.double().cpu()[pages].permute(0, 2, 1, 3).reshape(-1, nkv, hd)[:L]
        for h in range(nq):
            kh = h // (nq // nkv)
            p = torch.softmax((k[:, kh] @ q[b, h].double().cpu()) / math.sqrt(hd), dim=0)
            out[b, h] = p @ v[:, kh]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_entry_point_matches_the_allocating_one(dtype):
    from ccinfer_b200 import kernels
    fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for call, (seed, splits) in enumerate([(1, 5), (2, 3)]):  # two calls in a row share the library's array
        q, kc, vc, pos, eot, bt = _case(dtype, seed)
        B, nq, hd = q.shape
        pages, nkv, P, _ = kc.shape
        want = torch.zeros_like(q)
        part_acc = torch.empty(B * nq * splits * hd, dtype=torch.float32, device="cuda")
        part_ml = torch.empty(B * nq * splits * 2, dtype=torch.float32, device="cuda")
        kernels.attention_split(q, kc, vc, want, part_acc, part_ml, pos, eot, bt, B, 0, B, 0, 1 / math.sqrt(hd),
                                splits, status)
        got = torch.zeros_like(q)
        rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), got.data_ptr(), pos.data_ptr(), eot.data_ptr(),
                bt.data_ptr(), bt.stride(0), B, 0, B, nq, nkv, hd, P, pages, 0, 1 / math.sqrt(hd), splits,
                kernels._DT[dtype], status.data_ptr(), stream)
        assert rc == 0, f"call {call}: return code {rc}"
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.isfinite(got.float()).all()
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err <= (1e-5 if dtype == torch.float32 else 1.5e-2), f"call {call}: relative error {err}"
        # and both against plain float64 attention of each row over the keys its block table names
        ref = _plain_attention(q, kc, vc, pos, bt)
        err = float((got.double().cpu() - ref).abs().max() / ref.abs().max())
        assert err <= (1e-5 if dtype == torch.float32 else 1.5e-2), f"call {call}: relative error {err} to plain"


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from ccinfer_b200 import kernels
    fn = _symbol()
    q, kc, vc, pos, eot, bt = _case(torch.bfloat16, 3)
    B, nq, hd = q.shape
    pages, nkv, P, _ = kc.shape
    splits = SCRATCH_FLOATS // (B * nq * (hd + 2)) + 1  # one split too many for the array
    out = torch.full_like(q, 7.0)
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), pos.data_ptr(), eot.data_ptr(),
            bt.data_ptr(), bt.stride(0), B, 0, B, nq, nkv, hd, P, pages, 0, 0.125, splits, kernels.BF16, 0,
            torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == REFUSE_TOO_LARGE
    assert float((out.float() - 7.0).abs().max()) == 0.0  # nothing was launched
