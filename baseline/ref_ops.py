#!/usr/bin/env python3
"""Per-operation timings of 7QiC/ccInfer's own CUDA kernels, compiled unchanged for sm_100a, beside this
package's kernels for the same work at the Qwen3-8B layer shape.  CONTEXT ONLY: it is not the reference arm.

The reference as a whole cannot be built or run here (CMake/C++23 with boost, spdlog and fmt, real bfloat16
checkpoints only), so ``bench.py --impl reference`` stays ``unavailable`` and no end-to-end ratio exists.  Its
kernels, however, need only ``base/result.h`` and the CUDA headers.  This script

  1. compiles ``<checkout>/src/kernel/**/*.cu`` as they are, with a few lines of ``extern "C"`` shims of its own
     around the ``launch_*`` functions of ``src/kernel/cuda_kernels.h``, into ``baseline/_ref/libref_ops.so``
     (``python baseline/ref_ops.py --build``; no GPU needed),
  2. times each operation with CUDA events, caches flushed between launches (``--run``, on a B200), on inputs
     inside what each kernel's launcher accepts (page size 16, head size 128), and
  3. prints a table: the reference's kernel(s) for a piece of a layer, this package's kernel(s) for the same.

Matrix products are cuBLAS in both (``cublasGemmEx``, src/backend/cuda/cuda_backend.cpp:82-108) and are left out.
"""
import argparse
import ctypes
import glob
import math
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
OUT_DIR = os.path.join(ROOT, "baseline", "_ref")
LIB = os.path.join(OUT_DIR, "libref_ops.so")

SHIM = r"""
#include "kernel/cuda_kernels.h"
using namespace ccinfer;
#define API extern "C" __attribute__((visibility("default")))
static int rc(const Result<void>& r) { return r ? 0 : 1 + (int)r.error(); }
API int ref_embed(const void* table, const int* ids, void* out, int T, int D, void* s) {
  return rc(launch_embed((const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out, T, D, (cudaStream_t)s)); }
API int ref_rms_norm(const void* x, const void* w, void* y, int rows, int dim, float eps, void* s) {
  return rc(launch_rms_norm((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rows, dim, eps, (cudaStream_t)s)); }
API int ref_rope(void* q, void* k, const int* pos, const void* cache, int T, int nq, int nkv, int hd, int maxpos, void* s) {
  return rc(launch_rope((__nv_bfloat16*)q, (__nv_bfloat16*)k, pos, (const float2*)cache, T, nq, nkv, hd, hd, maxpos, (cudaStream_t)s)); }
API int ref_silu_mul(const void* g, const void* u, void* o, long long n, void* s) {
  return rc(launch_silu_mul((const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)o, n, (cudaStream_t)s)); }
API int ref_element_add(void* dst, const void* src, long long n, void* s) {
  return rc(launch_element_add((__nv_bfloat16*)dst, (const __nv_bfloat16*)src, n, (cudaStream_t)s)); }
API int ref_split_qkv(const void* qkv, void* q, void* k, void* v, int T, int nq, int nkv, int hd, void* s) {
  return rc(launch_split_qkv((const __nv_bfloat16*)qkv, (__nv_bfloat16*)q, (__nv_bfloat16*)k, (__nv_bfloat16*)v, T, nq, nkv, hd, (cudaStream_t)s)); }
API int ref_write_kv(const void* k, const void* v, void* kc, void* vc, const int* slots, int T, int nkv, int hd, int max_slots, void* s) {
  return rc(launch_write_kv_cache((const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, slots, T, nkv, hd, max_slots, (cudaStream_t)s)); }
API int ref_prefill_attn(const void* q, const void* kc, const void* vc, const int* bt, const int* qsl, const int* ctx, void* o,
                         int B, int T, int stride, int nq, int nkv, int hd, int P, void* s) {
  return rc(launch_prefill_attention((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, bt, qsl, ctx,
                                     (__nv_bfloat16*)o, B, T, stride, nq, nkv, hd, P, (cudaStream_t)s)); }
API int ref_decode_attn(const void* q, const void* kc, const void* vc, const int* bt, const int* ctx, void* o, int B, int stride,
                        int nq, int nkv, int hd, int P, void* s) {
  return rc(launch_decode_attention((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, bt, ctx,
                                    (__nv_bfloat16*)o, B, stride, nq, nkv, hd, P, (cudaStream_t)s)); }
API int ref_greedy(const float* logits, int* tokens, const int* idx, int B, int V, int T, void* s) {
  return rc(launch_greedy_sample(logits, tokens, idx, B, V, T, (cudaStream_t)s)); }
"""


def build(reference: str) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    shim = os.path.join(OUT_DIR, "ref_ops_shim.cu")
    with open(shim, "w") as f:
        f.write(SHIM)
    srcs = sorted(glob.glob(os.path.join(reference, "src", "kernel", "**", "*.cu"), recursive=True))
    cmd = ["nvcc", "-std=c++20", "-Xcompiler", "-std=c++23", "-Xcompiler", "-fPIC", "-O3", "-gencode",
           "arch=compute_100a,code=sm_100a", "-I", os.path.join(reference, "src"), "-shared", "-o", LIB, shim] + srcs
    subprocess.check_call(cmd)
    print(f"built {LIB} from {len(srcs)} kernel files of {reference}, unchanged")
    return LIB


def run() -> int:
    import torch
    from ccinfer_b200 import kernels as k
    lib = ctypes.CDLL(LIB)
    dev = "cuda"
    D, nq, nkv, hd, F, V, P, eps = 4096, 32, 8, 128, 12288, 151936, 16, 1e-6
    bf = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev).to(bf)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rows = []

    def timed(fn, reps=7):
        ts = []
        for i in range(reps + 2):
            flush.zero_()   # 256 MB: what the last launch left in L2 is gone
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 2:
                ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    def check(code, what):
        if code != 0:
            raise RuntimeError(f"{what}: the reference's launcher returned error {code - 1}")

    def add(what, ref_us, ours_us, note=""):
        rows.append((what, ref_us, ours_us, note))
        print(f"| {what} | {ref_us:.1f} | {ours_us:.1f} | {ref_us / ours_us:.1f}x | {note} |", flush=True)

    print("| piece of a layer (Qwen3-8B shape, bf16) | reference kernels, us | this package, us | ratio | what runs |")
    print("|---|---|---|---|---|")
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for T in (8, 2048):
        # residual add + RMSNorm
        x, delta, w = rnd(T, D), rnd(T, D), (1 + 0.02 * torch.randn(D, generator=g, device=dev))
        wb, y = w.to(bf), torch.empty((T, D), dtype=bf, device=dev)
        h32 = x.float().clone()

        def ref_norm():
            check(lib.ref_element_add(p(x), p(delta), ctypes.c_longlong(T * D), stream()), "element_add")
            check(lib.ref_rms_norm(p(x), p(wb), p(y), T, D, ctypes.c_float(eps), stream()), "rms_norm")
        add(f"residual add + RMSNorm, {T} tokens", timed(ref_norm),
            timed(lambda: k.residual_rmsnorm(y, h32, delta, w, eps, status=status)),
            "element_add + rms_norm / residual_rmsnorm (float residual stream)")
        # split q|k|v, head norms, rotation, cache write
        pages = T // P + 2
        qkv = rnd(T, (nq + 2 * nkv) * hd)
        q, kk, vv = (torch.empty((T, n, hd), dtype=bf, device=dev) for n in (nq, nkv, nkv))
        kc_ref, vc_ref = (torch.zeros((pages * P, nkv, hd), dtype=bf, device=dev) for _ in range(2))
        kc, vc = (torch.zeros((pages, nkv, P, hd), dtype=bf, device=dev) for _ in range(2))
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        slots = torch.arange(T, dtype=torch.int32, device=dev)
        inv = torch.from_numpy(__import__("ccinfer_b200.parts.position", fromlist=["x"]).rotary_inv_freq(hd, 1e6)).to(dev)
        ang = pos.float()[:, None] * inv[None, :]
        rope_cache = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()   # float2 [T, hd / 2]
        qw, kw = (1 + 0.02 * torch.randn(hd, generator=g, device=dev) for _ in range(2))
        qwb, kwb = qw.to(bf), kw.to(bf)

        def ref_rope_path():
            check(lib.ref_split_qkv(p(qkv), p(q), p(kk), p(vv), T, nq, nkv, hd, stream()), "split_qkv")
            check(lib.ref_rms_norm(p(q), p(qwb), p(q), T * nq, hd, ctypes.c_float(eps), stream()), "q norm")
            check(lib.ref_rms_norm(p(kk), p(kwb), p(kk), T * nkv, hd, ctypes.c_float(eps), stream()), "k norm")
            check(lib.ref_rope(p(q), p(kk), p(pos), p(rope_cache), T, nq, nkv, hd, T, stream()), "rope")
            check(lib.ref_write_kv(p(kk), p(vv), p(kc_ref), p(vc_ref), p(slots), T, nkv, hd, pages * P, stream()), "write_kv")
        add(f"q/k norm + rotation + cache write, {T} tokens", timed(ref_rope_path),
            timed(lambda: k.qk_norm_rope_kv_write(qkv, q, kc, vc, pos, slots, inv, qw, kw, eps, nq, nkv, hd, P, status)),
            "split_qkv + rms_norm x2 + rope + write_kv_cache / qk_norm_rope_kv_write"
            + (" (in decode steps of up to 48 rows it is part of the attention kernel)" if T == 8 else ""))
        # SiLU * up
        gate, up, act = rnd(T, F), rnd(T, F), torch.empty((T, F), dtype=bf, device=dev)
        gu = torch.cat([gate, up], dim=1).contiguous()
        add(f"SiLU * up, {T} tokens", timed(lambda: check(lib.ref_silu_mul(p(gate), p(up), p(act), ctypes.c_longlong(T * F), stream()), "silu_mul")),
            timed(lambda: k.silu_mul(act, gu, 0)), "silu_mul / silu_mul (in decode steps it is the gate|up product's epilogue)")

    # prefill attention, one prompt of 2,048 tokens
    T = 2048
    pages = T // P
    q = rnd(T, nq, hd)
    kc_ref, vc_ref = rnd(pages * P, nkv, hd), rnd(pages * P, nkv, hd)
    kc = kc_ref.view(pages, P, nkv, hd).permute(0, 2, 1, 3).contiguous()
    vc = vc_ref.view(pages, P, nkv, hd).permute(0, 2, 1, 3).contiguous()
    bt = torch.arange(pages, dtype=torch.int32, device=dev)[None, :].contiguous()
    qsl = torch.tensor([0, T], dtype=torch.int32, device=dev)
    ctx = torch.tensor([T], dtype=torch.int32, device=dev)
    o_ref, o = torch.empty_like(q), torch.empty_like(q)
    cu, pos0 = qsl, torch.zeros(1, dtype=torch.int32, device=dev)
    t_ref = timed(lambda: check(lib.ref_prefill_attn(p(q), p(kc_ref), p(vc_ref), p(bt), p(qsl), p(ctx), p(o_ref), 1, T, pages,
                                                     nq, nkv, hd, P, stream()), "prefill_attention"), reps=3)
    t_own = timed(lambda: k.attention_prefill_tc(q, kc, vc, o, cu, pos0, bt, 0, 1, T, 0, 1 / math.sqrt(hd), status))
    err = float((o.float() - o_ref.float()).abs().max())
    add("prefill attention, 2,048-token prompt", t_ref, t_own, f"prefill_attention / attention_prefill_tc (max difference {err:.3f})")

    # decode attention, one new token per request after 2,048 cached
    for B in (8, 64):
        c = 2048
        per = c // P + 1
        pages = B * per
        kc_ref, vc_ref = rnd(pages * P, nkv, hd), rnd(pages * P, nkv, hd)
        kc = kc_ref.view(pages, P, nkv, hd).permute(0, 2, 1, 3).contiguous()
        vc = vc_ref.view(pages, P, nkv, hd).permute(0, 2, 1, 3).contiguous()
        bt = torch.arange(pages, dtype=torch.int32, device=dev).view(B, per).contiguous()
        q = rnd(B, nq, hd)
        ctx = torch.full((B,), c + 1, dtype=torch.int32, device=dev)
        o_ref, o = torch.empty_like(q), torch.empty_like(q)
        pos = torch.full((B,), c, dtype=torch.int32, device=dev)
        eot = torch.arange(B, dtype=torch.int32, device=dev)
        splits, n_acc, n_ml = k.attention_split_plan(B, nq, nkv, hd, k.DECODE_MMA_HEADS_PER_BLOCK)
        acc, ml = torch.empty(n_acc, device=dev), torch.empty(n_ml, device=dev)
        t_ref = timed(lambda: check(lib.ref_decode_attn(p(q), p(kc_ref), p(vc_ref), p(bt), p(ctx), p(o_ref), B, per, nq, nkv, hd, P,
                                                        stream()), "decode_attention"))
        t_own = timed(lambda: k.attention_decode_tma(q, kc, vc, o, acc, ml, pos, eot, bt, B, 0, B, 0, 1 / math.sqrt(hd), splits, status))
        err = float((o.float() - o_ref.float()).abs().max())
        add(f"decode attention, {B} requests at 2,048 tokens", t_ref, t_own,
            f"decode_attention / attention_decode_tma + merge (max difference {err:.3f})")

    # greedy sampling over the vocabulary
    B = 8
    logits = torch.randn((B, V), generator=g, device=dev)
    toks = torch.empty(B, dtype=torch.int32, device=dev)
    idx = torch.arange(B, dtype=torch.int32, device=dev)
    add("greedy sampling, 8 rows of 151,936 logits",
        timed(lambda: check(lib.ref_greedy(p(logits), p(toks), p(idx), B, V, B, stream()), "greedy_sample")),
        timed(lambda: k.sample_rows(logits, toks)), "greedy_sample / sample_rows")
    assert int(status.item()) == 0
    return 0


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CCINFER_REFERENCE", "/root/reference"))
    ap.add_argument("--build", action="store_true")
    ap.add_argument("--run", action="store_true")
    a = ap.parse_args()
    if a.build:
        build(a.reference)
    if a.run:
        sys.exit(run())
