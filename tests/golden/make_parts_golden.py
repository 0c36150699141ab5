#!/usr/bin/env python3
"""Makes parts_golden.npz: what 7QiC/ccInfer's own CPU functions compute for the parts of the model.

The reference's kernels run on a GPU only, but its kernel tests carry plain CPU functions of the same
operations, which it compares its kernels with:

  rms_norm_cpu                          tests/kernel/test_rms_norm.cu
  build_rope_cache_cpu, rope_cpu        tests/kernel/test_rope.cu
  silu_mul_cpu                          tests/kernel/test_silu_mul.cu
  naive_attn_cpu                        tests/kernel/test_naive_attn.cu
  decode_reference                      tests/kernel/test_decode_attn.cu

This script takes those function bodies out of a checkout AT RUN TIME (by name, up to the brace that closes
them; nothing of them is kept in this repository), puts a small main() of its own around them, compiles the
whole for the host with nvcc (they use the host side of cuda_bf16.h), feeds them seeded inputs and stores
inputs and outputs.  tests/test_plain.py compares the plain implementation of the tests
(tests/plain_qwen3.py) with the stored file; the script itself is not run by the tests.

    python tests/golden/make_parts_golden.py --reference CHECKOUT

What the file pins: RMSNorm (the weight multiplies directly), the rotate-half pairing and the inverse
frequencies as the reference evaluates them in 32-bit floating point (1.0f / std::pow(theta, float(2 i) /
float(dim))), SiLU * up, causal grouped-query attention with its scale, and attention of one query over
paged keys through a block table.  What it cannot pin: the order of the operations in a layer, which rests
on reading src/model/qwen3/qwen3_model.cpp (that file needs a GPU, boost and real weights to run).
"""
import argparse
import os
import re
import subprocess
import tempfile

import numpy as np

FUNCTIONS = [
    ("tests/kernel/test_rms_norm.cu", "rms_norm_cpu"),
    ("tests/kernel/test_rope.cu", "build_rope_cache_cpu"),
    ("tests/kernel/test_rope.cu", "rope_cpu"),
    ("tests/kernel/test_silu_mul.cu", "silu_mul_cpu"),
    ("tests/kernel/test_naive_attn.cu", "naive_attn_cpu"),
    ("tests/kernel/test_decode_attn.cu", "decode_reference"),
]


def extract_function(path: str, name: str) -> str:
    """The definition of ``name`` in a C++ file: from the line of its return type to its closing brace."""
    with open(path) as f:
        lines = f.read().split("\n")
    start = None
    for i, line in enumerate(lines):
        if re.search(r"\b" + re.escape(name) + r"\s*\(", line) and not line.lstrip().startswith("//") \
                and re.match(r"^(static\s+)?[\w:<>]+[\w:<>\s\*&]*\b" + re.escape(name) + r"\s*\(", line):
            start = i
            break
    if start is None:
        raise SystemExit(f"{path}: no definition of {name}")
    depth, seen, out = 0, False, []
    for line in lines[start:]:
        out.append(line)
        depth += line.count("{") - line.count("}")
        seen = seen or "{" in line
        if seen and depth == 0:
            return "\n".join(out)
    raise SystemExit(f"{path}: {name} does not end")


MAIN = r"""
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

@FUNCTIONS@

static std::vector<float> load(const std::string& dir, const char* name, size_t n) {
  std::vector<float> v(n);
  FILE* f = fopen((dir + "/" + name + ".f32").c_str(), "rb");
  if (!f || fread(v.data(), 4, n, f) != n) { fprintf(stderr, "cannot read %s\n", name); exit(2); }
  fclose(f);
  return v;
}
static std::vector<int32_t> load_i(const std::string& dir, const char* name, size_t n) {
  std::vector<int32_t> v(n);
  FILE* f = fopen((dir + "/" + name + ".i32").c_str(), "rb");
  if (!f || fread(v.data(), 4, n, f) != n) { fprintf(stderr, "cannot read %s\n", name); exit(2); }
  fclose(f);
  return v;
}
static void store(const std::string& dir, const char* name, const std::vector<float>& v) {
  FILE* f = fopen((dir + "/" + name + ".f32").c_str(), "wb");
  fwrite(v.data(), 4, v.size(), f);
  fclose(f);
}
static std::vector<__nv_bfloat16> bf(const std::vector<float>& v) {
  std::vector<__nv_bfloat16> o(v.size());
  for (size_t i = 0; i < v.size(); ++i) o[i] = __float2bfloat16(v[i]);   // the inputs are bfloat16 values already
  return o;
}
static std::vector<float> fl(const std::vector<__nv_bfloat16>& v) {
  std::vector<float> o(v.size());
  for (size_t i = 0; i < v.size(); ++i) o[i] = __bfloat162float(v[i]);
  return o;
}

int main(int argc, char** argv) {
  const std::string dir = argv[1];
  {  // RMSNorm
    const int rows = @NORM_ROWS@, dim = @NORM_DIM@;
    auto x = bf(load(dir, "norm_x", rows * dim)), w = bf(load(dir, "norm_w", dim));
    store(dir, "norm_out", fl(rms_norm_cpu(x.data(), w.data(), rows, dim, @NORM_EPS@f)));
  }
  {  // inverse frequencies as the cache builder evaluates them (cos, sin of position 1 are cos, sin of inv_freq)
     // and the rotation itself
    const int T = @ROPE_T@, nq = @ROPE_NQ@, nkv = @ROPE_NKV@, hd = @ROPE_HD@, maxpos = @ROPE_MAXPOS@;
    auto cache = build_rope_cache_cpu(maxpos, hd, @ROPE_THETA@f);
    auto q = bf(load(dir, "rope_q", (size_t)T * nq * hd)), k = bf(load(dir, "rope_k", (size_t)T * nkv * hd));
    auto pos = load_i(dir, "rope_pos", T);
    rope_cpu(q.data(), k.data(), pos.data(), cache.data(), T, nq, nkv, hd, hd, maxpos);
    store(dir, "rope_q_out", fl(q));
    store(dir, "rope_k_out", fl(k));
  }
  {  // the frequencies alone, for several (theta, dim).  The cache builder keeps only cos and sin of
     // position * inv_freq, so the line that computes inv_freq is restated here, and checked: at position 1
     // the builder's own cos and sin must be those of the restated value, bit for bit.
    const float thetas[] = {10000.0f, 50000.0f, 1000000.0f};
    const int dims[] = {16, 32, 48, 64, 128};
    std::vector<float> out;
    for (float th : thetas)
      for (int d : dims) {
        auto c = build_rope_cache_cpu(2, d, th);
        for (int i = 0; i < d / 2; ++i) {
          const float inv_freq = 1.0f / std::pow(th, static_cast<float>(2 * i) / static_cast<float>(d));
          const float angle = 1.0f * inv_freq;
          if (std::cos(angle) != c[d / 2 + i].x || std::sin(angle) != c[d / 2 + i].y) {
            fprintf(stderr, "the restated inverse frequency differs from the builder's at theta %g dim %d pair %d\n",
                    th, d, i);
            return 3;
          }
          out.push_back(inv_freq);
        }
      }
    store(dir, "inv_freq", out);
  }
  {  // SiLU * up
    const int n = @SILU_N@;
    auto g = bf(load(dir, "silu_g", n)), u = bf(load(dir, "silu_u", n));
    store(dir, "silu_out", fl(silu_mul_cpu(g.data(), u.data(), n)));
  }
  {  // causal grouped-query attention of a whole sequence
    const int T = @ATT_T@, nq = @ATT_NQ@, nkv = @ATT_NKV@, hd = @ATT_HD@;
    auto q = bf(load(dir, "att_q", (size_t)T * nq * hd)), k = bf(load(dir, "att_k", (size_t)T * nkv * hd)),
         v = bf(load(dir, "att_v", (size_t)T * nkv * hd));
    std::vector<__nv_bfloat16> o((size_t)T * nq * hd);
    naive_attn_cpu(o.data(), q.data(), k.data(), v.data(), T, nq, nkv, hd);
    store(dir, "att_out", fl(o));
  }
  {  // one query per request over paged keys
    const int B = @DEC_B@, nq = @DEC_NQ@, nkv = @DEC_NKV@, hd = @DEC_HD@, P = @DEC_P@, pages = @DEC_PAGES@,
              stride = @DEC_STRIDE@;
    auto q = bf(load(dir, "dec_q", (size_t)B * nq * hd));
    auto kc = bf(load(dir, "dec_k", (size_t)pages * P * nkv * hd)), vc = bf(load(dir, "dec_v", (size_t)pages * P * nkv * hd));
    auto bt = load_i(dir, "dec_bt", (size_t)B * stride), ctx = load_i(dir, "dec_ctx", B);
    store(dir, "dec_out", decode_reference(q, kc, vc, bt, ctx, B, stride, nq, nkv, hd, P));
  }
  return 0;
}
"""


def bf16_values(rng, shape, scale=1.0):
    """Random float32 values that bfloat16 holds exactly."""
    x = (rng.standard_normal(shape) * scale).astype(np.float32)
    return (x.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of 7QiC/ccInfer")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "parts_golden.npz"))
    ap.add_argument("--nvcc", default="nvcc")
    args = ap.parse_args()
    rng = np.random.default_rng(20240607)
    sizes = dict(NORM_ROWS=3, NORM_DIM=80, NORM_EPS="1e-5", ROPE_T=6, ROPE_NQ=4, ROPE_NKV=2, ROPE_HD=32,
                 ROPE_MAXPOS=300, ROPE_THETA="1000000.0", SILU_N=96, ATT_T=11, ATT_NQ=4, ATT_NKV=2, ATT_HD=16,
                 DEC_B=2, DEC_NQ=4, DEC_NKV=2, DEC_HD=16, DEC_P=16, DEC_PAGES=5, DEC_STRIDE=3)
    s = sizes
    inputs = {
        "norm_x": bf16_values(rng, (s["NORM_ROWS"], s["NORM_DIM"]), 2.0),
        "norm_w": bf16_values(rng, (s["NORM_DIM"],), 0.1) + np.float32(1.0),
        "rope_q": bf16_values(rng, (s["ROPE_T"], s["ROPE_NQ"], s["ROPE_HD"])),
        "rope_k": bf16_values(rng, (s["ROPE_T"], s["ROPE_NKV"], s["ROPE_HD"])),
        "rope_pos": np.array([0, 1, 2, 17, 255, 299], dtype=np.int32),
        "silu_g": bf16_values(rng, (s["SILU_N"],), 3.0),
        "silu_u": bf16_values(rng, (s["SILU_N"],)),
        "att_q": bf16_values(rng, (s["ATT_T"], s["ATT_NQ"], s["ATT_HD"])),
        "att_k": bf16_values(rng, (s["ATT_T"], s["ATT_NKV"], s["ATT_HD"])),
        "att_v": bf16_values(rng, (s["ATT_T"], s["ATT_NKV"], s["ATT_HD"])),
        "dec_q": bf16_values(rng, (s["DEC_B"], s["DEC_NQ"], s["DEC_HD"])),
        # the reference's cache layout: [slot = page * P + offset][kv head][head_dim]
        "dec_k": bf16_values(rng, (s["DEC_PAGES"] * s["DEC_P"], s["DEC_NKV"], s["DEC_HD"])),
        "dec_v": bf16_values(rng, (s["DEC_PAGES"] * s["DEC_P"], s["DEC_NKV"], s["DEC_HD"])),
        "dec_bt": np.array([[4, 1, 3], [2, 0, -1]], dtype=np.int32),
        "dec_ctx": np.array([41, 17], dtype=np.int32),
    }
    inputs["norm_w"] = (inputs["norm_w"].view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
    functions = "\n\n".join(extract_function(os.path.join(args.reference, p), n) for p, n in FUNCTIONS)
    src = MAIN.replace("@FUNCTIONS@", functions)
    for k, v in sizes.items():
        src = src.replace(f"@{k}@", str(v))
    outputs = ["norm_out", "rope_q_out", "rope_k_out", "inv_freq", "silu_out", "att_out", "dec_out"]
    with tempfile.TemporaryDirectory() as tmp:
        for name, arr in inputs.items():
            arr.tofile(os.path.join(tmp, name + (".i32" if arr.dtype == np.int32 else ".f32")))
        with open(os.path.join(tmp, "driver.cu"), "w") as f:
            f.write(src)
        subprocess.check_call([args.nvcc, "-std=c++17", "-O1", "-Xcompiler", "-ffp-contract=off",
                               os.path.join(tmp, "driver.cu"), "-o", os.path.join(tmp, "driver")])
        subprocess.check_call([os.path.join(tmp, "driver"), tmp])
        got = {name: np.fromfile(os.path.join(tmp, name + ".f32"), dtype=np.float32) for name in outputs}
    meta = {k: np.array(float(v) if isinstance(v, str) else v) for k, v in sizes.items()}
    np.savez_compressed(args.out, **inputs, **got, **{"size_" + k: v for k, v in meta.items()})
    print(f"wrote {args.out}: {sum(v.size for v in got.values())} output values of {len(FUNCTIONS)} functions")


if __name__ == "__main__":
    main()
