#!/usr/bin/env python3
"""Makes config_parse.json: what 7QiC/ccInfer's own configuration parser reads from config.json files.

The only model-side code of 7QiC/ccInfer that runs without a GPU is ``ModelConfig::from_json``
(src/model/config.h:41-160, header-only; it needs base/result.h, core/dtype.h and nlohmann/json.hpp).
This script writes a driver of a few lines, compiles it with g++ against a checkout of 7QiC/ccInfer and a
nlohmann/json header, feeds it the cases below and stores for each either the fields it parsed or the
error code it returned.  tests/test_config_weights.py compares the package's parser with the stored file;
the script itself is not run by the tests.

    python tests/golden/make_config_golden.py --reference CHECKOUT --json-include DIR_WITH_nlohmann

Everything else of the model (layers, attention, cache) is CUDA-only in 7QiC/ccInfer, so the plain
implementation in tests/plain_qwen3.py rests on the formulas of its kernels, not on live outputs.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import tiny_configs  # noqa: E402

DRIVER = r"""
#include <cstdio>
#include <fstream>
#include <iostream>
#include "model/config.h"
int main(int argc, char** argv) {
  std::ifstream f(argv[1]);
  nlohmann::json cases = nlohmann::json::parse(f);
  nlohmann::json out = nlohmann::json::object();
  for (auto& [name, j] : cases.items()) {
    auto r = ccinfer::ModelConfig::from_json(j);
    nlohmann::json o;
    if (!r) {
      const auto e = r.error();
      o["error"] = e == ccinfer::ErrorCode::ModelConfigInvalid      ? "ModelConfigInvalid"
                   : e == ccinfer::ErrorCode::ModelUnsupportedArch  ? "ModelUnsupportedArch"
                   : e == ccinfer::ErrorCode::ModelUnsupportedDType ? "ModelUnsupportedDType"
                                                                    : "other";
    } else {
      o["arch"] = r->arch_name();
      o["num_hidden_layers"] = r->n_layers_;
      o["num_attention_heads"] = r->n_q_heads_;
      o["num_key_value_heads"] = r->n_kv_heads_;
      o["hidden_size"] = r->d_model_;
      o["head_dim"] = r->head_dim_;
      o["intermediate_size"] = r->d_ff_;
      o["vocab_size"] = r->vocab_size_;
      o["max_position_embeddings"] = r->max_seq_len_;
      o["rope_theta"] = static_cast<double>(r->rope_theta_);
      o["rms_norm_eps"] = static_cast<double>(r->rms_norm_eps_);
    }
    out[name] = o;
  }
  std::cout << out.dump(1) << std::endl;
  return 0;
}
"""


def cases():
    """name -> config.json contents: the tiny configurations of the tests and variations of the first."""
    out = {f"tiny_{k}": v[0] for k, v in tiny_configs.ALL.items()}
    base = tiny_configs.TINY_A

    def vary(**kw):
        j = dict(base)
        for k, v in kw.items():
            if v is None:
                j.pop(k, None)
            else:
                j[k] = v
        return j

    out["defaults"] = vary(num_key_value_heads=None, head_dim=None, max_position_embeddings=None,
                           rope_theta=None, rms_norm_eps=None, torch_dtype=None)
    out["head_dim_not_hidden_over_heads"] = vary(head_dim=48)
    out["missing_hidden_size"] = vary(hidden_size=None)
    out["missing_vocab_size"] = vary(vocab_size=None)
    out["hidden_size_is_a_string"] = vary(hidden_size="64")
    out["zero_layers"] = vary(num_hidden_layers=0)
    out["heads_not_divisible_by_groups"] = vary(num_attention_heads=6, num_key_value_heads=4)
    out["negative_eps"] = vary(rms_norm_eps=-1e-6)
    out["zero_theta"] = vary(rope_theta=0.0)
    out["unknown_dtype"] = vary(torch_dtype="int8")
    out["unknown_architecture"] = vary(architectures=["LlamaForCausalLM"])
    out["no_architectures"] = vary(architectures=None)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of 7QiC/ccInfer")
    ap.add_argument("--json-include", required=True, help="folder that holds nlohmann/json.hpp")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "config_parse.json"))
    args = ap.parse_args()
    with tempfile.TemporaryDirectory() as tmp:
        src, exe, inp = (os.path.join(tmp, n) for n in ("driver.cpp", "driver", "cases.json"))
        with open(src, "w") as f:
            f.write(DRIVER)
        with open(inp, "w") as f:
            json.dump(cases(), f)
        subprocess.check_call(["g++", "-std=c++23", "-O1", "-I", os.path.join(args.reference, "src"),
                               "-I", args.json_include, src, "-o", exe])
        parsed = json.loads(subprocess.check_output([exe, inp]))
    with open(args.out, "w") as f:
        json.dump({"cases": cases(), "parsed": parsed}, f, indent=1, sort_keys=True)
        f.write("\n")
    print(f"wrote {args.out}: {len(parsed)} cases")


if __name__ == "__main__":
    main()
