"""The random-weights stream: one model per seed, whatever the route.

The package draws it on the host (NumPy) and on the device (a CUDA kernel); tests/plain_qwen3.py restates
it a third time in plain torch.  All three must agree bit for bit, the values must be normal, and a
tensor's values must depend on (seed, tensor name, element index) only.
"""
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import tiny_configs
from ccinfer_b200.weights import random_init


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.mark.parametrize("n,seed,name,add_one", [
    (1, 0, "a", False), (7, 1, "model.norm.weight", True), (4096, 42, "model.layers.3.mlp.up_proj.weight", False),
    (100003, 2 ** 40 + 5, "lm_head.weight", False)])
def test_host_stream_equals_the_plain_restatement(n, seed, name, add_one):
    a = random_init.normal_host(n, seed, name, 0.02, add_one)
    b = plain.stream_normal(n, seed, name, 0.02, add_one).numpy()
    assert a.dtype == np.float32 and a.shape == (n,)
    assert np.array_equal(_bits(a), _bits(b))


def test_stream_is_a_function_of_seed_name_and_index():
    a = random_init.normal_host(1000, 3, "x", 0.05)
    assert np.array_equal(_bits(random_init.normal_host(250, 3, "x", 0.05)), _bits(a[:250]))   # a prefix
    assert np.array_equal(_bits(random_init.normal_host(1000, 3, "x", 0.05, chunk_groups=7)), _bits(a))
    assert not np.array_equal(random_init.normal_host(1000, 4, "x", 0.05), a)
    assert not np.array_equal(random_init.normal_host(1000, 3, "y", 0.05), a)
    # seeds that differ only above 32 bits are different streams
    assert not np.array_equal(random_init.normal_host(1000, 3 + 2 ** 32, "x", 0.05), a)


def test_stream_is_normal():
    from scipy import stats
    z = random_init.normal_host(2_000_000, 11, "t", 1.0).astype(np.float64)
    assert abs(z.mean()) < 3e-3 and abs(z.std() - 1.0) < 3e-3
    assert abs(stats.skew(z)) < 1e-2 and abs(stats.kurtosis(z)) < 2e-2
    assert stats.kstest(z[:300000], "norm").pvalue > 1e-3
    assert np.abs(z).max() > 4.5                                   # the tails are there
    for lag in (1, 2, 3, 4):                                        # neighbours, also across the pairs of a call
        assert abs(np.corrcoef(z[:-lag], z[lag:])[0, 1]) < 3e-3
    w = random_init.normal_host(200000, 11, "n", 0.02, add_one=True)
    assert abs(w.mean() - 1.0) < 2e-4 and abs(w.std() - 0.02) < 2e-4


def test_random_model_file_holds_the_stream(tmp_path):
    """write_random_model: every tensor is its stream, rounded once to the stored type."""
    from ccinfer_b200.config import Qwen3Config
    from ccinfer_b200.weights import write_random_model
    from ccinfer_b200.weights.safetensors_io import SafetensorsFile
    cfg = tiny_configs.TINY_B
    d = write_random_model(str(tmp_path / "m"), Qwen3Config.from_json(cfg), seed=9, std=0.05, store_dtype="bfloat16")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    want = plain.stream_weights(cfg, 9, 0.05)
    assert set(want) == set(f.entries)
    for name, w in want.items():
        assert torch.equal(f.tensor(name), w.to(torch.bfloat16)), name


# ---------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,add_one", [(1, False), (7, True), (1000003, False), (4096 * 12288, False)])
def test_device_stream_equals_host_stream(dtype, n, add_one):
    from ccinfer_b200 import kernels
    out = torch.empty(n, dtype=dtype, device="cuda")
    key = random_init.tensor_key("model.layers.0.mlp.gate_proj.weight")
    kernels.init_random(out, 42, key, 0.02, add_one)
    if n > 10_000_000:   # the large tensor: the plain restatement on the device stands in for the host loop
        want = plain.stream_normal(n, 42, "model.layers.0.mlp.gate_proj.weight", 0.02, add_one, device="cuda")
        head = torch.from_numpy(random_init.normal_host(100000, 42, "model.layers.0.mlp.gate_proj.weight", 0.02, add_one))
        assert torch.equal(want[:100000].cpu(), head)
    else:
        want = torch.from_numpy(random_init.normal_host(n, 42, "model.layers.0.mlp.gate_proj.weight", 0.02, add_one)).cuda()
    assert torch.equal(out, want.to(dtype))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_seed_names_one_model_whatever_the_route(tmp_path, dtype):
    """Engine.from_random(seed) holds bit for bit what loading write_random_model(seed) gives."""
    from ccinfer_b200.config import Qwen3Config
    from ccinfer_b200.config.registry import architecture_of
    from ccinfer_b200.weights import open_weights, random_fetch, write_random_model
    cfg = Qwen3Config.from_json(tiny_configs.TINY_B)
    d = write_random_model(str(tmp_path / "m"), cfg, seed=1, std=0.05, store_dtype="float32")
    plan = architecture_of(cfg.to_json()).build_plan(cfg)
    specs = plan.tensor_specs()
    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    from_file = open_weights(d, specs, "cuda", tdt)
    drawn = random_fetch(specs, 1, 0.05, "cuda", tdt)
    for s in specs:
        a, b = from_file(s.name), drawn(s.name)
        assert a.dtype == b.dtype and torch.equal(a, b), s.name
    from_file.close()
