"""Configuration, registry, and the loader's errors (no GPU)."""
import copy
import json
import os

import pytest
import torch

import tiny_configs
from ccinfer_b200.config import Qwen3Config, architecture_of, load_config, register_architecture
from ccinfer_b200.errors import (ModelConfigInvalid, ModelLoadFailed, ModelUnsupportedArch, ModelUnsupportedDType)
from ccinfer_b200.weights import (SafetensorsFile, check_tensors, open_weights, write_random_model,
                                  write_safetensors)


def test_parse_tiny_configs():
    a = Qwen3Config.from_json(tiny_configs.TINY_A)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == \
        (2, 64, 4, 2, 16)
    assert a.tie_word_embeddings and a.rope_theta == 10000.0 and a.rms_norm_eps == 1e-6
    assert a.q_width == 64 and a.kv_width == 32 and a.group_size == 2
    assert all(a.layer_window(l) is None for l in range(2))
    b = Qwen3Config.from_json(tiny_configs.TINY_B)
    assert b.q_width == 256 != b.hidden_size and b.group_size == 4 and not b.tie_word_embeddings
    c = Qwen3Config.from_json(tiny_configs.TINY_C)
    assert [c.layer_window(l) for l in range(4)] == [None, 24, 24, 24]


def test_layer_types_win_over_the_window_rule():
    j = dict(tiny_configs.TINY_C, layer_types=["sliding_attention", "full_attention", "full_attention",
                                                "sliding_attention"])
    c = Qwen3Config.from_json(j)
    assert [c.layer_window(l) for l in range(4)] == [24, None, None, 24]
    assert Qwen3Config.from_json(c.to_json()) == c
    with pytest.raises(ModelConfigInvalid):
        Qwen3Config.from_json(dict(j, layer_types=["full_attention"]))
    with pytest.raises(ModelConfigInvalid):
        Qwen3Config.from_json(dict(j, sliding_window=None, use_sliding_window=False))
    # the keys as a stock checkpoint has them: a window size is named but not in use
    stock = dict(tiny_configs.TINY_A, use_sliding_window=False, sliding_window=4096, max_window_layers=2,
                 layer_types=["full_attention", "full_attention"], attention_dropout=0.0, bos_token_id=1)
    assert all(Qwen3Config.from_json(stock).layer_window(l) is None for l in range(2))


def test_defaults_follow_the_reference():
    j = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 64, "num_attention_heads": 4,
         "num_hidden_layers": 1, "intermediate_size": 8, "vocab_size": 10}
    c = Qwen3Config.from_json(j)
    assert c.num_key_value_heads == 4 and c.head_dim == 16 and c.max_position_embeddings == 2048
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6 and not c.tie_word_embeddings


@pytest.mark.parametrize("key", ["hidden_size", "num_attention_heads", "num_hidden_layers", "intermediate_size",
                                 "vocab_size"])
def test_required_keys(key):
    j = copy.deepcopy(tiny_configs.TINY_A)
    del j[key]
    with pytest.raises(ModelConfigInvalid, match=key):
        Qwen3Config.from_json(j)
    j[key] = "12"
    with pytest.raises(ModelConfigInvalid, match=key):
        Qwen3Config.from_json(j)
    j[key] = 0
    with pytest.raises(ModelConfigInvalid, match=key):
        Qwen3Config.from_json(j)


@pytest.mark.parametrize("patch", [
    {"num_key_value_heads": 3}, {"rope_theta": 0}, {"rms_norm_eps": -1e-6}, {"head_dim": 15},
    {"attention_bias": True}, {"rope_scaling": {"type": "yarn"}}, {"hidden_act": "gelu"},
    {"use_sliding_window": True, "sliding_window": None}, {"sliding_window": 0}, {"tie_word_embeddings": "yes"},
    {"max_position_embeddings": 0},
])
def test_refused_options(patch):
    j = copy.deepcopy(tiny_configs.TINY_A)
    j.update(patch)
    with pytest.raises(ModelConfigInvalid):
        Qwen3Config.from_json(j)


def test_dtype_and_architecture_errors():
    j = copy.deepcopy(tiny_configs.TINY_A)
    j["torch_dtype"] = "int8"
    with pytest.raises(ModelUnsupportedDType):
        Qwen3Config.from_json(j)
    for archs in (["LlamaForCausalLM"], ["Qwen2ForCausalLM"], [], None, "Qwen3ForCausalLM"):
        j = copy.deepcopy(tiny_configs.TINY_A)
        j["architectures"] = archs
        with pytest.raises(ModelUnsupportedArch):
            architecture_of(j)
    assert architecture_of(tiny_configs.TINY_A).name == "Qwen3ForCausalLM"


def test_registry_takes_another_architecture():
    register_architecture("ToyForTests", lambda j: ("cfg", j["x"]), lambda cfg: ("plan", cfg), replace=True)
    arch = architecture_of({"architectures": ["ToyForTests"], "x": 3})
    assert arch.build_plan(arch.parse_config({"x": 3})) == ("plan", ("cfg", 3))
    with pytest.raises(ValueError):
        register_architecture("ToyForTests", None, None)


def test_json_round_trip():
    for cfg in (tiny_configs.TINY_A, tiny_configs.TINY_B, tiny_configs.TINY_C):
        c = Qwen3Config.from_json(cfg)
        assert Qwen3Config.from_json(c.to_json()) == c


# ---------------------------------------------------------------------------------------------
def _specs(cfg):
    return architecture_of(cfg).build_plan(Qwen3Config.from_json(cfg)).tensor_specs()


def test_tensor_names_match_the_plain_implementation():
    import plain_qwen3 as plain
    for cfg in (tiny_configs.TINY_A, tiny_configs.TINY_B, tiny_configs.TINY_C):
        specs = {s.name: tuple(s.shape) for s in _specs(cfg)}
        assert specs == {k: tuple(v) for k, v in plain.tensor_shapes(cfg).items()}
    assert "lm_head.weight" not in {s.name for s in _specs(tiny_configs.TINY_A)}


def test_random_model_round_trip(tmp_path):
    cfg = Qwen3Config.from_json(tiny_configs.TINY_B)
    d = write_random_model(str(tmp_path / "m"), cfg, seed=5, std=0.05, store_dtype="bfloat16")
    arch, cfg2 = load_config(d)
    assert cfg2 == Qwen3Config.from_json({**tiny_configs.TINY_B, "torch_dtype": "bfloat16"})
    assert cfg2.torch_dtype == "bfloat16"
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    specs = arch.build_plan(cfg2).tensor_specs()
    check_tensors(specs, f.entries, "file")
    assert all(dt == "BF16" for dt, _ in f.entries.values())
    w = f.tensor("model.layers.0.self_attn.q_proj.weight").float()
    n = f.tensor("model.layers.2.input_layernorm.weight").float()
    assert abs(float(w.std()) - 0.05) < 0.01 and abs(float(w.mean())) < 0.01
    assert abs(float(n.mean()) - 1.0) < 0.05
    # the same seed gives the same file, another seed another
    d2 = write_random_model(str(tmp_path / "m2"), cfg, seed=5, std=0.05, store_dtype="bfloat16")
    f2 = SafetensorsFile(os.path.join(d2, "model.safetensors"))
    assert torch.equal(f2.tensor("lm_head.weight"), f.tensor("lm_head.weight"))
    d3 = write_random_model(str(tmp_path / "m3"), cfg, seed=6, std=0.05, store_dtype="float32")
    f3 = SafetensorsFile(os.path.join(d3, "model.safetensors"))
    assert not torch.equal(f3.tensor("lm_head.weight").to(torch.bfloat16), f.tensor("lm_head.weight"))
    assert f3.entries["lm_head.weight"][0] == "F32"


def test_one_error_lists_everything(tmp_path):
    cfg = tiny_configs.TINY_A
    specs = _specs(cfg)
    tensors = {s.name: torch.zeros(s.shape, dtype=torch.bfloat16) for s in specs}
    del tensors["model.norm.weight"]
    del tensors["model.layers.1.mlp.up_proj.weight"]
    tensors["lm_head.weight"] = torch.zeros(256, 64)  # tied model: not wanted
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.k_norm.weight"] = torch.zeros(16, dtype=torch.int32)
    d = tmp_path / "bad"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), tensors)
    with pytest.raises(ModelLoadFailed) as ei:
        open_weights(str(d), specs, "cpu", torch.float32)
    msg = str(ei.value)
    assert "missing tensors (2)" in msg and "model.norm.weight" in msg and "mlp.up_proj" in msg
    assert "unexpected tensors (2)" in msg and "lm_head.weight" in msg and "inv_freq" in msg
    assert "wrong shapes (1)" in msg and "[64, 32]" in msg and "[64, 64]" in msg
    assert "wrong storage types (1)" in msg and "k_norm" in msg


def test_extra_tensors_alone_are_no_fault(tmp_path):
    """A tied checkpoint that still carries lm_head.weight and an old rotary table loads (the reference loads by
    name and never looks at the rest: src/model/qwen3/qwen3_weights.cpp:74-152); strict loading refuses it."""
    cfg = tiny_configs.TINY_A
    specs = _specs(cfg)
    tensors = {s.name: torch.zeros(s.shape, dtype=torch.bfloat16) for s in specs}
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    d = tmp_path / "extra"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), tensors)
    with pytest.warns(UserWarning, match="ignored"):
        fetch = open_weights(str(d), specs, "cpu", torch.float32)
    assert fetch.unexpected == ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert fetch("model.norm.weight").shape == (64,)
    fetch.close()
    with pytest.raises(ModelLoadFailed, match=r"unexpected tensors \(2\)"):
        open_weights(str(d), specs, "cpu", torch.float32, strict=True)


def test_loader_types_on_load(tmp_path):
    cfg = tiny_configs.TINY_A
    specs = _specs(cfg)
    g = torch.Generator().manual_seed(0)
    tensors = {s.name: torch.randn(s.shape, generator=g) for s in specs}  # stored in 32 bits
    d = tmp_path / "f32"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), tensors)
    fetch = open_weights(str(d), specs, "cpu", torch.bfloat16, shared={"model.embed_tokens.weight"})
    q = fetch("model.layers.0.self_attn.q_proj.weight")
    n = fetch("model.layers.0.input_layernorm.weight")
    assert q.dtype == torch.bfloat16 and torch.equal(q, tensors["model.layers.0.self_attn.q_proj.weight"].bfloat16())
    assert n.dtype == torch.float32 and torch.equal(n, tensors["model.layers.0.input_layernorm.weight"])
    assert fetch("model.embed_tokens.weight") is fetch("model.embed_tokens.weight")  # the tied tensor is shared
    assert fetch("model.norm.weight") is not fetch("model.norm.weight")


def test_sharded_checkpoint(tmp_path):
    """Large checkpoints come as shards named by model.safetensors.index.json: same tensors, same one error."""
    import json
    cfg = tiny_configs.TINY_B
    specs = _specs(cfg)
    g = torch.Generator().manual_seed(1)
    tensors = {s.name: torch.randn(s.shape, generator=g).bfloat16() for s in specs}
    names = sorted(tensors)
    d = tmp_path / "sharded"
    d.mkdir()
    shards = {"model-00001-of-00003.safetensors": names[0::3], "model-00002-of-00003.safetensors": names[1::3],
              "model-00003-of-00003.safetensors": names[2::3]}
    for fn, ns in shards.items():
        write_safetensors(str(d / fn), {n: tensors[n] for n in ns})
    index = {"metadata": {}, "weight_map": {n: fn for fn, ns in shards.items() for n in ns}}
    (d / "model.safetensors.index.json").write_text(json.dumps(index))
    fetch = open_weights(str(d), specs, "cpu", torch.bfloat16)
    for n in names[:5] + names[-5:]:
        spec = next(s for s in specs if s.name == n)
        want = tensors[n].float() if spec.role == "vector" else tensors[n]
        assert torch.equal(fetch(n), want)
    fetch.close()
    # a tensor that the index lists but no shard holds is missing; a shard that is not there is named
    lost = names[4]
    write_safetensors(str(d / "model-00002-of-00003.safetensors"), {n: tensors[n] for n in names[1::3] if n != lost})
    with pytest.raises(ModelLoadFailed, match="missing tensors \\(1\\)") as ei:
        open_weights(str(d), specs, "cpu", torch.bfloat16)
    assert lost in str(ei.value)
    (d / "model-00003-of-00003.safetensors").unlink()
    with pytest.raises(ModelLoadFailed, match="model-00003-of-00003"):
        open_weights(str(d), specs, "cpu", torch.bfloat16)
    (d / "model.safetensors.index.json").write_text("[1, 2]")
    with pytest.raises(ModelLoadFailed, match="weight_map"):
        open_weights(str(d), specs, "cpu", torch.bfloat16)


@pytest.mark.parametrize("damage", ["short", "header_len", "json", "offsets", "dtype", "missing_file"])
def test_damaged_files(tmp_path, damage):
    d = tmp_path / "m"
    d.mkdir()
    path = d / "model.safetensors"
    write_safetensors(str(path), {"a": torch.zeros(4, 4)})
    raw = path.read_bytes()
    if damage == "short":
        path.write_bytes(raw[:5])
    elif damage == "header_len":
        path.write_bytes((10 ** 9).to_bytes(8, "little") + raw[8:])
    elif damage == "json":
        path.write_bytes(raw[:8] + b"{" * 10 + raw[18:])
    elif damage == "offsets":
        path.write_bytes(raw[:-8])
    elif damage == "dtype":
        path.write_bytes(raw.replace(b'"F32"', b'"F8X"'))
    else:
        path.unlink()
    with pytest.raises(ModelLoadFailed):
        open_weights(str(d), [], "cpu", torch.float32)


def _golden_config_cases():
    import json
    import os
    with open(os.path.join(os.path.dirname(__file__), "golden", "config_parse.json")) as f:
        g = json.load(f)
    return [(name, g["cases"][name], g["parsed"][name]) for name in sorted(g["cases"])]


@pytest.mark.parametrize("name,config_json,theirs", _golden_config_cases(), ids=lambda v: v if isinstance(v, str) else "")
def test_parser_agrees_with_the_reference_parser(name, config_json, theirs):
    """golden/config_parse.json holds what ModelConfig::from_json of 7QiC/ccInfer (src/model/config.h:41-160)
    read from these files (made by golden/make_config_golden.py).  Same fields, same error class; the
    reference stores theta and eps as 32-bit floats, this package as given."""
    import ccinfer_b200.errors as errors
    if "error" in theirs:
        with pytest.raises(getattr(errors, theirs["error"])):
            architecture_of(config_json).parse_config(config_json)
        return
    cfg = architecture_of(config_json).parse_config(config_json)
    for key in ("num_hidden_layers", "num_attention_heads", "num_key_value_heads", "hidden_size", "head_dim",
                "intermediate_size", "vocab_size", "max_position_embeddings"):
        assert getattr(cfg, key) == theirs[key], key
    for key in ("rope_theta", "rms_norm_eps"):
        assert getattr(cfg, key) == pytest.approx(theirs[key], rel=1e-6), key
