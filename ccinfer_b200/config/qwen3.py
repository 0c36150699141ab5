"""Typed configuration of Qwen3 dense, read from the architecture's config.json keys.

Keys and defaults follow 7QiC/ccInfer's parser (src/model/config.h:55-154):
``hidden_size``, ``num_attention_heads``, ``num_hidden_layers``,
``intermediate_size`` and ``vocab_size`` are required integers > 0;
``num_key_value_heads`` defaults to the number of heads, ``head_dim`` to
hidden / heads, ``max_position_embeddings`` to 2048, ``rope_theta`` to 10000
and ``rms_norm_eps`` to 1e-6.  Beyond the reference, which silently ignores
them, ``tie_word_embeddings`` and the sliding-window keys are honoured and
options the engine does not compute (``attention_bias``, ``rope_scaling``, an
activation other than silu) are refused instead of ignored.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

from ..errors import ModelConfigInvalid, ModelUnsupportedDType

_DTYPES = ("bfloat16", "float16", "float32")


def _req_int(j: dict, key: str) -> int:
    if key not in j:
        raise ModelConfigInvalid(f"config.json: required key '{key}' is missing")
    return _int(j, key)


def _int(j: dict, key: str) -> int:
    v = j[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ModelConfigInvalid(f"config.json: '{key}' must be an integer, got {v!r}")
    if not (-(2 ** 31) <= v < 2 ** 31):
        raise ModelConfigInvalid(f"config.json: '{key}' = {v} does not fit 32 bits")
    return v


def _num(j: dict, key: str) -> float:
    v = j[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ModelConfigInvalid(f"config.json: '{key}' must be a number, got {v!r}")
    return float(v)


@dataclasses.dataclass(frozen=True)
class Qwen3Config:
    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    max_position_embeddings: int = 2048
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    layer_types: Optional[tuple] = None   # per layer "full_attention" / "sliding_attention", if the file has it

    # -- derived -----------------------------------------------------------
    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def layer_window(self, layer: int) -> Optional[int]:
        """Keys a layer's queries see besides causality: None = all of them.

        With ``use_sliding_window`` the layers from ``max_window_layers`` on
        see the last ``sliding_window`` keys (their own included).  A
        ``layer_types`` list, where the file has one, says it layer by layer
        and wins over that rule.
        """
        if self.layer_types is not None:
            return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        first = self.num_hidden_layers if self.max_window_layers is None else self.max_window_layers
        return self.sliding_window if layer >= first else None

    # -- json --------------------------------------------------------------
    @classmethod
    def from_json(cls, j: dict) -> "Qwen3Config":
        arch = j["architectures"][0]
        hidden = _req_int(j, "hidden_size")
        heads = _req_int(j, "num_attention_heads")
        layers = _req_int(j, "num_hidden_layers")
        inter = _req_int(j, "intermediate_size")
        vocab = _req_int(j, "vocab_size")
        for k, v in (("hidden_size", hidden), ("num_attention_heads", heads),
                     ("num_hidden_layers", layers), ("intermediate_size", inter),
                     ("vocab_size", vocab)):
            if v <= 0:
                raise ModelConfigInvalid(f"config.json: '{k}' must be > 0, got {v}")
        kv_heads = _int(j, "num_key_value_heads") if "num_key_value_heads" in j else heads
        head_dim = _int(j, "head_dim") if "head_dim" in j else hidden // heads
        max_pos = _int(j, "max_position_embeddings") if "max_position_embeddings" in j else 2048
        theta = _num(j, "rope_theta") if "rope_theta" in j else 10000.0
        eps = _num(j, "rms_norm_eps") if "rms_norm_eps" in j else 1e-6
        dtype = j.get("torch_dtype", j.get("dtype", "bfloat16"))
        if dtype not in _DTYPES:
            raise ModelUnsupportedDType(f"config.json: torch_dtype {dtype!r} is not one of {_DTYPES}")
        if theta <= 0 or eps <= 0:
            raise ModelConfigInvalid("config.json: rope_theta and rms_norm_eps must be > 0")
        if kv_heads <= 0 or max_pos <= 0 or head_dim <= 0:
            raise ModelConfigInvalid(
                "config.json: num_key_value_heads, max_position_embeddings and head_dim must be > 0")
        if heads % kv_heads != 0:
            raise ModelConfigInvalid(
                f"config.json: num_attention_heads {heads} is not a multiple of "
                f"num_key_value_heads {kv_heads}")
        if head_dim % 2 != 0:
            raise ModelConfigInvalid(f"config.json: head_dim {head_dim} must be even for rotate-half RoPE")
        tie = j.get("tie_word_embeddings", False)
        if not isinstance(tie, bool):
            raise ModelConfigInvalid("config.json: 'tie_word_embeddings' must be true or false")
        # options the engine does not compute are refused, never ignored
        if j.get("attention_bias", False):
            raise ModelConfigInvalid("config.json: attention_bias = true is not supported")
        if j.get("rope_scaling") is not None:
            raise ModelConfigInvalid("config.json: rope_scaling is not supported")
        if j.get("hidden_act", "silu") != "silu":
            raise ModelConfigInvalid(f"config.json: hidden_act {j['hidden_act']!r} is not supported (silu only)")
        use_sw = j.get("use_sliding_window", False)
        if not isinstance(use_sw, bool):
            raise ModelConfigInvalid("config.json: 'use_sliding_window' must be true or false")
        sw = j.get("sliding_window")
        if sw is not None:
            sw = _int(j, "sliding_window")
            if sw <= 0:
                raise ModelConfigInvalid("config.json: 'sliding_window' must be > 0 or null")
        mwl = j.get("max_window_layers")
        if mwl is not None:
            mwl = _int(j, "max_window_layers")
            if mwl < 0:
                raise ModelConfigInvalid("config.json: 'max_window_layers' must be >= 0")
        if use_sw and sw is None:
            raise ModelConfigInvalid("config.json: use_sliding_window is true but sliding_window is null")
        lt = j.get("layer_types")
        if lt is not None:
            if (not isinstance(lt, list) or len(lt) != layers
                    or any(t not in ("full_attention", "sliding_attention") for t in lt)):
                raise ModelConfigInvalid("config.json: 'layer_types' must list full_attention or "
                                         "sliding_attention for each of the layers")
            if "sliding_attention" in lt and sw is None:
                raise ModelConfigInvalid("config.json: layer_types has sliding_attention but sliding_window is null")
            lt = tuple(lt)
        return cls(architecture=arch, vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers,
                   num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
                   intermediate_size=inter, max_position_embeddings=max_pos, rope_theta=theta,
                   rms_norm_eps=eps, tie_word_embeddings=tie, torch_dtype=dtype,
                   use_sliding_window=use_sw, sliding_window=sw, max_window_layers=mwl, layer_types=lt)

    def to_json(self) -> dict:
        j = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.torch_dtype,
            "hidden_act": "silu",
            "attention_bias": False,
            "rope_scaling": None,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
        }
        if self.layer_types is not None:
            j["layer_types"] = list(self.layer_types)
        return j
