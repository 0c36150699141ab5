"""Weights by tensor name: checking, loading to the device, and the random-weights mode.

As in 7QiC/ccInfer the model folder holds one ``model.safetensors``
(src/worker/worker.cpp:256) and tensors are asked for by their HF names with
an expected shape (src/model/loader.h:87-155).  Unlike the reference, which
stops at the first missing tensor and never looks at the others, the whole
file is compared with the model's wants first and ONE error lists every
missing tensor, every unexpected one and every wrong shape.  Tensors the model
does not ask for are no fault by themselves (the reference never enumerates
the file, src/model/qwen3/qwen3_weights.cpp:74-152, and checkpoints of tied
models may still carry ``lm_head.weight`` or old rotary tables): alone they are
reported by a warning and ``fetch.unexpected``; beside a real fault they are
listed in the error, where a mistyped name shows up as one missing and one
unexpected tensor.

Types on the device: matrices in the compute type (bfloat16 for serving, float
for the 32-bit path); per-channel vectors (norm weights) always in float, which
holds a bfloat16 value exactly and leaves a tensor stored in 32 bits as it is;
integer tables as int32.  A matrix stored in float is rounded to nearest-even
when the compute type is bfloat16.
"""
from __future__ import annotations

import json
import os
import warnings
from typing import Callable, Dict, List

import torch

from ..errors import ModelLoadFailed
from ..parts.base import TensorSpec
from .random_init import normal_tensor
from .safetensors_io import SafetensorsFile, write_safetensors

WEIGHTS_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"   # large checkpoints: {"weight_map": {tensor name: shard file}}


class _Shards:
    """Several safetensors files behind the interface of one (``entries``, ``tensor``, ``close``).

    What the index promises is not trusted: the tensors are those the shard files really hold, so a name
    the index lists but no shard has shows up as missing in the one error."""

    def __init__(self, model_dir: str, index_path: str):
        try:
            with open(index_path) as f:
                weight_map = json.load(f)["weight_map"]
            shard_names = sorted(set(weight_map.values()))
        except (OSError, ValueError, KeyError, AttributeError, TypeError) as e:
            raise ModelLoadFailed(f"{index_path} is not a safetensors index (a JSON object with a weight_map): {e}")
        self.files = []
        self.entries: Dict[str, tuple] = {}
        self._owner: Dict[str, SafetensorsFile] = {}
        for shard in shard_names:
            path = os.path.join(model_dir, shard)
            if os.path.basename(shard) != shard or not os.path.isfile(path):
                self.close()
                raise ModelLoadFailed(f"{index_path} names the shard '{shard}', which is not a file of {model_dir}")
            f = SafetensorsFile(path)
            self.files.append(f)
            for name, entry in f.entries.items():
                if name in self._owner:
                    self.close()
                    raise ModelLoadFailed(f"tensor '{name}' is stored in more than one shard of {model_dir}")
                self.entries[name] = entry
                self._owner[name] = f

    def tensor(self, name: str) -> torch.Tensor:
        return self._owner[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def open_checkpoint(model_dir: str):
    """The folder's weights: ``model.safetensors``, or the shards that ``model.safetensors.index.json`` names."""
    path = os.path.join(model_dir, WEIGHTS_FILE)
    if os.path.isfile(path):
        return SafetensorsFile(path), path
    index = os.path.join(model_dir, INDEX_FILE)
    if os.path.isfile(index):
        return _Shards(model_dir, index), index
    raise ModelLoadFailed(f"{path} does not exist (the model folder holds config.json and {WEIGHTS_FILE}, "
                          f"or {INDEX_FILE} with its shards)")


def check_tensors(specs: List[TensorSpec], entries: Dict[str, tuple], where: str, strict: bool = False) -> List[str]:
    """Raises ModelLoadFailed naming all missing, unexpected and mis-shaped tensors, or returns the names
    of the tensors that the file holds and the model does not want (with ``strict`` those raise as well)."""
    wanted = {s.name: s for s in specs}
    missing = sorted(n for n in wanted if n not in entries)
    unexpected = sorted(n for n in entries if n not in wanted)
    wrong = []
    for n, s in wanted.items():
        if n in entries and tuple(entries[n][1]) != tuple(s.shape):
            wrong.append(f"{n}: file has {list(entries[n][1])}, model wants {list(s.shape)}")
    bad_type = []
    for n, s in wanted.items():
        if n in entries:
            integer = entries[n][0] in ("I32", "I64")
            if integer != (s.role == "table"):
                bad_type.append(f"{n}: stored as {entries[n][0]}, model wants "
                                f"{'an integer table' if s.role == 'table' else 'floating point'}")
    if not (missing or wrong or bad_type or (strict and unexpected)):
        return unexpected
    lines = [f"{where} does not match the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(sorted(wrong)))
    if bad_type:
        lines.append(f"  wrong storage types ({len(bad_type)}): " + "; ".join(sorted(bad_type)))
    raise ModelLoadFailed("\n".join(lines))


def device_dtype(spec: TensorSpec, compute_dtype: torch.dtype) -> torch.dtype:
    if spec.role == "vector":
        return torch.float32
    if spec.role == "table":
        return torch.int32
    return compute_dtype


def open_weights(model_dir: str, specs: List[TensorSpec], device, compute_dtype,
                 shared=(), strict: bool = False) -> Callable[[str], torch.Tensor]:
    """Checks the folder's file against ``specs`` and returns ``fetch(name) -> device tensor``.

    Tensors of the file that the model does not want are left alone: ``fetch.unexpected`` names them and a
    warning says so once (``strict`` turns them into the load error).

    Names in ``shared`` (wanted by more than one part, like a tied head) are
    copied once and handed out again; every other call makes a fresh copy that
    the asking part owns."""
    f, path = open_checkpoint(model_dir)
    try:
        unexpected = check_tensors(specs, f.entries, path, strict=strict)
    except ModelLoadFailed:
        f.close()
        raise
    if unexpected:
        warnings.warn(f"{path}: {len(unexpected)} tensors that the model does not use are ignored: "
                      + ", ".join(unexpected[:8]) + (" ..." if len(unexpected) > 8 else ""), stacklevel=2)
    by_name = {s.name: s for s in specs}
    cache: Dict[str, torch.Tensor] = {}

    def fetch(name: str) -> torch.Tensor:
        if name in cache:
            return cache[name]
        spec = by_name[name]
        t = f.tensor(name).to(device=device, dtype=device_dtype(spec, compute_dtype)).contiguous()
        if name in shared:
            cache[name] = t
        return t

    fetch.close = f.close  # type: ignore[attr-defined]
    fetch.unexpected = unexpected  # type: ignore[attr-defined]
    return fetch


# ---------------------------------------------------------------------------------------------
# random weights
# ---------------------------------------------------------------------------------------------
def random_tensor(spec: TensorSpec, seed: int, std: float, device="cpu", dtype=torch.float32) -> torch.Tensor:
    """One tensor of the random model: N(0, std), or 1 + N(0, std) for norm weights, in ``dtype``.

    The values are those of the counter-based stream of (seed, tensor name) (see ``random_init``): they do
    not change with the order or the number of the other tensors, nor with where they are drawn; bfloat16
    is the float value rounded once.
    """
    if spec.role == "table":
        raise ModelLoadFailed(f"no random rule for the integer table '{spec.name}'")
    return normal_tensor(spec.shape, seed, spec.name, std, spec.init == "one_plus_normal", dtype, device)


def write_random_model(model_dir: str, config, seed: int, std: float = 0.02, store_dtype: str = None) -> str:
    """Writes ``config.json`` and ``model.safetensors`` for a typed configuration and a seed.

    Values are drawn in float and stored in ``store_dtype`` ("bfloat16" or
    "float32"; default: the configuration's torch_dtype).
    """
    from ..config.registry import architecture_of
    cj = config.to_json()
    arch = architecture_of(cj)
    store_dtype = store_dtype or cj.get("torch_dtype", "bfloat16")
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[store_dtype]
    cj["torch_dtype"] = store_dtype
    plan = arch.build_plan(config)
    os.makedirs(model_dir, exist_ok=True)
    tensors = {s.name: random_tensor(s, seed, std).to(tdt) for s in plan.tensor_specs()}
    write_safetensors(os.path.join(model_dir, WEIGHTS_FILE), tensors,
                      metadata={"format": "pt", "weights_seed": seed, "weights_std": std})
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cj, f, indent=1)
    return model_dir


def random_fetch(specs: List[TensorSpec], seed: int, std: float, device, compute_dtype, shared=()):
    """``fetch`` that draws every tensor on the device (no file; for measurements on large shapes)."""
    by_name = {s.name: s for s in specs}
    cache: Dict[str, torch.Tensor] = {}

    def fetch(name: str) -> torch.Tensor:
        if name in cache:
            return cache[name]
        spec = by_name[name]
        t = random_tensor(spec, seed, std, device=device, dtype=device_dtype(spec, compute_dtype))
        if name in shared:
            cache[name] = t
        return t

    fetch.close = lambda: None  # type: ignore[attr-defined]
    return fetch
