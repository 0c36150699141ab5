"""Reader and writer of the safetensors container.

Format (as 7QiC/ccInfer reads it, src/model/loader.cpp:67-162): an unsigned
64-bit little-endian header length, a JSON object ``{name: {dtype, shape,
data_offsets: [begin, end]}, "__metadata__": {...}}`` and the tensor bytes;
offsets are relative to the end of the header.  The file is memory-mapped and
tensors are handed out as views, so nothing is copied before the device copy.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Tuple

import numpy as np
import torch

from ..errors import ModelLoadFailed

# storage type -> (torch dtype, bytes per element, numpy type of the raw view)
_DTYPES = {
    "F32": (torch.float32, 4, np.float32),
    "BF16": (torch.bfloat16, 2, np.int16),
    "F16": (torch.float16, 2, np.float16),
    "I32": (torch.int32, 4, np.int32),
    "I64": (torch.int64, 8, np.int64),
}
_NAMES = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.int32: "I32",
          torch.int64: "I64"}


class SafetensorsFile:
    """A memory-mapped safetensors file: ``entries`` maps name -> (dtype name, shape)."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise ModelLoadFailed(f"cannot open {path}: {e}") from e
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise ModelLoadFailed(f"{path}: too short for a safetensors header ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise ModelLoadFailed(f"{path}: header length {hlen} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise ModelLoadFailed(f"{path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise ModelLoadFailed(f"{path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + hlen
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.entries: Dict[str, Tuple[str, Tuple[int, ...]]] = {}
        self._offsets: Dict[str, Tuple[int, int]] = {}
        data_len = size - self._data_start
        for name, info in header.items():
            try:
                dt, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError) as ex:
                raise ModelLoadFailed(f"{path}: malformed header entry for '{name}': {ex}") from ex
            if dt not in _DTYPES:
                raise ModelLoadFailed(f"{path}: tensor '{name}' has unsupported storage type {dt}")
            n = 1
            for s in shape:
                n *= s
            if not (0 <= b <= e <= data_len) or e - b != n * _DTYPES[dt][1]:
                raise ModelLoadFailed(
                    f"{path}: tensor '{name}' {dt}{list(shape)} has bad data offsets [{b}, {e}) "
                    f"(data section is {data_len} bytes)")
            self.entries[name] = (dt, shape)
            self._offsets[name] = (b, e)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the file's bytes (read-only memory: copy before writing)."""
        dt, shape = self.entries[name]
        tdt, _, ndt = _DTYPES[dt]
        b, e = self._offsets[name]
        n = (e - b) // _DTYPES[dt][1]
        arr = np.frombuffer(self._mm, dtype=ndt, count=n, offset=self._data_start + b)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns about the non-writable buffer
            t = torch.from_numpy(arr)
        if dt == "BF16":
            t = t.view(torch.bfloat16)
        return t.view(shape) if shape else t.view(())

    def close(self):
        # tensors handed out keep the map alive through numpy; closing is best-effort
        try:
            self._mm.close()
        except (BufferError, ValueError):
            pass
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata=None) -> None:
    """Writes CPU tensors in the order given; data of each tensor starts 8-byte aligned."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise ModelLoadFailed(f"cannot store tensor '{name}' of type {t.dtype}")
        raw = t.view(torch.int16).numpy().tobytes() if t.dtype == torch.bfloat16 else t.numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
