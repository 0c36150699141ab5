"""The random-weights stream: one counter-based generator, the same bits on the host and on the device.

7QiC/ccInfer has no random mode (src/model/qwen3/qwen3_weights.cpp:49-51 loads bfloat16 checkpoints only).
Here a seed names ONE model, whatever the route: drawn on the device by ``csrc/random_init.cu`` (a model of
tens of gigabytes in a second or two), or on the host by the NumPy code below (``write_random_model``
without a GPU).  Element i of a tensor depends on (seed, tensor name, i) only:

  words = Philox4x32-10(counter = (g lo, g hi, name key lo, name key hi), key = (seed lo, seed hi)), g = i // 4
  two Box-Muller pairs per call; logarithm, sine and cosine by fixed polynomials whose every product and
  sum is one IEEE float operation (no fused multiply-add, no library function), so both sides round alike.

``csrc/random_init.cu`` states the formulas; the two files must change together.
"""
from __future__ import annotations

import hashlib

import numpy as np
import torch

_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = np.uint64(0x9E3779B9), np.uint64(0xBB67AE85)
_MASK = np.uint64(0xFFFFFFFF)
_S32 = np.uint64(32)

f32 = np.float32
_SQRT2 = f32(1.41421354)
_LN2 = f32(0.693147182)
_PI_4 = f32(0.785398185)
_LN_COEF = [f32(1.0) / f32(d) for d in (11.0, 9.0, 7.0, 5.0, 3.0)]
_SIN_COEF = [f32(1.0) / f32(362880.0), f32(-1.0) / f32(5040.0), f32(1.0) / f32(120.0), f32(-1.0) / f32(6.0)]
_COS_COEF = [f32(-1.0) / f32(3628800.0), f32(1.0) / f32(40320.0), f32(-1.0) / f32(720.0), f32(1.0) / f32(24.0),
             f32(-0.5)]


def tensor_key(name: str) -> int:
    """The 64-bit number that stands for a tensor's name in the generator's counter."""
    return int.from_bytes(hashlib.sha256(name.encode()).digest()[:8], "little")


def _philox(g: np.ndarray, key: int, seed: int):
    c = [g & _MASK, g >> _S32, np.full_like(g, key & 0xFFFFFFFF), np.full_like(g, (key >> 32) & 0xFFFFFFFF)]
    k0, k1 = np.uint64(seed & 0xFFFFFFFF), np.uint64((seed >> 32) & 0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = _M0 * c[0], _M1 * c[2]
        c = [(p1 >> _S32) ^ c[1] ^ k0, p1 & _MASK, (p0 >> _S32) ^ c[3] ^ k1, p0 & _MASK]
        k0, k1 = (k0 + _W0) & _MASK, (k1 + _W1) & _MASK
    return c


def _normal_pair(wa: np.ndarray, wb: np.ndarray):
    u = ((wa >> np.uint64(9)).astype(f32) + f32(0.5)) * f32(1.0 / 8388608.0)
    bits = u.view(np.uint32)
    e = (bits >> np.uint32(23)).astype(np.int32) - np.int32(127)
    m = ((bits & np.uint32(0x7FFFFF)) | np.uint32(0x3F800000)).view(f32)
    big = m > _SQRT2
    m = np.where(big, m * f32(0.5), m)
    e = e + big.astype(np.int32)
    s = (m - f32(1.0)) / (m + f32(1.0))
    s2 = s * s
    poly = np.full_like(s, _LN_COEF[0])
    for c in _LN_COEF[1:]:
        poly = poly * s2 + c
    poly = poly * s2
    two_s = f32(2.0) * s
    ln_u = e.astype(f32) * _LN2 + (two_s + two_s * poly)
    r = np.sqrt(f32(-2.0) * ln_u)

    k = wb >> np.uint64(8)
    octant = (k >> np.uint64(21)).astype(np.int32)
    x = ((k & np.uint64(0x1FFFFF)).astype(f32) + f32(0.5)) * f32(1.0 / 2097152.0) * _PI_4
    x2 = x * x
    ps = np.full_like(x, _SIN_COEF[0])
    for c in _SIN_COEF[1:]:
        ps = ps * x2 + c
    sn = x + (x * x2) * ps
    pc = np.full_like(x, _COS_COEF[0])
    for c in _COS_COEF[1:]:
        pc = pc * x2 + c
    cs = f32(1.0) + x2 * pc
    swap = (((octant + 1) >> 1) & 1).astype(bool)
    c = np.where(swap, sn, cs)
    sv = np.where(swap, cs, sn)
    c = np.where((octant >= 2) & (octant <= 5), -c, c)
    sv = np.where(octant >= 4, -sv, sv)
    return r * c, r * sv


def normal_host(numel: int, seed: int, name: str, std: float, add_one: bool = False,
                chunk_groups: int = 1 << 20) -> np.ndarray:
    """float32 [numel]: std * z (+ 1), the stream of (seed, name); bit for bit what the device kernel writes."""
    out = np.empty(((numel + 3) // 4) * 4, dtype=f32)
    key = tensor_key(name)
    groups = (numel + 3) // 4
    with np.errstate(over="ignore"):   # the 64-bit products of Philox wrap by design
        for g0 in range(0, groups, chunk_groups):
            g = np.arange(g0, min(groups, g0 + chunk_groups), dtype=np.uint64)
            w = _philox(g, key, seed)
            z0, z1 = _normal_pair(w[0], w[1])
            z2, z3 = _normal_pair(w[2], w[3])
            block = np.stack([z0, z1, z2, z3], axis=1).reshape(-1) * f32(std)
            if add_one:
                block = block + f32(1.0)
            out[4 * g0:4 * g0 + block.size] = block
    return out[:numel]


def normal_tensor(shape, seed: int, name: str, std: float, add_one: bool, dtype: torch.dtype, device) -> torch.Tensor:
    """A tensor of the stream of (seed, name) in ``dtype`` (float32, or bfloat16 rounded once from it), drawn
    where it is to live: by the CUDA kernel on a CUDA device, by NumPy on the host."""
    device = torch.device(device)
    numel = 1
    for s in shape:
        numel *= int(s)
    if device.type == "cuda":
        from .. import kernels
        out = torch.empty(tuple(shape), dtype=dtype, device=device)
        with torch.cuda.device(device):
            kernels.init_random(out, seed, tensor_key(name), std, add_one)
        return out
    host = torch.from_numpy(normal_host(numel, seed, name, std, add_one)).view(tuple(shape))
    return host.to(dtype)
