"""What every part needs of the device: the compute type, scratch memory, the matrix product and the status word."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .. import kernels
from ..errors import DeviceFault, ExtensionMissing, ScratchMoved, Unsupported
from ..parts.base import UnscaledRows


class ScratchPool:
    """Named buffers that live as long as the engine.

    ``get(key, shape, dtype)`` returns the same storage for the same key; parts
    ask for their largest shape (``[max_tokens, width]``) and slice the rows of a
    step.  Layers share a buffer by using the same key; a key asked with a larger
    size gets new storage, which is harmless until a CUDA graph has recorded the
    old address.  The engine therefore runs a step eagerly (every key reaches the
    largest size the model's parts ask for) and then calls ``freeze()`` before it
    captures the first graph: from then on a request for more than an existing
    buffer holds raises instead of moving it from under the graphs (a key asked
    for the first time still gets its buffer: no graph can hold its address).
    """

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}
        self.frozen = False

    def get(self, key: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        full_key = f"{key}:{dtype}"
        buf = self._bufs.get(full_key)
        if buf is None or buf.numel() < n:
            if self.frozen and buf is not None:   # a new key is no harm: no graph holds an address of it
                raise ScratchMoved(f"scratch buffer '{key}' ({dtype}) is asked for {n} elements after CUDA graphs "
                                   f"recorded the addresses of the pool (it holds "
                                   f"{0 if buf is None else buf.numel()}): a part must ask for its largest "
                                   f"shape, not for the shape of the step")
            buf = torch.empty(n, dtype=dtype, device=self.device)
            self._bufs[full_key] = buf
        return buf[:n].view(shape)

    def freeze(self) -> None:
        self.frozen = True

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


class Runtime:
    def __init__(self, device, dtype: torch.dtype, max_tokens: int, max_entries: int):
        if not torch.cuda.is_available():
            raise ExtensionMissing("no CUDA device: the engine has no CPU path")
        if dtype not in (torch.float32, torch.bfloat16):
            raise Unsupported(f"compute type {dtype} is not supported (float32 or bfloat16)")
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_tokens = int(max_tokens)
        self.max_entries = int(max_entries)
        torch.cuda.set_device(self.device)
        kernels.lib()  # build / load now: fail loudly before anything else happens
        self.scratch = ScratchPool(self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.cublas = kernels.CublasHandle(self.device) if dtype == torch.bfloat16 else None
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.tc_counters = torch.zeros(4096, dtype=torch.int32, device=self.device)  # split-K tile counters
        self.merge_counters = torch.zeros(8192, dtype=torch.int32, device=self.device)  # attention split counters
        self._sink_turn = 0

    @staticmethod
    def rows(x):
        """x as a plain tensor (rows that a norm left short of their factor are finished)."""
        return x.finish() if isinstance(x, UnscaledRows) else x

    def _into_stream(self, out, x, w, sink) -> bool:
        """The product as the last one of a part, with few rows: added into the residual stream by its own
        epilogue, which also leaves the rows of the norm that follows short of one factor per row (the norm
        then needs no kernel).  False: not this time (another kind of norm)."""
        norm, h = sink.norm, sink.stream.h
        N, M = w.shape[0], x.shape[0]
        if (getattr(norm, "unscaled_rows_from", None) is None or sink.stream.pending is not None
                or h.shape != (M, N) or out.dtype != torch.bfloat16):
            return False
        self._sink_turn ^= 1   # two sets of buffers in turn: the rows of one norm are read while the next are written
        parts = kernels.gemm_fewrows_blocks(N)
        ssq = self.scratch.get(f"unscaled_ssq{self._sink_turn}", (kernels.FEWROWS_MAX_ROWS, parts), torch.float32)
        xw = self.scratch.get(f"unscaled_rows{self._sink_turn}", (kernels.FEWROWS_MAX_ROWS, N), self.dtype)[:M]
        rows = norm.unscaled_rows_from(sink.stream, xw, ssq, parts)
        if rows is None:
            return False
        kernels.gemm_fewrows_norm_bf16(xw, x, w, into=(h, norm.w, ssq), status=self.status)
        sink.stream.unscaled = rows
        return True

    def linear(self, out: torch.Tensor, x, w: torch.Tensor, sink=None):
        """out[M, N] = x[M, K] @ w[N, K]^T; out may be float for bfloat16 operands (the logits).

        ``x`` may be ``UnscaledRows``.  ``sink`` (a ``ResidualSink``): the product is the last of its part and
        may add its result into the residual stream itself; then None is returned instead of ``out``."""
        if self.dtype == torch.float32:
            kernels.gemm_f32(out, self.rows(x), w)
            return out
        xt = x.x if isinstance(x, UnscaledRows) else x
        M, K = xt.shape
        N = w.shape[0]
        choice = "library"
        if M <= kernels.SKINNY_MAX_ROWS:  # a few tokens: the product is a stream of the weights
            choice = kernels.few_rows_product_kernel(
                M, N, K, self.sm_count, kernels.gemm_tc_fits(K, xt, w), kernels.gemm_fewrows_fits(M, K, xt, w),
                kernels.gemm_skinny_fits(M, K, xt, w))
        if choice == "fewrows":
            if sink is not None and xt is x and self._into_stream(out, x, w, sink):
                return None
            if xt is not x:
                kernels.gemm_fewrows_norm_bf16(out, xt, w, scale=x.scale, status=self.status)
            else:
                kernels.gemm_fewrows_bf16(out, x, w, status=self.status)
            return out
        x = self.rows(x)
        if choice == "tc":
            kernels.gemm_tc_bf16(out, x, w, 1, None, None, self.status)
            return out
        if choice == "skinny":
            kernels.gemm_skinny_bf16(out, x, w)
            return out
        if choice == "tc_split":
            splits = kernels.gemm_tc_splits(M, N, K)
            partial = counters = None
            if splits > 1:
                partial = self.scratch.get("tc_partial", (splits * kernels.SKINNY_MAX_ROWS * N,), torch.float32)
                counters = self.tc_counters
            kernels.gemm_tc_bf16(out, x, w, splits, partial, counters, self.status)
            return out
        self.cublas.gemm_bf16(out, x, w)
        return out

    def gated_up(self, act: torch.Tensor, x: torch.Tensor, w: torch.Tensor, block: int) -> torch.Tensor:
        """act[M, F] = silu(x Wg^T) * (x Wu^T) for the merged weight w [2F, K] (``block``: see kernels.silu_mul).

        A few tokens in bfloat16 with the blocked layout: one kernel (the activation is the product's
        epilogue).  Otherwise the product into scratch and the activation kernel."""
        un = x if isinstance(x, UnscaledRows) else None
        if un is not None:
            x = un.x
        M, K = x.shape
        N = w.shape[0]
        if (self.dtype == torch.bfloat16 and block == kernels.SWIGLU_BLOCK and M <= kernels.SKINNY_MAX_ROWS
                and kernels.gemm_tc_fits(K, x, w) and -(-N // 128) >= self.sm_count
                and kernels.gemm_tc_splits(M, N, K) == 1):
            if un is not None:
                kernels.gemm_tc_swiglu_scaled_bf16(act, x, w, *un.scale, status=self.status)
            else:
                kernels.gemm_tc_swiglu_bf16(act, x, w, self.status)
            return act
        if (self.dtype == torch.bfloat16 and block == kernels.SWIGLU_BLOCK and M <= kernels.FEWROWS_MAX_ROWS
                and K >= kernels.FEWROWS_MIN_K and N % 128 == 0 and kernels.gemm_fewrows_fits(M, K, x, w)
                and -(-N // 128) < self.sm_count):
            if un is not None:
                kernels.gemm_fewrows_norm_bf16(act, x, w, swiglu=True, scale=un.scale, status=self.status)
            else:
                kernels.gemm_fewrows_bf16(act, x, w, swiglu=True, status=self.status)
            return act
        if un is not None:   # no kernel below takes such rows
            x = un.finish()
        if (self.dtype == torch.bfloat16 and block == kernels.SWIGLU_BLOCK and M >= kernels.PAIR_SWIGLU_MIN_ROWS
                and N % 128 == 0 and kernels.gemm_tc_fits(K, x, w)):
            # many tokens: the tcgen05 product on pairs of SMs with the activation as its epilogue (level with the
            # library's product by itself, ahead once the activation's own pass over gate|up is gone)
            kernels.gemm_tc_pair_bf16(act, x, w, swiglu=True, status=self.status)
            return act
        gu = self.scratch.get("ffn_gate_up", (self.max_tokens, N), self.dtype)[:M]
        self.linear(gu, x, w)
        kernels.silu_mul(act, gu, block)
        return act

    def check_status(self) -> None:
        """Reads the status word (synchronises) and raises if a kernel reported a bad index."""
        word = int(self.status.item())
        if word:
            self.status.zero_()
            raise DeviceFault("a kernel reported " + kernels.status_message(word))
