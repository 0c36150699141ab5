"""Grouped-query attention over a paged cache.

  [q|k|v] = x W_qkv^T (no bias); optional per-head RMSNorm of q and k over the
  head axis, before the rotation; rotate-half position encoding of q and k; k
  (rotated) and v go to the cache; q head h reads kv head h / (nq / nkv);
  s = q.k / sqrt(hd), causal (optionally windowed) softmax, o = P v; a = o W_o^T
  (7QiC/ccInfer: src/model/qwen3/qwen3_model.cpp:158-298).

The three projections are one merged matrix (rows q, then k, then v), as the
reference merges them at load (src/model/qwen3/qwen3_weights.cpp:16-43).  A
layer that reads another layer's cache (``own_kv=False``) has only the q and
o projections (and must use the position encoding of the layer whose keys it
reads).  Head sizes are multiples of 16 up to 256: others are refused (the
reference's decode kernel takes any head size up to 128,
src/kernel/attention/decode_attn.cu:521-569).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels
from ..errors import Unsupported
from .base import CacheNeed, Mixer, PositionEncoding, TensorSpec


class GroupedQueryAttention(Mixer):
    takes_unscaled = True

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PositionEncoding, names: dict, qk_norm_eps: Optional[float] = None,
                 window: Optional[int] = None, own_kv: bool = True, scale: Optional[float] = None):
        """``names``: tensor names under the keys q, k, v, o and (with qk_norm_eps) q_norm, k_norm."""
        if num_heads % num_kv_heads:
            raise Unsupported(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        if head_dim % 16 or head_dim > 256:
            raise Unsupported(f"head size {head_dim}: the attention kernels take multiples of 16 up to 256")
        if window is not None and window <= 0:
            raise Unsupported("a window must be > 0")
        self.hidden, self.nq, self.nkv, self.hd = int(hidden), int(num_heads), int(num_kv_heads), int(head_dim)
        self.position, self.names = position, dict(names)
        self.qk_norm_eps, self.window, self.own_kv = qk_norm_eps, window, own_kv
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.q_width, self.kv_width = self.nq * self.hd, self.nkv * self.hd
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None
        self.rt = None

    # -- what it wants ---------------------------------------------------------
    def tensor_specs(self):
        n, D = self.names, self.hidden
        specs = [TensorSpec(n["q"], (self.q_width, D)), TensorSpec(n["o"], (D, self.q_width))]
        if self.own_kv:
            specs += [TensorSpec(n["k"], (self.kv_width, D)), TensorSpec(n["v"], (self.kv_width, D))]
        if self.qk_norm_eps is not None:
            specs.append(TensorSpec(n["q_norm"], (self.hd,), role="vector", init="one_plus_normal"))
            if self.own_kv:
                specs.append(TensorSpec(n["k_norm"], (self.hd,), role="vector", init="one_plus_normal"))
        return specs

    def cache_need(self):
        return CacheNeed.keys_and_values(self.nkv, self.hd, self.window)

    def bind(self, rt, fetch):
        self.rt = rt
        n = self.names
        self.position.bind(rt, fetch)
        if self.position.score_bias() is not None:
            raise Unsupported("a position encoding that adds to the scores: the attention kernels take rotations "
                              "of q and k only")
        table = self.position.rotary_table()
        if table is not None and (table.dtype != torch.float32 or table.numel() != self.hd // 2):
            raise Unsupported(f"a rotary table of {self.hd // 2} float frequencies is wanted for head size "
                              f"{self.hd}, the position encoding gives {tuple(table.shape)} {table.dtype}")
        # the encoding's own pairing of coordinates, brought into the kernels' layout (pairs (j, j + hd / 2))
        # by permuting the rows of the query and key projections and the head norms' weights alike
        perm = self.position.head_permutation()
        if perm is not None:
            if sorted(perm) != list(range(self.hd)):
                raise Unsupported(f"head_permutation() must name each of the {self.hd} coordinates once")
            idx = torch.tensor(perm, device=rt.device)

            def heads(w, n_heads):
                return w.view(n_heads, self.hd, -1)[:, idx, :].reshape(n_heads * self.hd, -1)
        else:
            idx = None

            def heads(w, n_heads):
                return w
        if self.own_kv:
            self.w_qkv = torch.cat([heads(fetch(n["q"]), self.nq), heads(fetch(n["k"]), self.nkv), fetch(n["v"])],
                                   dim=0).contiguous()
        else:
            self.w_qkv = heads(fetch(n["q"]), self.nq).contiguous()
        self.w_o = fetch(n["o"])
        if self.qk_norm_eps is not None:
            self.q_norm_w = fetch(n["q_norm"])
            self.k_norm_w = fetch(n["k_norm"]) if self.own_kv else None
            if idx is not None:
                self.q_norm_w = self.q_norm_w[idx].contiguous()
                self.k_norm_w = self.k_norm_w[idx].contiguous() if self.k_norm_w is not None else None

    def _attend(self, q, o, cache, step, T):
        """Attention of every token row of the step over its request's pages.

        A step lists its single-token requests first.  On the tensor-core path (bfloat16, head size 64 or
        128) those rows go to the decode kernel (key range split over blocks) and the portions of prompts to
        a prefill kernel (tcgen05 with 128 query tokens a block, or mma.sync with 64); otherwise every row is
        a single query of the split kernel, which takes all sizes and both types."""
        rt, g = self.rt, cache.group
        mma = rt.dtype == torch.bfloat16 and self.hd in kernels.DECODE_MMA_HEAD_SIZES
        n_rows = step.n_single if mma else T
        if n_rows > 0:
            per_block = kernels.DECODE_MMA_HEADS_PER_BLOCK if mma else 0
            splits, n_acc, n_ml = kernels.attention_split_plan(n_rows, self.nq, self.nkv, self.hd, per_block)
            part_acc = rt.scratch.get("attn_part_acc", (n_acc,), torch.float32)
            part_ml = rt.scratch.get("attn_part_ml", (n_ml,), torch.float32)
            args = (q, cache.k, cache.v, o, part_acc, part_ml, step.positions, step.entry_of_token, g.block_table,
                    step.n_entries, 0, n_rows, self.window or 0, self.scale, splits)
            if mma and kernels.attention_decode_tma_fits(self.hd, g.page_size):
                # pages arrive as TMA boxes.  Many splits (few rows, long contexts): the last block of a row
                # and head group merges them; few splits: a second small kernel does, during which the
                # output projection already loads its first weights (measured: 2 us a layer either way)
                kernels.attention_decode_tma(*args, status=rt.status,
                                             merge_counters=rt.merge_counters if splits >= self.MERGE_IN_KERNEL_MIN_SPLITS else None)
            else:
                fn = kernels.attention_decode_mma if mma else kernels.attention_split
                fn(*args, status=rt.status)
        if mma and step.n_entries > step.n_single:
            # long portions: 128-token tiles on tcgen05 with the accumulators in tensor memory; short ones
            # (and page sizes a TMA box cannot take): 64-token tiles on mma.sync
            tc = step.max_q_len > 64 and kernels.attention_prefill_tc_fits(self.hd, g.page_size)
            fn = kernels.attention_prefill_tc if tc else kernels.attention_prefill_mma
            fn(q, cache.k, cache.v, o, step.cu_q, step.pos0, g.block_table, step.n_single,
               step.n_entries - step.n_single, step.max_q_len, self.window or 0, self.scale, status=rt.status)

    MERGE_IN_KERNEL_MIN_SPLITS = 8   # from here on the block that finishes last merges the splits itself
    FUSED_DECODE_MAX_ROWS = 48   # measured: 1.3-2.3 us a layer faster up to 32 rows, 1.6 us slower at 64

    def _fused_decode(self, step, g) -> bool:
        """A step of single tokens only, on the path of the TMA decode kernel (bfloat16, head size 64 or 128,
        a page size it takes), with few enough rows that every block redoing the queries' norm and rotation
        costs less than a kernel of its own."""
        return (self.rt.dtype == torch.bfloat16 and self.hd in kernels.DECODE_MMA_HEAD_SIZES
                and kernels.attention_decode_tma_fits(self.hd, g.page_size)
                and step.n_single == step.n_entries == step.n_tokens
                and step.n_tokens <= self.FUSED_DECODE_MAX_ROWS)

    # -- a step ----------------------------------------------------------------
    def forward(self, x, step, cache, state):
        rt = self.rt
        T = x.shape[0]
        nkv_w = self.nkv if self.own_kv else 0
        width = self.q_width + 2 * nkv_w * self.hd
        qkv = rt.scratch.get("attn_qkv", (rt.max_tokens, width), rt.dtype)[:T]
        rt.linear(qkv, x, self.w_qkv)
        g = cache.group
        o = rt.scratch.get("attn_o", (rt.max_tokens, self.nq, self.hd), rt.dtype)[:T]
        if self._fused_decode(step, g):
            # every row brings one token: the decode attention norms and rotates the queries itself, writes
            # the row's key and value to their page and attends to them: one kernel less in every layer
            splits, n_acc, n_ml = kernels.attention_split_plan(T, self.nq, self.nkv, self.hd,
                                                               kernels.DECODE_MMA_HEADS_PER_BLOCK)
            kernels.attention_decode_tma_fused(
                qkv, cache.k, cache.v, o, rt.scratch.get("attn_part_acc", (n_acc,), torch.float32),
                rt.scratch.get("attn_part_ml", (n_ml,), torch.float32), step.positions, step.entry_of_token,
                g.block_table, step.n_entries, 0, T, self.nq, self.window or 0, self.scale, splits,
                self.q_norm_w, self.k_norm_w, self.qk_norm_eps if self.qk_norm_eps is not None else 1.0,
                self.position.rotary_table(), write_kv=self.own_kv, status=rt.status,
                merge_counters=rt.merge_counters if splits >= self.MERGE_IN_KERNEL_MIN_SPLITS else None)
        else:
            q = rt.scratch.get("attn_q", (rt.max_tokens, self.nq, self.hd), rt.dtype)[:T]
            kernels.qk_norm_rope_kv_write(
                qkv, q, cache.k if self.own_kv else None, cache.v if self.own_kv else None, step.positions,
                g.slot_map if self.own_kv else None, self.position.rotary_table(), self.q_norm_w, self.k_norm_w,
                self.qk_norm_eps if self.qk_norm_eps is not None else 1.0, self.nq, nkv_w, self.hd, g.page_size,
                status=rt.status)
            self._attend(q, o, cache, step, T)
        out = rt.scratch.get("attn_out", (rt.max_tokens, self.hidden), rt.dtype)[:T]
        return rt.linear(out, o.view(T, self.q_width), self.w_o, sink=step.take_sink())
