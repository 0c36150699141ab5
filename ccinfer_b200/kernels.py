"""Python face of the CUDA kernels: one function per launcher of ``csrc``.

The shared object is loaded with ctypes; tensors are passed as raw device
pointers and every launch goes to torch's current CUDA stream, so the kernels
take part in stream capture like any other work.  A launcher that refuses its
arguments or whose launch fails raises; nothing falls back to another
implementation.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_size_t, c_void_p

import torch

from .csrc import build as _build
from .errors import ExtensionMissing, InvalidArgument, Unsupported

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

ST_BAD_TOKEN, ST_BAD_SLOT, ST_BAD_PAGE, ST_BAD_ROW, ST_WAIT_TIMEOUT = 1, 2, 4, 8, 16
STATUS_TEXT = {
    ST_BAD_TOKEN: "a token id outside the vocabulary",
    ST_BAD_SLOT: "a cache slot outside the pool",
    ST_BAD_PAGE: "a block-table entry outside the pool where a key was needed",
    ST_BAD_ROW: "a row index outside the batch",
    ST_WAIT_TIMEOUT: "a bounded wait inside a kernel gave up",
}

_lock = threading.Lock()
_libs = {}

_SIGNATURES = {
    "ccb_embed_gather": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                         c_void_p],
    "ccb_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "ccb_gemm_tc_swiglu_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                c_void_p],
    "ccb_gemm_fewrows_set_stages": [c_int],
    "ccb_gemm_fewrows_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_void_p, c_void_p],
    "ccb_gemm_fewrows_blocks": [c_int],
    "ccb_gemm_fewrows_norm_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_void_p, c_int, c_float, c_float, c_void_p, c_int, c_void_p, c_void_p,
                                   c_void_p, c_void_p],
    "ccb_gemm_tc_swiglu_scaled_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_void_p, c_int, c_float, c_float, c_void_p, c_void_p],
    "ccb_residual_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                             c_int, c_void_p, c_void_p],
    "ccb_embed_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int,
                          c_void_p, c_int, c_void_p, c_void_p],
    "ccb_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    "ccb_qk_norm_rope_kv_write": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_void_p, c_void_p],
    "ccb_paged_attention_generic": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                    c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                    c_void_p, c_void_p],
    "ccb_attention_split": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                            c_int, c_void_p, c_void_p],
    "ccb_attention_decode_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_float, c_int, c_void_p, c_void_p],
    "ccb_attention_decode_tma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_float, c_int, c_void_p, c_void_p, c_void_p],
    "ccb_attention_decode_tma_fused": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_float, c_void_p, c_int,
                                       c_void_p, c_void_p, c_void_p],
    "ccb_attention_prefill_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                  c_void_p],
    "ccb_attention_prefill_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                 c_void_p],
    "ccb_gemm_f32": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "ccb_cublas_create": [ctypes.POINTER(c_void_p)],
    "ccb_cublas_destroy": [c_void_p],
    "ccb_cublas_set_workspace": [c_void_p, c_void_p, c_size_t],
    "ccb_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_void_p],
    "ccb_gemm_skinny_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_void_p],
    "ccb_gemm_tc_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_void_p, c_void_p, c_void_p, c_void_p],
    "ccb_gemm_tc_pair_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_void_p, c_void_p],
    "ccb_init_random": [c_void_p, c_longlong, c_int, ctypes.c_ulonglong, ctypes.c_ulonglong, c_float, c_int, c_void_p],
    "ccb_sample_rows": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                        c_int, c_void_p, c_void_p, c_int, c_void_p],
}


def lib(group: str = "core"):
    """The loaded shared object of a kernel group (built at the first call)."""
    with _lock:
        if group in _libs:
            return _libs[group]
        path = _build.library_path(group)
        try:
            handle = ctypes.CDLL(path)
        except OSError as e:
            raise ExtensionMissing(f"cannot load {path}: {e}") from e
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is not None:
                fn.argtypes = argtypes
                fn.restype = c_int
        _libs[group] = handle
        return handle


def set_pdl(on) -> None:
    """Launch the library's kernels so that each may start while its predecessor finishes (programmatic
    dependent launch); every kernel waits for its predecessor before it reads what that one wrote."""
    fn = lib().ccb_set_pdl
    fn.argtypes = [c_int]
    fn.restype = c_int
    fn(int(on))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class _Counters:
    """Launches since import: ``own`` = kernels of this package, ``library`` = cuBLAS products."""
    own = 0
    library = 0


counters = _Counters()


def _check(code: int, what: str) -> None:
    if code == 0:
        if what == "gemm_bf16":
            counters.library += 1
        elif not what.startswith("cublas"):
            counters.own += 1
        return
    if code == -2:
        raise Unsupported(f"{what}: a size outside what the kernel takes")
    if code == -3:
        raise Unsupported(f"{what}: element type not supported")
    if code == -4:
        raise InvalidArgument(f"{what}: a required argument is missing")
    if code >= 1000:
        raise RuntimeError(f"{what}: cuBLAS status {code - 1000}")
    raise RuntimeError(f"{what}: CUDA error {code}")


def _p(t):
    return 0 if t is None else t.data_ptr()


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise Unsupported(f"element type {t.dtype} is not supported by the kernels") from None


def _cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise InvalidArgument("kernels take contiguous CUDA tensors")


def status_message(word: int) -> str:
    return "; ".join(text for bit, text in STATUS_TEXT.items() if word & bit) or "no fault"


# ---------------------------------------------------------------------------------------------
def embed_gather(h: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, status=None, pending=None) -> None:
    """h[t, :] = float(table[ids[t], :]); h is the float residual stream [T, D].

    With ``pending`` (int32 [slots]) an id of -1 - s stands for pending[s]: the token that sample_rows
    last stored for request slot s."""
    _cuda(h, table, ids, status, pending)
    T, D = h.shape
    assert h.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == D and ids.numel() >= T
    assert pending is None or pending.dtype == torch.int32
    _check(lib().ccb_embed_gather(_p(h), _p(table), _p(ids), T, D, table.shape[0], _dt(table), _p(pending),
                                  0 if pending is None else pending.numel(), _p(status), _stream()), "embed_gather")


def embed_rmsnorm(y, h, table, ids, w, eps: float, status=None, pending=None) -> None:
    """embed_gather and the norm of the rows it wrote in one pass: h[t, :] = float(table[ids[t], :]) and
    y[t, :] = RMSNorm(h[t, :]) * w (y and table in the storage type, w float)."""
    _cuda(y, h, table, ids, w, status, pending)
    T, D = h.shape
    assert h.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == D and ids.numel() >= T
    assert y.shape == (T, D) and y.dtype == table.dtype and w.dtype == torch.float32 and w.numel() == D
    assert h.is_contiguous() and y.is_contiguous() and table.is_contiguous()
    assert pending is None or pending.dtype == torch.int32
    _check(lib().ccb_embed_rmsnorm(_p(y), _p(h), _p(table), _p(ids), _p(w), T, D, table.shape[0], float(eps),
                                   _dt(table), _p(pending), 0 if pending is None else pending.numel(), _p(status),
                                   _stream()), "embed_rmsnorm")


def silu_mul(act: torch.Tensor, gate_up: torch.Tensor, block: int = 0) -> None:
    """act[t, f] = silu(gate[t, f]) * up[t, f] for gate_up[t, :] = [all gate | all up] (block = 0) or in
    blocks of ``block`` gate columns followed by the ``block`` up columns of the same channels."""
    _cuda(act, gate_up)
    T, F = act.shape
    assert gate_up.shape == (T, 2 * F) and act.dtype == gate_up.dtype
    _check(lib().ccb_silu_mul(_p(act), _p(gate_up), T, F, int(block), _dt(act), _stream()), "silu_mul")


SWIGLU_BLOCK = 64   # rows of gate, then of up, in a weight matrix laid out for gemm_tc_swiglu_bf16


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int) -> torch.Tensor:
    """[2F, D]: ``block`` rows of gate, the ``block`` rows of up for the same channels, and so on."""
    F, D = gate.shape
    assert up.shape == (F, D) and F % block == 0
    return torch.cat([gate.view(F // block, block, D), up.view(F // block, block, D)], dim=1).reshape(2 * F, D).contiguous()


def gemm_tc_swiglu_bf16(act, a, w, status=None) -> None:
    """act[M, F] = silu(a Wg^T) * (a Wu^T) in one tensor-core kernel; w [2F, K] interleaved in blocks of
    SWIGLU_BLOCK rows (interleave_gate_up), M <= 16, F a multiple of 64."""
    _cuda(act, a, w, status)
    assert act.dtype == a.dtype == w.dtype == torch.bfloat16
    M, K = a.shape
    F = w.shape[0] // 2
    assert w.shape == (2 * F, K) and act.shape == (M, F) and a.stride(1) == w.stride(1) == act.stride(1) == 1
    _check(lib().ccb_gemm_tc_swiglu_bf16(_p(act), _p(a), _p(w), M, F, K, a.stride(0), w.stride(0), act.stride(0),
                                         _p(status), _stream()), "gemm_tc_swiglu_bf16")


def gemm_tc_swiglu_scaled_bf16(act, a, w, ssq, parts: int, dim: int, eps: float, status=None) -> None:
    """gemm_tc_swiglu_bf16 whose token rows still lack the factor of their RMSNorm: token t of both products is
    multiplied by 1 / sqrt(sum_p ssq[t, p] / dim + eps) before the activation (ssq float [16, parts])."""
    _cuda(act, a, w, ssq, status)
    assert act.dtype == a.dtype == w.dtype == torch.bfloat16 and ssq.dtype == torch.float32
    M, K = a.shape
    F = w.shape[0] // 2
    assert w.shape == (2 * F, K) and act.shape == (M, F) and a.stride(1) == w.stride(1) == act.stride(1) == 1
    assert ssq.is_contiguous() and ssq.numel() >= parts * 16
    _check(lib().ccb_gemm_tc_swiglu_scaled_bf16(_p(act), _p(a), _p(w), M, F, K, a.stride(0), w.stride(0),
                                                act.stride(0), _p(ssq), int(parts), float(dim), float(eps),
                                                _p(status), _stream()), "gemm_tc_swiglu_scaled_bf16")


def residual_rmsnorm(y, h, delta, w, eps: float, row_idx=None, n_rows=None, status=None) -> None:
    """y = RMSNorm(h + delta) * w, and h <- h + delta when no rows are picked.

    h float [T, D]; delta (optional) and y in the storage type; w float [D].
    With ``row_idx`` (int32 [R]) only those rows of h are normed, into y [R, D].
    """
    _cuda(y, h, delta, w, row_idx, status)
    D = h.shape[1]
    rows = y.shape[0] if n_rows is None else n_rows
    assert h.dtype == torch.float32 and w.dtype == torch.float32 and w.numel() == D and y.shape[1] == D
    assert delta is None or (delta.dtype == y.dtype and delta.shape[1] == D)
    _check(lib().ccb_residual_rmsnorm(_p(y), _p(h), _p(delta), _p(w), _p(row_idx), rows, h.shape[0], D,
                                      float(eps), _dt(y), _p(status), _stream()), "residual_rmsnorm")


def rmsnorm(y, x, w, eps: float) -> None:
    """Plain RMSNorm over the last axis of a contiguous tensor; w float."""
    _cuda(y, x, w)
    D = x.shape[-1]
    assert w.dtype == torch.float32 and w.numel() == D and y.dtype == x.dtype and y.shape == x.shape
    _check(lib().ccb_rmsnorm(_p(y), _p(x), _p(w), x.numel() // D, D, float(eps), _dt(x), _stream()), "rmsnorm")


def qk_norm_rope_kv_write(qkv, q_out, k_cache, v_cache, positions, slot_map, inv_freq, q_w, k_w, eps,
                          nq: int, nkv: int, hd: int, page_size: int, status=None) -> None:
    """Head norms, rotation and cache write in one pass over qkv [T, (nq + 2 nkv) hd].

    q goes to q_out [T, nq, hd]; k and v go to their caches [pages, nkv, page, hd]
    at slot_map[t] (a negative slot skips the write).  inv_freq, q_w, k_w may
    be None to leave that step out; nkv = 0 handles q alone.
    """
    _cuda(qkv, q_out, k_cache, v_cache, positions, slot_map, inv_freq, q_w, k_w, status)
    T = q_out.shape[0]
    assert qkv.shape[0] >= T and qkv.shape[1] >= (nq + 2 * nkv) * hd and qkv.dtype == q_out.dtype
    num_slots = 0
    if nkv > 0:
        assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
        assert k_cache.shape[1:] == (nkv, page_size, hd) and v_cache.shape == k_cache.shape
        num_slots = k_cache.shape[0] * page_size
    _check(lib().ccb_qk_norm_rope_kv_write(_p(qkv), qkv.stride(0), _p(q_out), _p(k_cache), _p(v_cache),
                                           _p(positions), _p(slot_map), _p(inv_freq), _p(q_w), _p(k_w),
                                           float(eps), T, nq, nkv, hd, page_size, num_slots, _dt(qkv),
                                           _p(status), _stream()), "qk_norm_rope_kv_write")


def paged_attention_generic(q, k_cache, v_cache, out, positions, entry_of_token, block_table, n_entries: int,
                            window: int, scale: float, status=None) -> None:
    """Causal attention of q [T, nq, hd] over paged caches [pages, nkv, page, hd].

    Token t belongs to request row entry_of_token[t] of block_table [B, stride]
    and sits at absolute position positions[t]; window <= 0 means all keys.
    """
    _cuda(q, k_cache, v_cache, out, positions, entry_of_token, block_table, status)
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    assert hd2 == hd and out.shape == q.shape and q.dtype == k_cache.dtype == v_cache.dtype == out.dtype
    _check(lib().ccb_paged_attention_generic(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(positions),
                                             _p(entry_of_token), _p(block_table), block_table.stride(0),
                                             n_entries, T, nq, nkv, hd, page_size, num_pages, int(window),
                                             float(scale), _dt(q), _p(status), _stream()),
           "paged_attention_generic")


B200_SM_COUNT = 148
_sm_count = None


def sm_count() -> int:
    """SMs of the current CUDA device, asked once.  Without a device: a B200's number, so that the rules
    that size grids can be tabulated on a CPU."""
    global _sm_count
    if _sm_count is None:
        if not torch.cuda.is_available():
            return B200_SM_COUNT
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def split_target_blocks() -> int:
    """Blocks the split attention kernels aim for: two per SM."""
    return 2 * sm_count()


SPLIT_MAX = 32


def attention_split_heads_per_block(nq: int, nkv: int, hd: int) -> int:
    g = nq // nkv
    return 4 if (g >= 4 and hd <= 128) else (2 if g >= 2 else 1)


def attention_split_plan(n_rows: int, nq: int, nkv: int, hd: int, heads_per_block: int = 0):
    """(num_splits, scratch floats for the accumulators, scratch floats for max and sum).

    The number of splits depends on the number of token rows only, so a step of a given size always
    launches the same grid (and its results do not depend on the lengths in the batch)."""
    gt = heads_per_block or attention_split_heads_per_block(nq, nkv, hd)
    per_split = n_rows * nkv * -(-(nq // nkv) // gt)
    target = split_target_blocks()
    splits = max(1, min(SPLIT_MAX, target // max(1, per_split)))
    return splits, target * gt * hd, target * gt * 2


def attention_split(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table,
                    n_entries: int, row0: int, n_rows: int, window: int, scale: float, num_splits: int,
                    status=None) -> None:
    """Attention of the token rows row0 .. row0 + n_rows - 1, each a single query with its own position
    and request; the key range is cut into ``num_splits`` pieces merged afterwards (scratch from
    ``attention_split_plan``; unused with one split)."""
    _cuda(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table, status)
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    assert hd2 == hd and out.shape == q.shape and q.dtype == k_cache.dtype == v_cache.dtype == out.dtype
    assert 0 <= row0 and row0 + n_rows <= T
    if num_splits > 1:
        assert part_acc.dtype == part_ml.dtype == torch.float32
        assert part_acc.numel() >= n_rows * nq * num_splits * hd and part_ml.numel() >= n_rows * nq * num_splits * 2
    _check(lib().ccb_attention_split(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(part_acc), _p(part_ml),
                                     _p(positions), _p(entry_of_token), _p(block_table), block_table.stride(0),
                                     n_entries, row0, n_rows, nq, nkv, hd, page_size, num_pages, int(window),
                                     float(scale), num_splits, _dt(q), _p(status), _stream()), "attention_split")
    if num_splits > 1:
        counters.own += 1  # the merge kernel


DECODE_MMA_HEAD_SIZES = (64, 128)
DECODE_MMA_HEADS_PER_BLOCK = 16


def attention_decode_mma(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table,
                         n_entries: int, row0: int, n_rows: int, window: int, scale: float, num_splits: int,
                         status=None) -> None:
    """As attention_split, on tensor cores: bfloat16, head size 64 or 128, a block per (row, kv head, split)
    serving the whole group of q heads."""
    _cuda(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table, status)
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    assert hd2 == hd and out.shape == q.shape
    assert q.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16
    assert 0 <= row0 and row0 + n_rows <= T
    if num_splits > 1:
        assert part_acc.dtype == part_ml.dtype == torch.float32
        assert part_acc.numel() >= n_rows * nq * num_splits * hd and part_ml.numel() >= n_rows * nq * num_splits * 2
    _check(lib().ccb_attention_decode_mma(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(part_acc), _p(part_ml),
                                          _p(positions), _p(entry_of_token), _p(block_table),
                                          block_table.stride(0), n_entries, row0, n_rows, nq, nkv, hd, page_size,
                                          num_pages, int(window), float(scale), num_splits, _p(status),
                                          _stream()), "attention_decode_mma")
    if num_splits > 1:
        counters.own += 1  # the merge kernel


def attention_decode_tma_fits(hd: int, page_size: int) -> bool:
    return hd in DECODE_MMA_HEAD_SIZES and 8 <= page_size <= 64 and page_size & (page_size - 1) == 0


def attention_decode_tma(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table,
                         n_entries: int, row0: int, n_rows: int, window: int, scale: float, num_splits: int,
                         status=None, merge_counters=None) -> None:
    """As attention_decode_mma, with keys and values loaded page by page through TMA boxes by a producer warp
    (page size a power of two from 8 to 64).

    ``merge_counters`` (int32 zeros, left zero): with them the block that finishes last merges the splits
    of its row and head group; without them (or where they are too few) a second kernel does."""
    _cuda(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table, status, merge_counters)
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    assert hd2 == hd and out.shape == q.shape
    assert q.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16
    assert 0 <= row0 and row0 + n_rows <= T
    if num_splits > 1:
        assert part_acc.dtype == part_ml.dtype == torch.float32
        assert part_acc.numel() >= n_rows * nq * num_splits * hd and part_ml.numel() >= n_rows * nq * num_splits * 2
    if merge_counters is not None:
        groups = nkv * -(-(nq // nkv) // DECODE_MMA_HEADS_PER_BLOCK)
        if num_splits == 1 or merge_counters.numel() < n_rows * groups:
            merge_counters = None
        else:
            assert merge_counters.dtype == torch.int32
    _check(lib().ccb_attention_decode_tma(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(part_acc), _p(part_ml),
                                          _p(positions), _p(entry_of_token), _p(block_table),
                                          block_table.stride(0), n_entries, row0, n_rows, nq, nkv, hd, page_size,
                                          num_pages, int(window), float(scale), num_splits, _p(merge_counters),
                                          _p(status), _stream()), "attention_decode_tma")
    if num_splits > 1 and merge_counters is None:
        counters.own += 1  # the merge kernel


def attention_prefill_mma(q, k_cache, v_cache, out, cu_q, pos0, block_table, entry0: int, n_entries: int,
                          max_new: int, window: int, scale: float, status=None) -> None:
    """Causal attention of the new tokens of the step's requests entry0 .. entry0 + n_entries - 1 over their
    pages, on tensor cores (bfloat16, head size 64 or 128).  cu_q [B + 1] gives each request's first token
    row, pos0 [B] the position of that token; max_new is the most new tokens any of them has."""
    _cuda(q, k_cache, v_cache, out, cu_q, pos0, block_table, status)
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    assert hd2 == hd and out.shape == q.shape
    assert q.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16
    assert entry0 >= 0 and entry0 + n_entries <= block_table.shape[0] and cu_q.numel() >= entry0 + n_entries + 1
    _check(lib().ccb_attention_prefill_mma(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(cu_q), _p(pos0),
                                           _p(block_table), block_table.stride(0), entry0, n_entries, max_new,
                                           nq, nkv, hd, page_size, num_pages, int(window), float(scale),
                                           _p(status), _stream()), "attention_prefill_mma")


def attention_decode_tma_fused(qkv, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token,
                               block_table, n_entries: int, row0: int, n_rows: int, nq: int, window: int,
                               scale: float, num_splits: int, q_norm_w, k_norm_w, eps: float, inv_freq,
                               write_kv: bool = True, status=None, merge_counters=None) -> None:
    """attention_decode_tma for rows of ONE new token each, straight from the q|k|v product ``qkv``
    [T, (nq + 2 nkv) * hd] (only the nq query heads when ``write_kv`` is false): the kernel norms and rotates
    the queries itself and, with ``write_kv``, also the row's key, which it writes with the value to their
    page and attends to.  qk_norm_rope_kv_write is not needed for these rows."""
    _cuda(qkv, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table, status,
          merge_counters, q_norm_w, k_norm_w, inv_freq)
    T = qkv.shape[0]
    num_pages, nkv, page_size, hd = k_cache.shape
    assert out.shape == (T, nq, hd) and qkv.stride(1) == 1
    assert qkv.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16
    assert all(w is None or (w.dtype == torch.float32 and w.numel() >= n) for w, n in
               ((q_norm_w, hd), (k_norm_w, hd), (inv_freq, hd // 2)))
    assert 0 <= row0 and row0 + n_rows <= T
    if num_splits > 1:
        assert part_acc.dtype == part_ml.dtype == torch.float32
        assert part_acc.numel() >= n_rows * nq * num_splits * hd and part_ml.numel() >= n_rows * nq * num_splits * 2
    if merge_counters is not None:
        groups = nkv * -(-(nq // nkv) // DECODE_MMA_HEADS_PER_BLOCK)
        if num_splits == 1 or merge_counters.numel() < n_rows * groups:
            merge_counters = None
    _check(lib().ccb_attention_decode_tma_fused(
        _p(qkv), qkv.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(part_acc), _p(part_ml), _p(positions),
        _p(entry_of_token), _p(block_table), block_table.stride(0), n_entries, row0, n_rows, nq, nkv, hd, page_size,
        num_pages, int(window), float(scale), num_splits, _p(q_norm_w), _p(k_norm_w), float(eps), _p(inv_freq),
        1 if write_kv else 0, _p(merge_counters), _p(status), _stream()), "attention_decode_tma_fused")
    if num_splits > 1 and merge_counters is None:
        counters.own += 1  # the merge kernel


def attention_prefill_tc_fits(hd: int, page_size: int) -> bool:
    return hd in (64, 128) and 8 <= page_size <= 128 and page_size & (page_size - 1) == 0


def attention_prefill_tc(q, k_cache, v_cache, out, cu_q, pos0, block_table, entry0: int, n_entries: int,
                         max_new: int, window: int, scale: float, status=None) -> None:
    """As attention_prefill_mma, with both products on tcgen05 tensor cores and the accumulators in tensor
    memory (128-token query tiles, TMA loads page by page).  Page size a power of two from 8 to 128.  Where the
    groups hold an even number of q heads, two heads of a group share a block and its key and value tiles."""
    _cuda(q, k_cache, v_cache, out, cu_q, pos0, block_table, status)
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    assert hd2 == hd and out.shape == q.shape
    assert q.dtype == k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16
    assert entry0 >= 0 and entry0 + n_entries <= block_table.shape[0] and cu_q.numel() >= entry0 + n_entries + 1
    _check(lib().ccb_attention_prefill_tc(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(cu_q), _p(pos0),
                                          _p(block_table), block_table.stride(0), entry0, n_entries, max_new, T,
                                          nq, nkv, hd, page_size, num_pages, int(window), float(scale),
                                          _p(status), _stream()), "attention_prefill_tc")


def attention_prefill_tc_single_head(on: bool) -> None:
    """Measurements and tests: with ``on`` attention_prefill_tc always runs one q head per block, also where two
    heads of a kv group would share a block (and its key and value tiles)."""
    fn = lib().ccb_attention_prefill_tc_single_head
    fn.argtypes = [c_int]
    fn.restype = c_int
    fn(1 if on else 0)


def gemm_f32(c, a, w) -> None:
    """c[M, N] = a[M, K] @ w[N, K]^T in true 32-bit arithmetic (row strides may exceed the widths)."""
    assert c.dtype == a.dtype == w.dtype == torch.float32 and c.is_cuda and a.is_cuda and w.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    _check(lib().ccb_gemm_f32(_p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), _stream()),
           "gemm_f32")


SKINNY_MAX_ROWS = 16


def gemm_skinny_fits(M: int, K: int, a, w) -> bool:
    """Whether the few-rows product takes this shape (else the library product does)."""
    return (M <= SKINNY_MAX_ROWS and K % 32 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny_bf16(c, a, w) -> None:
    """c[M, N] (bfloat16 or float) = a[M, K] @ w[N, K]^T for M <= 32, K a multiple of 32 (own kernel)."""
    assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT and c.is_cuda and a.is_cuda and w.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    _check(lib().ccb_gemm_skinny_bf16(_p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0),
                                      _dt(c), _stream()), "gemm_skinny_bf16")


TC_SWAP_MAX_ROWS = 64     # up to here the weights are the 128-row side of the tensor-core tile


def tc_target_blocks() -> int:
    """Blocks a tensor-core product of a few rows aims for: one per SM."""
    return sm_count()



def gemm_tc_fits(K: int, a, w) -> bool:
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    """How many slices of K run as separate blocks (decode shapes only): enough blocks for every SM."""
    if M > TC_SWAP_MAX_ROWS:
        return 1
    tiles = -(-N // 128)
    kb = -(-K // 64)
    s = max(1, min(-(-tc_target_blocks() // tiles), kb // 4, 16))
    while s > 1 and (s - 1) * (-(-kb // s)) >= kb:   # every slice must hold a k block
        s -= 1
    return s


def gemm_tc_bf16(c, a, w, splits: int = 1, partial=None, counters=None, status=None) -> None:
    """c[M, N] (bfloat16 or float) = a[M, K] @ w[N, K]^T on tcgen05 tensor cores with TMA loads.

    M <= 64 streams the weights as the 128-row operand and may cut K into ``splits`` slices
    (``partial``: float scratch of splits * M * N, ``counters``: int32 zeros, one per 128 features)."""
    assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT and c.is_cuda and a.is_cuda and w.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    if splits > 1:
        assert partial.dtype == torch.float32 and partial.numel() >= splits * M * N
        assert counters.dtype == torch.int32 and counters.numel() >= -(-N // 128)
    _check(lib().ccb_gemm_tc_bf16(_p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), _dt(c),
                                  splits, _p(partial), _p(counters), _p(status), _stream()), "gemm_tc_bf16")


def gemm_tc_pair_bf16(c, a, w, swiglu: bool = False, status=None) -> None:
    """c[M, N] (bfloat16 or float) = a[M, K] @ w[N, K]^T for many rows on tcgen05 tensor cores, two SMs on every
    256 x 256 tile (cta_group::2: each SM holds half of both operands, which halves what its shared memory has
    to deliver per product), one cluster per pair of SMs walking over the tiles, two accumulators in tensor
    memory so that a tile's epilogue runs under the next tile's products.  With ``swiglu`` w [2F, K] is
    interleaved in blocks of SWIGLU_BLOCK rows (interleave_gate_up) and c[M, F] = silu(a Wg^T) * (a Wu^T)."""
    _cuda(w, status)
    assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT and c.is_cuda and a.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N // 2 if swiglu else N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    _check(lib().ccb_gemm_tc_pair_bf16(_p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), _dt(c),
                                       1 if swiglu else 0, sm_count(), _p(status), _stream()), "gemm_tc_pair_bf16")


PAIR_SWIGLU_MIN_ROWS = 1024   # from here on gate|up with the activation fused beats the library product + silu_mul


FEWROWS_MAX_ROWS = 16
FEWROWS_MIN_K = 2048      # below, the register-streaming kernel starts up faster


def gemm_fewrows_fits(M: int, K: int, a, w) -> bool:
    return (M <= FEWROWS_MAX_ROWS and K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_fewrows_bf16(c, a, w, swiglu: bool = False, status=None) -> None:
    """c[M, N] (bfloat16 or float) = a[M, K] @ w[N, K]^T for M <= 16: blocks of 16 features over the whole K
    range, weights and tokens through a TMA ring, mma.sync; with ``swiglu`` w [2F, K] is interleaved in blocks
    of SWIGLU_BLOCK rows (interleave_gate_up) and c[M, F] = silu(a Wg^T) * (a Wu^T)."""
    _cuda(w, status)
    assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT and c.is_cuda and a.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N // 2 if swiglu else N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    _check(lib().ccb_gemm_fewrows_bf16(_p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), _dt(c),
                                       1 if swiglu else 0, _p(status), _stream()), "gemm_fewrows_bf16")


def gemm_fewrows_blocks(N: int) -> int:
    """Partial sums per token that gemm_fewrows_norm_bf16 writes when it adds into a residual stream of width N."""
    return int(lib().ccb_gemm_fewrows_blocks(int(N)))


def gemm_fewrows_norm_bf16(c, a, w, swiglu: bool = False, scale=None, into=None, status=None) -> None:
    """gemm_fewrows_bf16 with the halves of an RMSNorm that has no kernel of its own in its epilogue.

    ``scale = (ssq, parts, dim, eps)``: the rows of ``a`` still lack the factor of their norm; token t of the
    result is multiplied by 1 / sqrt(sum_p ssq[t, p] / dim + eps) (before the activation, with ``swiglu``).
    ``into = (h, norm_w, ssq_out)``: h [M, N] (float) += the result; c = bfloat16(h * norm_w); ssq_out
    [16, gemm_fewrows_blocks(N)] gets each block's sum of h^2 per token: what the next product needs as ``scale``."""
    _cuda(w, status)
    assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT and c.is_cuda and a.is_cuda
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N // 2 if swiglu else N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    ssq, parts, dim, eps = scale if scale is not None else (None, 0, 0.0, 0.0)
    h, norm_w, ssq_out = into if into is not None else (None, None, None)
    if ssq is not None:
        assert ssq.dtype == torch.float32 and ssq.is_contiguous() and ssq.numel() >= parts * 16
    if h is not None:
        assert not swiglu and c.dtype == torch.bfloat16 and h.dtype == torch.float32 and h.shape == (M, N)
        assert h.stride(1) == 1 and norm_w.dtype == torch.float32 and norm_w.numel() == N and norm_w.is_contiguous()
        assert ssq_out.dtype == torch.float32 and ssq_out.is_contiguous() and ssq_out.numel() >= gemm_fewrows_blocks(N) * 16
    _check(lib().ccb_gemm_fewrows_norm_bf16(
        _p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), _dt(c), 1 if swiglu else 0,
        _p(ssq), int(parts), float(dim), float(eps), _p(h), h.stride(0) if h is not None else 0, _p(norm_w),
        _p(ssq_out), _p(status), _stream()), "gemm_fewrows_norm_bf16")


def few_rows_product_kernel(M: int, N: int, K: int, sm_count: int, fits_tc: bool, fits_fewrows: bool,
                            fits_skinny: bool) -> str:
    """Which kernel takes out[M, N] = x[M, K] @ w[N, K]^T in bfloat16: "tc", "tc_split", "fewrows", "skinny" or
    "library".  Measured on B200 (graph-timed, weights larger than L2): with up to 16 tokens the tcgen05 kernel
    wins where one block per 128 features fills the machine (gate|up, the vocabulary), the TMA-ring kernel
    with blocks of 16 features on everything smaller from K = 2048 on (q|k|v, o, down).  (For one or two
    tokens it used to have those only where its blocks fit two per SM; since it carries the sum into the
    residual stream and the norm after it in its epilogues, it wins there too: a step of one token at the
    8B / 14B / 32B layer shapes 2.3 / 5.2 / 3.1 % faster.)  What it does not fit goes to the register-streaming
    kernel (short K) or the tcgen05 kernel with K cut into slices (K >= 8192: inside a step the
    register-streaming kernel was 40 us a layer slower there than alone).  More tokens go to the library."""
    if M > SKINNY_MAX_ROWS:
        return "library"
    if fits_tc and -(-N // 128) >= sm_count:
        return "tc"
    if K >= FEWROWS_MIN_K and fits_fewrows:
        return "fewrows"
    if fits_skinny and not (fits_tc and K >= 8192):
        return "skinny"
    if fits_tc:
        return "tc_split"
    return "library"


class CublasHandle:
    """One cuBLAS handle with a caller-owned workspace (no allocation inside a step)."""

    def __init__(self, device, workspace_bytes: int = 64 << 20):
        self._h = c_void_p()
        with torch.cuda.device(device):
            _check(lib().ccb_cublas_create(ctypes.byref(self._h)), "cublas_create")
            self.workspace = torch.empty(workspace_bytes, dtype=torch.uint8, device=device)
            _check(lib().ccb_cublas_set_workspace(self._h, self.workspace.data_ptr(), workspace_bytes),
                   "cublas_set_workspace")

    def gemm_bf16(self, c, a, w) -> None:
        """c[M, N] (bfloat16 or float) = a[M, K] @ w[N, K]^T, bfloat16 operands, float accumulation."""
        assert a.dtype == w.dtype == torch.bfloat16 and c.dtype in _DT
        M, K = a.shape
        N = w.shape[0]
        assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
        _check(lib().ccb_gemm_bf16(self._h, _p(c), _p(a), _p(w), M, N, K, a.stride(0), w.stride(0), c.stride(0),
                                   _dt(c), _stream()), "gemm_bf16")

    def close(self):
        if self._h:
            lib().ccb_cublas_destroy(self._h)
            self._h = c_void_p()


def sample_rows(logits, tokens, temperature=None, seed=None, out_index=None, slot_of_row=None, by_slot=None,
                top_k=None, top_p=None) -> None:
    """tokens[r] = greedy or temperature draw of logits[r, :] (float), per-row parameters.

    temperature float [R] (<= 0 greedy), seed uint32-valued int32/int64 [R] taken
    as 32 bits, out_index int32 [R].  temperature None = greedy for all rows.
    top_k int32 [R] (0 = off) and top_p float [R] (>= 1 = off) restrict a temperature draw to the k largest
    logits and, within those, to the most probable tokens that hold a share p of the probability.
    With ``slot_of_row`` (int32 [R]) the token of row r is also stored in by_slot[slot_of_row[r]]
    (rows with a slot outside by_slot are skipped).
    """
    _cuda(tokens, temperature, seed, out_index, slot_of_row, by_slot, top_k, top_p)
    assert slot_of_row is None or (slot_of_row.dtype == torch.int32 and by_slot.dtype == torch.int32
                                   and slot_of_row.numel() >= logits.shape[0])
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and tokens.dtype == torch.int32
    assert temperature is None or (temperature.dtype == torch.float32 and seed.dtype == torch.int32
                                   and out_index.dtype == torch.int32)
    assert top_k is None or (top_k.dtype == torch.int32 and top_k.numel() >= R)
    assert top_p is None or (top_p.dtype == torch.float32 and top_p.numel() >= R)
    _check(lib().ccb_sample_rows(_p(logits), logits.stride(0), _p(tokens), _p(temperature), _p(seed),
                                 _p(out_index), _p(top_k), _p(top_p), R, V, _p(slot_of_row), _p(by_slot),
                                 0 if by_slot is None else by_slot.numel(), _stream()), "sample_rows")


def init_random(out: torch.Tensor, seed: int, key: int, std: float, add_one: bool = False) -> None:
    """out (float or bfloat16, contiguous) = std * z (+ 1), z ~ N(0, 1) from the counter-based stream of
    (seed, key); the same bits as ``weights.random_init.normal_host`` (bfloat16: rounded once from float)."""
    _cuda(out)
    _check(lib().ccb_init_random(_p(out), out.numel(), _dt(out), int(seed) & (2 ** 64 - 1), int(key) & (2 ** 64 - 1),
                                 float(std), 1 if add_one else 0, _stream()), "init_random")
