"""ctypes bindings of the kernel library: torch tensors in, asynchronous launches on the current stream.

There is no CPU fallback and no library model code behind these functions: if the shared object
cannot be built or loaded, `load()` raises, and every function below raises with it.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_long, c_float, c_void_p

import torch

from . import build as _build

F32, BF16 = 0, 1
MODE_STORE, MODE_ADD, MODE_SWIGLU, MODE_GEGLU = 0, 1, 2, 3      # GEGLU: the gated mode with a gelu (tanh form) gate
MODE_CLAMPED_GLU = 4             # the gated mode with g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(1.702 g') (u' + 1)
MODE_STORE_RELU2 = 5             # the storing mode with max(x, 0)^2 applied to the float32 accumulator
MODE_STORE_GELU = 6              # the storing mode with the tanh form of gelu applied to the float32 accumulator
GATED_MODES = (MODE_SWIGLU, MODE_GEGLU, MODE_CLAMPED_GLU)
WINDOW_FULL, WINDOW_CHUNK, WINDOW_SLIDING = 0, 1, 2
WINDOW_KINDS = {"full": WINDOW_FULL, "chunk": WINDOW_CHUNK, "sliding": WINDOW_SLIDING}
MAX_DECODE_SPLITS = 256          # key splits that the combine kernel of decode attention takes
GENERAL_ATTENTION_MAX_DIM = 640  # largest key or value row of the general attention kernel
PREFILL_TILE_ROWS = 256          # most query rows of one sequence that a block of the prefill attention kernel takes

ABI_VERSION = 5                  # what cpi_abi_version() of a matching library answers

_lib = None
scratch_generation = 0    # grows whenever a scratch buffer of this module is (re)allocated
launch_count = 0          # kernels launched through this module since import (bench reports it)


class KernelError(RuntimeError):
    pass


def load():
    global _lib
    if _lib is None:
        path = _build.library_path()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cpi_b200: cannot load the kernel library {path}: {e}") from None
        _lib.cpi_last_error.restype = ctypes.c_char_p
        if _lib.cpi_abi_version() != ABI_VERSION:
            raise KernelError(f"cpi_b200: {path} has ABI version {_lib.cpi_abi_version()}, this package "
                              f"wants {ABI_VERSION}")
    return _lib


def kernel_launches() -> int:
    """Kernels this library has launched from host code (graph replays are counted by the engine)."""
    load().cpi_launch_count.restype = c_long
    return int(load().cpi_launch_count())


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"cpi_b200 kernels take float32 or bfloat16, not {dt}")


def _p(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _call(name, *args):
    global launch_count
    rc = getattr(load(), name)(*args)
    if rc != 0:
        raise KernelError(load().cpi_last_error().decode())
    launch_count += 1


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("cpi_b200 kernels run on CUDA tensors only (there is no CPU path)")


def _rowmajor(t, what):
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what}: expected a 2-D tensor with contiguous rows, got shape "
                          f"{tuple(t.shape)} strides {t.stride()}")


# ------------------------------------------------------------------------------------------------
def embedding(tokens, table, out, err_flag):
    """out[t, :] = table[tokens[t], :] as float32; a token outside the table sets err_flag[0] = 1 + t."""
    _need_cuda(tokens, table, out, err_flag)
    T, H = out.shape
    assert tokens.dtype == torch.int32 and out.dtype == torch.float32 and out.is_contiguous()
    assert table.is_contiguous() and table.shape[1] == H
    _call("cpi_embedding", _p(tokens), _p(table), c_int(dtype_code(table.dtype)), _p(out), c_int(T), c_int(H),
          c_int(table.shape[0]), _p(err_flag), _stream())


def rmsnorm(x, weight, eps, out, rows=None, weight_offset=0.0):
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * (weight_offset + weight); weight may be None."""
    _need_cuda(x, weight, out, rows)
    _rowmajor(x, "rmsnorm x"); _rowmajor(out, "rmsnorm out")
    n_rows, n = out.shape
    assert x.shape[1] == n and (rows is not None or x.shape[0] == n_rows)
    assert rows is None or rows.dtype == torch.int32
    assert weight is None or (weight.numel() == n and weight.is_contiguous())
    _call("cpi_rmsnorm", _p(x), c_int(dtype_code(x.dtype)), c_long(x.stride(0)), _p(rows), _p(weight),
          c_int(F32 if weight is None else dtype_code(weight.dtype)), _p(out), c_int(dtype_code(out.dtype)),
          c_long(out.stride(0)), c_int(n_rows), c_int(n), c_float(eps), c_float(weight_offset), _stream())


def gemm_simt(a, w, out, mode=MODE_STORE, *, n_out=None, m_rows=None, a_rows=None, out_rows=None,
              row_scale=None, group_offsets=None, n_groups=0, rows_per_group_hint=None, gate_limit=0.0):
    """out[m, n] (+)= sum_k a[a_rows[m] or m, k] * w[g(m)][n, k] on the FP32 pipe (see gemm_simt.cu).

    w is [N, K], or [2N, K] in SWIGLU mode, or [G, N or 2N, K] with group_offsets (int32 [G+1]).
    """
    _need_cuda(a, w, out, a_rows, out_rows, row_scale, group_offsets)
    _rowmajor(a, "gemm a"); _rowmajor(out, "gemm out")
    K = a.shape[1]
    if group_offsets is not None:
        assert w.dim() == 3 and w.is_contiguous() and w.shape[0] == n_groups
        rows_w, stride_g = w.shape[1], w.shape[1] * w.shape[2]
    else:
        _rowmajor(w, "gemm w")
        rows_w, stride_g = w.shape[0], 0
    assert w.shape[-1] == K, f"gemm: a has K={K}, w has K={w.shape[-1]}"
    N = n_out if n_out is not None else (rows_w // 2 if mode in GATED_MODES else rows_w)
    assert rows_w == (2 * N if mode in GATED_MODES else N)
    assert out.shape[1] == N
    M = m_rows if m_rows is not None else (a_rows.numel() if a_rows is not None else a.shape[0])
    ldw = w.stride(-2)
    hint = rows_per_group_hint if rows_per_group_hint is not None else M
    _call("cpi_gemm_simt", _p(a), c_int(dtype_code(a.dtype)), c_long(a.stride(0)), _p(a_rows),
          _p(w), c_int(dtype_code(w.dtype)), c_long(ldw), c_long(stride_g),
          _p(out), c_int(dtype_code(out.dtype)), c_long(out.stride(0)), _p(out_rows), _p(row_scale),
          _p(group_offsets), c_int(n_groups), c_int(M), c_int(N), c_int(K), c_int(mode), c_int(hint),
          c_float(gate_limit), _stream())


_errors = {}          # device index -> int32[2]: [0] a tensor-core kernel gave up a wait, [1] a token id out of range


def device_error_flags(device) -> torch.Tensor:
    """int32[2] on the device that kernels write when something went wrong: word 0 is set to 1 by a tensor-core
    kernel whose bounded barrier wait ran out, word 1 to 1 + t by the embedding kernel when token t of a step
    was outside the vocabulary.  The engine reads and clears them."""
    idx = torch.device(device).index or 0
    if idx not in _errors:
        _errors[idx] = torch.zeros(2, dtype=torch.int32, device=device)
    return _errors[idx]


def tc_error_flag(device) -> torch.Tensor:
    """int32[1] that a tensor-core kernel sets when one of its bounded waits ran out."""
    return device_error_flags(device)[0:1]


def sm_count() -> int:
    """Multiprocessors of the current CUDA device."""
    return int(load().cpi_sm_count())


def gemm_tc(a, w, out, mode=MODE_STORE, *, n_out=None, m_rows=None, a_rows=None, out_rows=None, row_scale=None,
            group_offsets=None, n_groups=0, rows_per_group_hint=None, gate_limit=0.0) -> bool:
    """The tcgen05 kernel for out[m, n] (+)= sum_k a[m, k] w[g(m)][n, k] in bfloat16 (see gemm_tc.cu).

    Returns False, having launched nothing, when the call is outside what the kernel takes (a row
    gather, K or a row stride that is no multiple of 8, unaligned operands, an output dtype the
    epilogue does not write); the caller then uses the FP32-pipe kernel."""
    if a_rows is not None or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    if a.dim() != 2 or a.stride(1) != 1 or not w.is_contiguous() or out.stride(-1) != 1:
        return False
    K = a.shape[1]
    if K % 8 or a.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16 or w.shape[-1] != K:
        return False
    if mode in GATED_MODES and out.dtype != torch.bfloat16:
        return False
    if mode == MODE_ADD and out.dtype != torch.float32:
        return False
    _need_cuda(a, w, out, out_rows, row_scale, group_offsets)
    grouped = group_offsets is not None
    rows_w = w.shape[-2]
    N = n_out if n_out is not None else (rows_w // 2 if mode in GATED_MODES else rows_w)
    if rows_w != (2 * N if mode in GATED_MODES else N) or out.shape[1] != N:
        raise KernelError(f"gemm_tc: weight rows {rows_w} do not match {N} outputs in mode {mode}")
    if grouped and (w.dim() != 3 or w.shape[0] != n_groups):
        raise KernelError("gemm_tc: grouped weights must be [groups, rows, K]")
    T = m_rows if m_rows is not None else a.shape[0]
    if T > a.shape[0]:
        raise KernelError("gemm_tc: more logical rows than activation rows")
    bn, splits, live_y = c_int(), c_int(), c_int()
    load().cpi_gemm_tc_plan(c_int(T), c_int(N), c_int(K), c_int(n_groups if grouped else 0),
                            c_int(int(mode in GATED_MODES)), ctypes.byref(bn), ctypes.byref(splits),
                            ctypes.byref(live_y))
    _call("cpi_gemm_tc", _p(a), c_long(a.stride(0)), _p(w), _p(out), c_int(dtype_code(out.dtype)),
          c_long(out.stride(0)), _p(out_rows), _p(row_scale), _p(group_offsets), c_int(n_groups if grouped else 0),
          c_int(T), c_int(N), c_int(K), c_int(mode), c_int(bn.value), c_int(splits.value),
          _p(tc_error_flag(a.device)), c_float(gate_limit), _stream())
    return True


def gemm_tc_plan(T: int, N: int, K: int, n_groups: int = 0, swiglu: bool = False):
    """(token rows per tile, k splits) that `gemm_tc` uses for a product of these sizes on this device."""
    bn, splits, live_y = c_int(), c_int(), c_int()
    load().cpi_gemm_tc_plan(c_int(T), c_int(N), c_int(K), c_int(n_groups), c_int(int(swiglu)), ctypes.byref(bn),
                            ctypes.byref(splits), ctypes.byref(live_y))
    return bn.value, splits.value


def gemm_tc_wait_probe(spin_limit: int = 0, tx_extra: int = 0) -> None:
    """For the test of the give-up path of `gemm_tc`: launches from now on poll each barrier at most
    `spin_limit` times and expect `tx_extra` bytes more per stage than their loads bring, so that the wait runs
    out, the kernel raises the error flag and returns.  (0, 0) puts the ordinary values back."""
    load().cpi_gemm_tc_wait_probe(c_int(int(spin_limit)), c_int(int(tx_extra)))


def gemm_pair_persistent(mode) -> None:
    """Dense products of `gemm_tc_pair`: 2 / True = always one pair of CTAs per SM pair working through the
    tiles (the epilogue of one tile under the MMAs of the next), 0 / False = always a launch slot per tile,
    1 = the library's choice by shape (the default)."""
    load().cpi_gemm_tc_pair_persistent(c_int(2 if mode is True else 0 if mode is False else int(mode)))


def gemm_tc_pair(a, w, out, mode=MODE_STORE, *, m_rows=None, out_rows=None, row_scale=None, group_offsets=None,
                 n_groups=0, rows_per_group_hint=None, gate_limit=0.0) -> bool:
    """The paired (two-SM) tcgen05 kernel for products with many tokens, dense or grouped (see
    gemm_tc_pair.cu).  Returns False, having launched nothing, when the product is outside what it takes."""
    grouped = group_offsets is not None
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != (3 if grouped else 2):
        return False
    if a.stride(1) != 1 or not w.is_contiguous() or out.stride(-1) != 1:
        return False
    K = a.shape[1]
    T = m_rows if m_rows is not None else a.shape[0]
    rows_w = w.shape[-2]
    N = rows_w // 2 if mode in GATED_MODES else rows_w
    if w.shape[-1] != K or out.shape[1] != N or a.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    if grouped and w.shape[0] != n_groups:
        return False
    if (mode in GATED_MODES and out.dtype != torch.bfloat16) or (mode == MODE_ADD and out.dtype != torch.float32):
        return False
    bn = load().cpi_gemm_tc_pair_plan(c_int(T), c_int(N), c_int(K), c_int(int(mode in GATED_MODES)),
                                      c_int(n_groups if grouped else 0))
    if bn <= 0:
        return False
    _need_cuda(a, w, out, out_rows, row_scale, group_offsets)
    _call("cpi_gemm_tc_pair", _p(a), c_long(a.stride(0)), _p(w), _p(out), c_int(dtype_code(out.dtype)),
          c_long(out.stride(0)), _p(out_rows), _p(row_scale), _p(group_offsets), c_int(n_groups if grouped else 0),
          c_int(T), c_int(N), c_int(K), c_int(mode), c_int(bn), _p(tc_error_flag(a.device)), c_float(gate_limit),
          _stream())
    return True


# ---- load time ----------------------------------------------------------------------------------------------
def random_normal(out, start, seed, std, table):
    """out.view(-1)[k] = table[hash(seed, start + k)] * std, rounded to out's dtype (float32 or bfloat16), for a
    contiguous CUDA tensor; `table`: float32 [65536] on the same device."""
    _need_cuda(out, table)
    assert out.is_contiguous() and table.dtype == torch.float32 and table.numel() == 65536 and table.is_contiguous()
    rc = load().cpi_random_normal(_p(out), c_int(dtype_code(out.dtype)), c_long(int(start)), c_long(out.numel()),
                                  ctypes.c_ulonglong(int(seed) & 0xFFFFFFFFFFFFFFFF), c_float(std), _p(table), _stream())
    if rc:
        raise KernelError(load().cpi_last_error().decode())


def widen_f16(src, dst):
    """dst (float32) = src (float16), exactly; contiguous CUDA tensors of equal size."""
    _need_cuda(src, dst)
    assert src.dtype == torch.float16 and dst.dtype == torch.float32 and src.is_contiguous() and dst.is_contiguous()
    assert src.numel() == dst.numel()
    if load().cpi_widen_f16(_p(src), _p(dst), c_long(src.numel()), _stream()):
        raise KernelError(load().cpi_last_error().decode())


def transpose_last2(src, dst=None):
    """dst [..., c, r] = src [..., r, c] for a contiguous CUDA tensor of 2- or 4-byte elements."""
    _need_cuda(src, dst)
    assert src.is_contiguous() and src.dim() >= 2 and src.element_size() in (2, 4)
    r, c = src.shape[-2], src.shape[-1]
    g = src.numel() // (r * c) if src.numel() else 0
    if dst is None:
        dst = torch.empty(*src.shape[:-2], c, r, dtype=src.dtype, device=src.device)
    assert dst.is_contiguous() and dst.dtype == src.dtype and dst.numel() == src.numel()
    if load().cpi_transpose(_p(src), _p(dst), c_int(src.element_size()), c_long(g), c_int(r), c_int(c), _stream()):
        raise KernelError(load().cpi_last_error().decode())
    return dst


def gather_rows(src, rows, dst):
    """dst[r] = src[rows[r]] for 2-D tensors whose rows are multiples of 16 bytes."""
    _need_cuda(src, rows, dst)
    _rowmajor(src, "gather_rows src")
    assert dst.is_contiguous() and dst.dtype == src.dtype and dst.shape[1] == src.shape[1]
    assert rows.dtype == torch.int32
    n = dst.shape[0]
    _call("cpi_gather_rows", _p(src), c_long(src.stride(0) * src.element_size()), _p(rows), _p(dst), c_int(n),
          c_int(src.shape[1] * src.element_size()), _stream())


def qkv_post(qkv, q_out, k_cache, v_cache, page_table, page_size, token_seq, token_pos, seq_slot, *,
             n_heads, n_kv_heads, head_dim, inv_freq=None, interleaved=False, qk_norm=False,
             norm_before_rope=False, norm_eps=0.0, temperature=None, write_kv=True):
    """Norm / rotate / scale q and k per head, write q to q_out and k, v into the cache pages."""
    _need_cuda(qkv, q_out, k_cache, v_cache, page_table, token_seq, token_pos, seq_slot, inv_freq)
    _rowmajor(qkv, "qkv_post qkv")
    T = qkv.shape[0]
    assert q_out.is_contiguous() and q_out.dtype == qkv.dtype
    assert k_cache is None or k_cache.dtype == qkv.dtype
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2)
    fl, sc = (temperature if temperature is not None else (1.0, 0.0))
    _call("cpi_qkv_post", _p(qkv), c_long(qkv.stride(0)), _p(q_out), _p(k_cache), _p(v_cache),
          c_int(dtype_code(qkv.dtype)), _p(page_table), c_int(page_table.shape[1]), c_int(page_size),
          _p(token_seq), _p(token_pos), _p(seq_slot), _p(inv_freq), c_int(int(interleaved)),
          c_int(int(qk_norm)), c_int(int(norm_before_rope)), c_float(norm_eps),
          c_int(int(temperature is not None)), c_float(fl), c_float(sc), c_int(T), c_int(n_heads),
          c_int(n_kv_heads), c_int(head_dim), c_int(int(write_kv)), _stream())


def attention_general(q, out, k_cache, v_cache, page_table, page_size, token_seq, token_pos, seq_slot, *,
                      n_heads, n_kv_heads, head_dim, window_kind, window_size, scale, score_bias=None, sink=None,
                      value_dim=None, keep_first=0, softcap=0.0):
    """Attention of any head size and dtype over the paged cache.  `score_bias`: float32 [heads, n_dist] added
    to the scaled scores, indexed by the distance query position - key position (the last column for longer).
    `sink`: float32 [heads]; exp(sink[h]) is one more term of the softmax denominator, without a key or a value.
    `value_dim`: elements of a value row when it differs from the keys' `head_dim`.  `keep_first`: with a sliding
    window, a sequence's first positions that every later query still sees.  `softcap` c > 0: a scaled score s
    becomes c * tanh(s / c) before anything is added to it."""
    _need_cuda(q, out, k_cache, v_cache, page_table, token_seq, token_pos, seq_slot, score_bias, sink)
    assert q.is_contiguous() and out.is_contiguous() and q.dtype == out.dtype == k_cache.dtype == v_cache.dtype
    assert score_bias is None or (score_bias.dtype == torch.float32 and score_bias.is_contiguous()
                                  and score_bias.dim() == 2 and score_bias.shape[0] == n_heads)
    assert sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == n_heads)
    value_dim = head_dim if value_dim is None else int(value_dim)
    assert k_cache.shape[-1] == head_dim and v_cache.shape[-1] == value_dim and out.shape[-1] == n_heads * value_dim
    T = q.shape[0]
    _call("cpi_attention_general", _p(q), _p(out), _p(k_cache), _p(v_cache), c_int(dtype_code(q.dtype)),
          _p(page_table), c_int(page_table.shape[1]), c_int(page_size), _p(token_seq), _p(token_pos),
          _p(seq_slot), c_int(T), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(window_kind),
          c_int(window_size), c_float(scale), _p(score_bias),
          c_int(0 if score_bias is None else score_bias.shape[1]), _p(sink), c_int(value_dim), c_int(int(keep_first)),
          c_float(float(softcap or 0.0)), _stream())


def qkv_prepare(qkv, q_out, k_cache, v_cache, page_table, page_size, token_seq, token_pos, seq_slot, *, n_heads,
                n_kv_heads, head_dim, value_dim, bias=None, q_norm=None, k_norm=None, norm_whole=False, norm_eps=0.0,
                inv_freq=None, rotary_dims=0, write_kv=True, head_norm=False, interleaved=False, v_first=None,
                v_mix=None, v_mix_mode=0, q2_out=None, k2_cache=None, values_from_keys=False, temperature=None,
                rotary_amplitude=1.0):
    """The general form of `qkv_post`, a block per token: rows [q | k | v] (float32 or the cache's dtype) get
    their bias, q and k an RMS norm over the whole projection (`norm_whole`, weights `q_norm` / `k_norm`), the
    first `rotary_dims` elements of each head their rotation, and then (`head_norm` True or 1) every q and k head a
    weightless RMS norm with `norm_eps`; q goes to q_out, k and v into the cache pages.  `head_norm` 2: every q and k
    head is normed before the rotation and multiplied by `q_norm` / `k_norm` ([head_dim], shared by the heads).
    `interleaved`: the rotation pairs elements (2i, 2i + 1) instead of (i, i + rotary_dims / 2).  Value mixing:
    `v_mix_mode` 1 also stores the values (float32) in `v_first` [T, kv heads * value_dim]; 2 writes
    (1 - m) v + m v_first[t] into the cache, m the one number `v_mix` holds.  With `q2_out` (and `k2_cache`) the rows
    hold two score maps: 2 * n_heads query heads and 2 * n_kv_heads key heads, the first halves going to q_out and
    k_cache, the second halves to q2_out and k2_cache (shaped alike); values have n_kv_heads heads.
    `values_from_keys`: rows are [q | k] and the cached values are the k rows as projected (bias added, before any
    norm).  `temperature` (f, a): q *= 1 + a * ln(floor((position + 1) / f) + 1).  `rotary_amplitude` multiplies the
    rotation's sines and cosines."""
    _need_cuda(qkv, q_out, k_cache, v_cache, page_table, token_seq, token_pos, seq_slot, bias, q_norm, k_norm, inv_freq,
               q2_out, k2_cache)
    maps = 1 if q2_out is None else 2
    assert q2_out is None or (q2_out.is_contiguous() and q2_out.shape == q_out.shape and q2_out.dtype == q_out.dtype)
    assert k2_cache is None or (k2_cache.shape == k_cache.shape and k2_cache.dtype == k_cache.dtype)
    fl, sc = (temperature if temperature is not None else (1.0, 0.0))
    _rowmajor(qkv, "qkv_prepare qkv")
    T = qkv.shape[0]
    assert q_out.is_contiguous() and q_out.shape[1] == n_heads * head_dim
    assert k_cache is None or (k_cache.dtype == q_out.dtype == v_cache.dtype and k_cache.shape[-1] == head_dim
                               and v_cache.shape[-1] == value_dim)
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dims // 2)
    assert bias is None or bias.is_contiguous()
    nw = q_norm if q_norm is not None else k_norm
    assert q_norm is None or k_norm is None or q_norm.dtype == k_norm.dtype
    _need_cuda(v_first, v_mix)
    assert v_first is None or (v_first.dtype == torch.float32 and v_first.stride(1) == 1
                               and v_first.shape == (T, n_kv_heads * value_dim))
    assert v_mix is None or v_mix.numel() == 1
    _call("cpi_qkv_prepare", _p(qkv), c_int(dtype_code(qkv.dtype)), c_long(qkv.stride(0)), _p(bias),
          c_int(F32 if bias is None else dtype_code(bias.dtype)), _p(q_norm), _p(k_norm),
          c_int(F32 if nw is None else dtype_code(nw.dtype)), c_int(int(norm_whole)), c_float(norm_eps),
          _p(inv_freq), c_int(rotary_dims), _p(q_out), _p(k_cache), _p(v_cache), c_int(dtype_code(q_out.dtype)),
          _p(page_table), c_int(page_table.shape[1]), c_int(page_size), _p(token_seq), _p(token_pos), _p(seq_slot),
          c_int(T), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(value_dim), c_int(int(write_kv)),
          c_int(int(head_norm)), c_int(int(interleaved)), _p(v_first), c_long(0 if v_first is None else v_first.stride(0)),
          _p(v_mix), c_int(F32 if v_mix is None else dtype_code(v_mix.dtype)), c_int(int(v_mix_mode)), c_int(maps),
          _p(q2_out), _p(k2_cache), c_int(int(values_from_keys)), c_int(int(temperature is not None)), c_float(fl),
          c_float(sc), c_float(float(rotary_amplitude)), _stream())


def head_post(a1, out, *, n_heads, value_dim, a2=None, lam=0.0, norm_eps=None, norm_scale=1.0, gate=None):
    """What follows attention per token and head, before the output projection: o = a1 - lam * a2 (a2 None: a1), then
    (norm_eps given) o / sqrt(mean(o^2) + norm_eps) * norm_scale over the head's values, then (gate given: float32
    [T, >= heads] rows, a column slice allowed) o * sigmoid(gate[t, head]); float32 arithmetic, out may be a1."""
    _need_cuda(a1, a2, out, gate)
    T = a1.shape[0]
    assert a1.is_contiguous() and out.is_contiguous() and a1.shape == out.shape == (T, n_heads * value_dim)
    assert a2 is None or (a2.is_contiguous() and a2.shape == a1.shape and a2.dtype == a1.dtype)
    assert gate is None or (gate.dtype == torch.float32 and gate.dim() == 2 and gate.stride(1) == 1 and gate.shape[1] >= n_heads)
    _call("cpi_head_post", _p(a1), _p(a2), c_int(dtype_code(a1.dtype)), _p(out), c_int(dtype_code(out.dtype)),
          c_float(float(lam)), c_int(int(norm_eps is not None)), c_float(float(norm_eps or 0.0)), c_float(float(norm_scale)),
          _p(gate), c_long(0 if gate is None else gate.stride(0)), c_int(T), c_int(n_heads), c_int(value_dim), _stream())


def sum_norm_add(branches, scales, weight, out, *, eps=0.0, add=True, h_out=None, normalise=True):
    """out (+)= rmsnorm(sum_b scales[b] * branches[b]) * weight over rows: up to four float32 [T, W] branches with a
    constant each, one norm over their sum (`normalise` False: the scaled sum as it is); `h_out` (any dtype, [T, W])
    also receives the new out rows."""
    _need_cuda(out, weight, h_out, *branches)
    n = len(branches)
    T, W = out.shape
    assert 1 <= n <= 4 and len(scales) == n and out.dtype == torch.float32 and out.stride(1) == 1
    for y in branches:
        assert y.dtype == torch.float32 and y.shape == (T, W) and y.stride(1) == 1
    assert weight is None or (weight.is_contiguous() and weight.numel() == W)
    assert h_out is None or (h_out.shape == (T, W) and h_out.stride(1) == 1)
    ys = (c_void_p * n)(*[y.data_ptr() for y in branches])
    st = (c_long * n)(*[y.stride(0) for y in branches])
    sc = (c_float * n)(*[float(x) for x in scales])
    _call("cpi_sum_norm_add", ys, st, sc, c_int(n), _p(weight), c_int(F32 if weight is None else dtype_code(weight.dtype)),
          c_int(T), c_int(W), c_float(eps), c_int(int(add)), _p(out), c_long(out.stride(0)), _p(h_out),
          c_int(F32 if h_out is None else dtype_code(h_out.dtype)), c_long(0 if h_out is None else h_out.stride(0)),
          c_int(int(normalise)), _stream())


def bias_rows(out, bias, *, add=False):
    """out[t, :] (+)= bias for float32 rows out [T, W] (a row stride allowed), bias [W]."""
    _need_cuda(out, bias)
    assert out.dtype == torch.float32 and out.dim() == 2 and out.stride(1) == 1 and bias.is_contiguous()
    assert bias.numel() == out.shape[1]
    _call("cpi_bias_rows", _p(out), c_long(out.stride(0)), _p(bias), c_int(dtype_code(bias.dtype)), c_int(out.shape[0]),
          c_int(out.shape[1]), c_int(int(add)), _stream())


def block_major_rows(x, out, offsets, *, parts):
    """out[b * T + t] = x[t, b * n : (b + 1) * n] in out's dtype, for float32 rows x [T, parts * n] (a column slice
    allowed) and out [parts * T, n] contiguous; offsets (int32 [parts + 1]) receives b * T, the groups of a grouped
    product with one group per part."""
    _need_cuda(x, out, offsets)
    T, W = x.shape
    n = W // parts
    assert x.dtype == torch.float32 and x.stride(1) == 1 and W == parts * n and out.is_contiguous()
    assert out.numel() == T * W and offsets.dtype == torch.int32 and offsets.numel() >= parts + 1
    _call("cpi_block_major_rows", _p(x), c_long(x.stride(0)), _p(out), c_int(dtype_code(out.dtype)), _p(offsets),
          c_int(T), c_int(parts), c_int(n), _stream())


def rglru_scan(gates, u, y, state, out, batch, *, block, lam, r_bias=None, i_bias=None, y_bias=None, rate=8.0):
    """The gated linear recurrent unit, a state per channel (float32 [slots, W], updated in place), per sequence:
    r = sigmoid(g_r + r_bias), i = sigmoid(g_i + i_bias), log a = -rate * softplus(lam) * r,
    S <- a S + sqrt(1 - a^2) * i * u, out = S * gelu_tanh(y + y_bias).  `gates`: float32 [W / block * T, 2 * block], row
    b * T + t holding block b's two gate products of token t (g_r, then g_i); u, y: float32 [T, W] rows (column slices
    allowed); the small vectors [W] of one dtype."""
    small = [t for t in (lam, r_bias, i_bias, y_bias) if t is not None]
    _need_cuda(gates, u, y, state, out, *small)
    T, W = u.shape
    assert W % block == 0 and gates.dtype == torch.float32 and gates.stride(1) == 1 and gates.shape == (W // block * T, 2 * block)
    for t in (u, y):
        assert t.dtype == torch.float32 and t.dim() == 2 and t.stride(1) == 1 and t.shape == (T, W)
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (W,)
    assert out.shape == (T, W) and out.stride(1) == 1
    assert all(t.dtype == lam.dtype and t.is_contiguous() and t.numel() == W for t in small)
    _call("cpi_rglru_scan", _p(gates), c_long(gates.stride(0)), _p(r_bias), _p(i_bias), _p(lam), _p(y_bias),
          c_int(dtype_code(lam.dtype)), _p(u), c_long(u.stride(0)), _p(y), c_long(y.stride(0)), _p(state), _p(out),
          c_int(dtype_code(out.dtype)), c_long(out.stride(0)), _p(batch.seq_slot), _p(batch.seq_tok0), _p(batch.seq_new),
          c_int(batch.n_seqs), c_int(batch.max_new), c_int(T), c_int(W), c_int(int(block)), c_float(float(rate)), _stream())


def latent_kv_write(x, norm_weight, eps, inv_freq, interleaved, cache, page_table, page_size, token_seq, token_pos,
                    seq_slot, *, rank, rot):
    """Per token, from float32 rows x [T, rank + rot] (a column slice allowed): the first `rank` elements RMS-normed
    (times `norm_weight`), the last `rot` rotated by the token's position; the row goes into the page of its position
    in `cache` [pages, 1, page_size, rank + rot]."""
    _need_cuda(x, norm_weight, inv_freq, cache, page_table, token_seq, token_pos, seq_slot)
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] == rank + rot
    assert cache.is_contiguous() and cache.shape[-1] == rank + rot and cache.shape[-3] == 1
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == rot // 2)
    assert norm_weight is None or (norm_weight.is_contiguous() and norm_weight.numel() == rank)
    _call("cpi_latent_kv_write", _p(x), c_long(x.stride(0)), _p(norm_weight),
          c_int(F32 if norm_weight is None else dtype_code(norm_weight.dtype)), c_float(eps), _p(inv_freq),
          c_int(int(interleaved)), _p(cache), c_int(dtype_code(cache.dtype)), _p(page_table), c_int(page_table.shape[1]),
          c_int(page_size), _p(token_seq), _p(token_pos), _p(seq_slot), c_int(x.shape[0]), c_int(rank), c_int(rot),
          _stream())


def latent_q_split(q, inv_freq, interleaved, plain, full, offsets, rows, token_pos, *, n_heads, dim, rot, rank):
    """From float32 rows q [T, heads * (dim + rot)]: a head's first `dim` elements go to plain[head * T + t] (rows laid
    out head by head), its last `rot`, rotated by the token's position, to full[t, head, rank : rank + rot].  Also
    fills offsets[h] = h * T (int32 [heads + 1]) and rows[h * T + t] = t * heads + h (int32 [heads * T])."""
    _need_cuda(q, inv_freq, plain, full, offsets, rows, token_pos)
    T = q.shape[0]
    assert q.dtype == torch.float32 and q.stride(1) == 1 and q.shape[1] == n_heads * (dim + rot)
    assert plain.is_contiguous() and plain.numel() == T * n_heads * dim and plain.dtype == full.dtype
    assert full.is_contiguous() and full.numel() == T * n_heads * (rank + rot)
    assert offsets.dtype == torch.int32 and offsets.numel() >= n_heads + 1 and rows.dtype == torch.int32
    assert rows.numel() >= T * n_heads
    _call("cpi_latent_q_split", _p(q), c_long(q.stride(0)), _p(inv_freq), c_int(int(interleaved)), _p(plain), _p(full),
          c_int(dtype_code(full.dtype)), _p(offsets), _p(rows), _p(token_pos), c_int(T), c_int(n_heads), c_int(dim),
          c_int(rot), c_int(rank), _stream())


def head_major_rows(x, out, *, n_heads, n):
    """out[h * T + t, :n] = x[t, h, :n] for contiguous rows x [T, heads * in_dim]."""
    _need_cuda(x, out)
    T = x.shape[0]
    in_dim = x.shape[1] // n_heads
    assert x.is_contiguous() and out.is_contiguous() and x.dtype == out.dtype and out.numel() == T * n_heads * n
    _call("cpi_head_major_rows", _p(x), _p(out), c_int(dtype_code(x.dtype)), c_int(T), c_int(n_heads), c_int(in_dim),
          c_int(n), _stream())


def gated_side_input(x, tokens, table, table_offset, gate, proj, norm_weight, eps):
    """x[t] += rmsnorm(proj @ (gelu_tanh(gate @ x[t]) * table[tokens[t], table_offset : table_offset + n])) * norm_weight
    in float32: x float32 [T, W] in place, gate [n, W], proj [W, n] (one dtype), table [vocab, *]."""
    _need_cuda(x, tokens, table, gate, proj, norm_weight)
    T, W = x.shape
    n = gate.shape[0]
    assert x.dtype == torch.float32 and x.stride(1) == 1 and tokens.dtype == torch.int32
    assert gate.is_contiguous() and proj.is_contiguous() and gate.dtype == proj.dtype
    assert gate.shape == (n, W) and proj.shape == (W, n) and table.stride(1) == 1 and table_offset + n <= table.shape[1]
    assert norm_weight is None or (norm_weight.is_contiguous() and norm_weight.numel() == W)
    _call("cpi_gated_side_input", _p(x), c_long(x.stride(0)), _p(tokens), _p(table), c_int(dtype_code(table.dtype)),
          c_long(table.stride(0)), c_int(int(table_offset)), c_int(table.shape[0]), _p(gate), _p(proj),
          c_int(dtype_code(gate.dtype)), _p(norm_weight),
          c_int(F32 if norm_weight is None else dtype_code(norm_weight.dtype)), c_float(eps), c_int(T), c_int(W),
          c_int(n), _stream())


def cast_rows(x, out):
    """out = x in out's dtype: float32 rows x [T, n] (a row stride allowed), out contiguous."""
    _need_cuda(x, out)
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1 and out.is_contiguous() and out.shape == x.shape
    _call("cpi_cast_rows", _p(x), c_long(x.stride(0)), _p(out), c_int(dtype_code(out.dtype)), c_int(x.shape[0]),
          c_int(x.shape[1]), _stream())


def side_gate_act(z, tokens, table, table_offset, out):
    """out[t, j] = gelu_tanh(z[t, j]) * table[tokens[t], table_offset + j]: z float32 [T, n] contiguous."""
    _need_cuda(z, tokens, table, out)
    T, n = z.shape
    assert z.dtype == torch.float32 and z.is_contiguous() and out.is_contiguous() and out.shape == z.shape
    assert tokens.dtype == torch.int32 and table.stride(1) == 1 and table_offset + n <= table.shape[1]
    _call("cpi_side_gate_act", _p(z), _p(tokens), _p(table), c_int(dtype_code(table.dtype)), c_long(table.stride(0)),
          c_int(int(table_offset)), c_int(table.shape[0]), _p(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(n),
          _stream())


def relu_squared(x, out):
    """out = max(x, 0)^2: float32 rows x into rows of out's dtype (the two may be one buffer)."""
    _need_cuda(x, out)
    assert x.dim() == 2 and x.stride(1) == 1 and x.dtype == torch.float32 and out.shape == x.shape and out.stride(1) == 1
    _call("cpi_relu_squared", _p(x), c_long(x.stride(0)), _p(out), c_int(dtype_code(out.dtype)), c_long(out.stride(0)),
          c_int(x.shape[0]), c_int(x.shape[1]), _stream())


def hc_step(x, *, y=None, mix=None, write=None, read=None, rows=None, norm_weight=None, norm_offset=0.0, eps=0.0,
            h_out=None, sum_out=None):
    """One boundary of a residual kept as streams x [S, T, W] (float32): with `y` [T, W] the write-back
    x_t <- sum_s mix[s, t] x_s + write[t] y; with `h_out` the next read u = sum_s read[s] x_s (read None: ones),
    normalised to h_out = u * rsqrt(mean(u^2) + eps) * (norm_offset + norm_weight); `rows` picks tokens (without
    y only); `sum_out` also receives u."""
    _need_cuda(x, y, mix, write, read, rows, norm_weight, h_out, sum_out)
    assert x.dim() == 3 and x.dtype == torch.float32 and x.stride(2) == 1 and x.stride(1) == x.shape[2]
    S, T, W = x.shape
    n = T if rows is None else rows.numel()
    for c in (mix, write, read):
        assert c is None or (c.dtype == torch.float32 and c.is_contiguous())
    assert y is None or (y.dtype == torch.float32 and y.shape == (T, W) and y.stride(1) == 1)
    assert h_out is None or (h_out.shape == (n, W) and h_out.stride(1) == 1)
    assert sum_out is None or (sum_out.dtype == torch.float32 and sum_out.is_contiguous() and sum_out.shape == (n, W))
    assert rows is None or rows.dtype == torch.int32
    _call("cpi_hc_step", _p(x), c_long(x.stride(0)), c_int(S), c_int(n), c_int(W), _p(y),
          c_long(0 if y is None else y.stride(0)), _p(mix), _p(write), _p(read), _p(rows), _p(norm_weight),
          c_int(F32 if norm_weight is None else dtype_code(norm_weight.dtype)), c_float(norm_offset), c_float(eps),
          _p(h_out), c_int(F32 if h_out is None else dtype_code(h_out.dtype)),
          c_long(0 if h_out is None else h_out.stride(0)), _p(sum_out), _stream())


def causal_conv(x, weight, bias, carry, out, batch, *, silu=True, in_bias=None):
    """out[t, c] = act(bias[c] + sum_j weight[c, j] x[t - (taps - 1) + j, c]) per sequence of the step; inputs
    before the step's first token come from carry[slot] ([slots, taps - 1, C] float32), which afterwards holds the
    sequence's last taps - 1 inputs.  x, out: float32 [T, C] (x may be a column slice).  `in_bias` [C] (the weight's
    dtype) is added to every input of the step before it is used or carried."""
    _need_cuda(x, weight, bias, carry, out, in_bias)
    assert in_bias is None or (in_bias.dtype == weight.dtype and in_bias.is_contiguous() and in_bias.numel() == x.shape[1])
    T, C = x.shape
    taps = weight.shape[1]
    assert x.dtype == torch.float32 and out.dtype == torch.float32 and x.stride(1) == 1 and out.stride(1) == 1
    assert weight.is_contiguous() and weight.shape[0] == C and (bias is None or (bias.dtype == weight.dtype and bias.numel() == C))
    assert carry.dtype == torch.float32 and carry.is_contiguous() and tuple(carry.shape[1:]) == (max(taps - 1, 0), C)
    _call("cpi_causal_conv", _p(x), c_long(x.stride(0)), _p(weight), _p(bias), c_int(dtype_code(weight.dtype)),
          _p(carry), _p(batch.token_seq), _p(batch.token_pos), _p(batch.seq_slot), _p(batch.seq_start),
          _p(batch.seq_tok0), _p(batch.seq_new), _p(out), c_long(out.stride(0)), c_int(T), c_int(batch.n_seqs),
          c_int(C), c_int(taps), c_int(int(silu)), _p(in_bias), _stream())
    global launch_count
    launch_count += int(taps > 1)


def linear_scan(k, q, v, state, out, batch, *, n_heads, heads_per_group, n_rows, n_cols, z=None, z_bias=None,
                tau=1.0, dt=None, dt_bias=None, a_log=None, skip=None, q_scale=1.0, decay_ready=False,
                decay_kind=0, beta=None):
    """The recurrence S_t = diag(a_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t (+ skip v_t) per sequence and head over the
    state [slots, heads, n_rows, n_cols] (float32, updated in place).  Give `z` [T, heads * n_rows] for a decay per
    row, a = sigmoid(z + z_bias)^(1 / tau); or `dt` [T, heads] for a decay per head with a step size,
    dt' = softplus(dt + dt_bias), a = exp(-exp(a_log) dt'), v' = dt' v.  All rows float32 (column slices allowed).
    `decay_ready`: `z` already holds a (`row_decay` ran over it).  `q_scale` multiplies the outputs' S^T q.
    `decay_kind` 1 (with `z` and `a_log`): a = exp(-exp(a_log[head]) softplus(z + z_bias)).  `beta` [T, heads]
    (before its sigmoid, with `z`): the delta rule, after the decay u = sigmoid(beta) (v - S^T k), S += k u^T."""
    small = [t for t in (z_bias, dt_bias, a_log, skip) if t is not None]
    _need_cuda(k, q, v, state, out, z, dt, beta, *small)
    for t in (k, q, v, out, z, dt, beta):
        assert t is None or (t.dtype == torch.float32 and t.dim() == 2 and t.stride(1) == 1)
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (n_heads, n_rows, n_cols)
    sd = small[0].dtype if small else torch.float32
    assert all(t.dtype == sd and t.is_contiguous() for t in small)
    _call("cpi_linear_scan", _p(k), c_long(k.stride(0)), _p(q), c_long(q.stride(0)), _p(v), c_long(v.stride(0)),
          _p(z), c_long(0 if z is None else z.stride(0)), _p(z_bias), c_float(1.0 / float(tau)),
          _p(dt), c_long(0 if dt is None else dt.stride(0)), _p(dt_bias), _p(a_log), _p(skip), c_int(dtype_code(sd)),
          c_float(q_scale), _p(state), _p(out), c_long(out.stride(0)), _p(batch.seq_slot), _p(batch.seq_tok0),
          _p(batch.seq_new), c_int(batch.n_seqs), c_int(getattr(batch, "max_new", 1 << 20)), c_int(n_heads),
          c_int(heads_per_group), c_int(n_rows), c_int(n_cols), c_int(int(decay_ready)), c_int(int(decay_kind)),
          _p(beta), c_long(0 if beta is None else beta.stride(0)), _stream())


def row_decay(z, z_bias, tau, *, kind=0, a_log=None, rows_per_head=0):
    """z <- sigmoid(z + z_bias)^(1 / tau) in place, z [T, n] float32 rows: the decays of `linear_scan`'s row flavour,
    prepared once per element for a step of many tokens (the recurrence computes the same expression itself when
    it is not given them).  kind 1: z <- exp(-exp(a_log[i // rows_per_head]) softplus(z + z_bias)); `a_log` has
    `z_bias`'s dtype."""
    _need_cuda(z, z_bias, a_log)
    assert a_log is None or (z_bias is not None and a_log.dtype == z_bias.dtype and a_log.is_contiguous())
    assert z.dtype == torch.float32 and z.dim() == 2 and z.stride(1) == 1
    assert z_bias is None or (z_bias.is_contiguous() and z_bias.numel() == z.shape[1])
    _call("cpi_row_decay", _p(z), c_long(z.stride(0)), _p(z_bias),
          c_int(F32 if z_bias is None else dtype_code(z_bias.dtype)), c_float(1.0 / float(tau)), c_int(z.shape[0]),
          c_int(z.shape[1]), c_int(int(kind)), _p(a_log), c_int(int(rows_per_head)), _stream())


GATE_NORM_ACTS = {"silu": 0, "sigmoid": 1}


def gated_norm(y, gate, weight, out, *, parts, gate_first, eps, gate_act="silu"):
    """out = norm(y * silu(gate)) * weight (gate_first) or norm(y) * weight * silu(gate): an RMS norm over each of
    `parts` equal pieces of a row by its own mean square; weight index = element % len(weight).  y, gate float32."""
    _need_cuda(y, gate, weight, out)
    T, W = y.shape
    assert y.dtype == torch.float32 and y.stride(1) == 1 and out.stride(1) == 1 and out.shape == (T, W)
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape == (T, W))
    assert weight is None or weight.is_contiguous()
    _call("cpi_gated_norm", _p(y), c_long(y.stride(0)), _p(gate), c_long(0 if gate is None else gate.stride(0)),
          _p(weight), c_int(F32 if weight is None else dtype_code(weight.dtype)),
          c_int(0 if weight is None else weight.numel()), _p(out), c_int(dtype_code(out.dtype)), c_long(out.stride(0)),
          c_int(T), c_int(W), c_int(parts), c_int(int(gate_first)), c_float(eps), c_int(GATE_NORM_ACTS[gate_act]),
          _stream())


GATE_ACTS = {"silu": 0, "gelu_tanh": 1, "swish_clamped": 2}


def gated_act(gate_up, out, act: str, limit: float = 0.0):
    """out = act(gate) * up for rows [gate | up] (float32, or out's dtype); "swish_clamped" is
    g sigmoid(1.702 g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit)."""
    _need_cuda(gate_up, out)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.is_contiguous() and out.is_contiguous()
    _call("cpi_gated_act", _p(gate_up), c_int(dtype_code(gate_up.dtype)), _p(out), c_int(dtype_code(out.dtype)),
          c_int(T), c_int(I), c_int(GATE_ACTS[act]), c_float(limit), _stream())


def head_unit(x, *, heads, dim, eps):
    """x[t, head, :] <- x / sqrt(sum(x^2) + eps) in place: float32 rows (a column slice allowed) of `heads` heads."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] == heads * dim
    _call("cpi_head_unit", _p(x), c_long(x.stride(0)), c_int(x.shape[0]), c_int(heads), c_int(dim), c_float(eps), _stream())


def branch_norm_sum(branches, weights, out, *, eps, scale=1.0, add=False):
    """out (+)= scale * sum_b rmsnorm(branches[b]) * weights[b]: up to four float32 [T, W] branches, each divided by
    its own root mean square over the row; weights [W] of one dtype; out float32 [T, W]."""
    _need_cuda(out, *branches, *weights)
    n = len(branches)
    T, W = out.shape
    assert 1 <= n <= 4 and len(weights) == n and out.dtype == torch.float32 and out.stride(1) == 1
    for y, w in zip(branches, weights):
        assert y.dtype == torch.float32 and y.shape == (T, W) and y.stride(1) == 1
        assert w.is_contiguous() and w.numel() == W and w.dtype == weights[0].dtype
    ys = (c_void_p * n)(*[y.data_ptr() for y in branches])
    st = (c_long * n)(*[y.stride(0) for y in branches])
    ws = (c_void_p * n)(*[w.data_ptr() for w in weights])
    _call("cpi_branch_norm_sum", ys, st, ws, c_int(dtype_code(weights[0].dtype)), c_int(n), c_int(T), c_int(W),
          c_float(eps), c_float(scale), c_int(int(add)), _p(out), c_long(out.stride(0)), _stream())


def concat_rows(a, b, out):
    """out[t] = [a[t] | b[t]] in out's dtype; a, b contiguous float32 [T, *]."""
    _need_cuda(a, b, out)
    T = a.shape[0]
    assert a.dtype == torch.float32 and b.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous()
    assert out.is_contiguous() and out.shape == (T, a.shape[1] + b.shape[1]) and b.shape[0] == T
    _call("cpi_concat_rows", _p(a), _p(b), _p(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(a.shape[1]),
          c_int(b.shape[1]), _stream())


def logit_post(logits, scale: float, softcap: float):
    """logits <- softcap * tanh(logits * scale / softcap) in place (softcap 0: only the scale)."""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    _call("cpi_logit_post", _p(logits), c_long(logits.numel()), c_float(scale), c_float(softcap), _stream())


_dec_scratch = {}


def attention_decode_supported(n_heads, n_kv_heads, head_dim, page_size) -> bool:
    return bool(load().cpi_attention_decode_supported(c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
                                                      c_int(page_size)))


def attention_decode(q, out, k_cache, v_cache, page_table, page_size, token_seq, token_pos, seq_slot, *,
                     n_heads, n_kv_heads, head_dim, window_kind, window_size, scale, n_splits, sink=None, keep_first=0,
                     softcap=0.0):
    """bfloat16 attention of independent tokens against the paged cache, keys split over `n_splits` blocks.
    `sink`: float32 [heads] whose exponentials join the softmax denominators.  `keep_first`: with a sliding window,
    a sequence's first positions that every later query still sees."""
    _need_cuda(q, out, k_cache, v_cache, page_table, token_seq, token_pos, seq_slot, sink)
    assert sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == n_heads)
    assert q.is_contiguous() and out.is_contiguous() and q.dtype == out.dtype == k_cache.dtype == torch.bfloat16
    T = q.shape[0]
    po = pml = None
    if n_splits > 1:
        idx = q.device.index or 0
        need = T * n_heads * n_splits * (head_dim + 2)
        buf = _dec_scratch.get(idx)
        if buf is None or buf.numel() < need:
            global scratch_generation
            buf = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=q.device)
            _dec_scratch[idx] = buf
            scratch_generation += 1
        po, pml = buf, buf[T * n_heads * n_splits * head_dim:]
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape
    _call("cpi_attention_decode", _p(q), _p(out), _p(k_cache), _p(v_cache), c_long(k_cache.shape[0]), _p(page_table),
          c_int(page_table.shape[1]), c_int(page_size), _p(token_seq), _p(token_pos), _p(seq_slot), c_int(T),
          c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(window_kind), c_int(window_size), c_float(scale),
          c_int(n_splits), _p(po), _p(pml), _p(tc_error_flag(q.device)), c_int(int(keep_first)), _p(sink),
          c_float(float(softcap or 0.0)), _stream())


def latent_attention_supported(row: int, rank: int) -> bool:
    """Whether the tensor-core kernel of attention over cached latent rows takes rows of `row` elements whose first
    `rank` are the value."""
    return bool(load().cpi_latent_attention_supported(c_int(int(row)), c_int(int(rank))))


def latent_attention_max_splits() -> int:
    return int(load().cpi_latent_attention_max_splits())


LATENT_KEY_TILE = 32             # cached positions that a block of the latent attention kernel takes at a time


def latent_attention(q, out, cache, page_table, page_size, token_seq, token_pos, seq_slot, *, n_heads, rank, scale,
                     sink=None, tile_tok0=None, tile_rows=None, n_splits=1):
    """bfloat16 softmax attention of q [T, heads * row] over cached rows [pages, 1, page_size, row] that all heads
    share: a row is the key, its first `rank` elements the value; a query sees every position up to its own.  out
    [heads * T, rank] is laid out head by head (row h * T + t).  With `tile_tok0` / `tile_rows` (runs of at most
    PREFILL_TILE_ROWS consecutive tokens of one sequence) a block takes a few tokens of a run; without, every token
    is alone and its keys are divided over `n_splits` blocks.  `sink`: float32 [heads], joins the denominators."""
    _need_cuda(q, out, cache, page_table, token_seq, token_pos, seq_slot, sink, tile_tok0, tile_rows)
    T = q.shape[0]
    row = cache.shape[-1]
    assert q.dtype == out.dtype == cache.dtype == torch.bfloat16
    assert q.is_contiguous() and out.is_contiguous() and cache.is_contiguous() and cache.shape[-3] == 1
    assert q.shape[1] == n_heads * row and out.numel() == T * n_heads * rank
    assert sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == n_heads)
    assert (tile_tok0 is None) == (tile_rows is None)
    po = pml = None
    if n_splits > 1:
        idx = q.device.index or 0
        need = T * n_heads * n_splits * (rank + 2)
        buf = _dec_scratch.get(idx)
        if buf is None or buf.numel() < need:
            global scratch_generation
            buf = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=q.device)
            _dec_scratch[idx] = buf
            scratch_generation += 1
        po, pml = buf, buf[T * n_heads * n_splits * rank:]
    _call("cpi_latent_attention", _p(q), _p(cache), _p(out), _p(po), _p(pml), _p(page_table),
          c_int(page_table.shape[1]), c_int(page_size), _p(token_seq), _p(token_pos), _p(seq_slot), _p(tile_tok0),
          _p(tile_rows), c_int(0 if tile_tok0 is None else tile_tok0.numel()), c_int(PREFILL_TILE_ROWS), _p(sink),
          c_int(T), c_int(n_heads), c_int(row), c_int(rank), c_int(int(n_splits)), c_float(scale), _stream())


def attention_decode_blocks_per_sm(head_dim: int) -> int:
    """Blocks of the decode attention kernel that share an SM."""
    return int(load().cpi_attention_decode_blocks_per_sm(c_int(head_dim)))


def attention_prefill_supported(n_heads, n_kv_heads, head_dim, page_size) -> bool:
    return bool(load().cpi_attention_prefill_supported(c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
                                                       c_int(page_size)))


def attention_prefill(q, out, k_cache, v_cache, page_table, page_size, token_seq, token_pos, seq_slot, tile_tok0,
                      tile_rows, *, n_heads, n_kv_heads, head_dim, window_kind, window_size, scale, sink=None,
                      keep_first=0, softcap=0.0):
    """bfloat16 attention of query tiles (<= PREFILL_TILE_ROWS consecutive tokens of one sequence each) on tcgen05.
    `sink`: float32 [heads] whose exponentials join the softmax denominators.  `keep_first`: as in `attention_decode`."""
    _need_cuda(q, out, k_cache, v_cache, page_table, token_seq, token_pos, seq_slot, tile_tok0, tile_rows, sink)
    assert sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == n_heads)
    assert q.is_contiguous() and out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert q.dtype == out.dtype == k_cache.dtype == torch.bfloat16
    _call("cpi_attention_prefill", _p(q), _p(out), _p(k_cache), _p(v_cache), c_long(k_cache.shape[0]), _p(page_table),
          c_int(page_table.shape[1]), c_int(page_size), _p(token_seq), _p(token_pos), _p(seq_slot), _p(tile_tok0),
          _p(tile_rows), c_int(tile_tok0.numel()), c_int(q.shape[0]), c_int(n_heads), c_int(n_kv_heads),
          c_int(head_dim), c_int(window_kind), c_int(window_size), c_float(scale), _p(tc_error_flag(q.device)),
          _p(sink), c_int(int(keep_first)), c_float(float(softcap or 0.0)), _stream())


ROUTER_GATES = {"none": 0, "sigmoid": 1, "softmax_chosen": 2, "sigmoid_normed": 3}


def _rule(rule):
    """The extra arguments of the selection: `rule` None, or for the gate "sigmoid_normed" a dictionary {"choice_bias":
    float32 [experts] or None, "groups": n, "keep": n, "scale": s}: the choice is made on sigmoid(logit) + choice_bias
    among the experts of the `keep` best of `groups` equal groups (a group's score: its two largest choice scores
    summed), the weights are the chosen sigmoids divided by their sum and multiplied by `scale`."""
    r = rule or {}
    cb = r.get("choice_bias")
    assert cb is None or (cb.dtype == torch.float32 and cb.is_contiguous() and cb.is_cuda)
    return _p(cb), c_int(int(r.get("groups", 1))), c_int(int(r.get("keep", 1))), c_float(float(r.get("scale", 1.0)))


def _gate_mode(sigmoid_gate) -> int:
    """False / True (the older spelling: no gate / sigmoid of the chosen logit) or a name of ROUTER_GATES."""
    return ROUTER_GATES[sigmoid_gate] if isinstance(sigmoid_gate, str) else int(bool(sigmoid_gate))


def router_topk(h, w, topk_idx, topk_gate, *, top_k, sigmoid_gate, logits_out=None, bias=None, rule=None):
    _need_cuda(h, w, topk_idx, topk_gate, logits_out, bias)
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == w.shape[0])
    _rowmajor(h, "router h")
    T, H = h.shape
    E = w.shape[0]
    assert w.is_contiguous() and w.shape[1] == H
    assert topk_idx.dtype == torch.int32 and topk_gate.dtype == torch.float32
    if logits_out is None:
        raise KernelError("router_topk: a float32 [tokens, experts] logits buffer is required")
    assert logits_out.dtype == torch.float32 and logits_out.is_contiguous() and logits_out.numel() >= T * E
    for t0 in range(0, T, 65535):            # the token axis is the grid's y dimension
        n = min(65535, T - t0)
        _call("cpi_router_topk", _p(h[t0:t0 + n]), c_int(dtype_code(h.dtype)), c_long(h.stride(0)), _p(w),
              c_int(dtype_code(w.dtype)), _p(logits_out[t0:t0 + n]), _p(topk_idx[t0:t0 + n]), _p(topk_gate[t0:t0 + n]),
              c_int(n), c_int(H), c_int(E), c_int(top_k), c_int(_gate_mode(sigmoid_gate)), _p(bias), c_int(0),
              *_rule(rule), _stream())


def router_select(logits, topk_idx, topk_gate, *, top_k, sigmoid_gate, rule=None):
    """The choice alone, from float32 router logits [T, E] (contiguous): the `top_k` experts of every token and their
    weights, by the gate `sigmoid_gate` names (see ROUTER_GATES and `_rule`)."""
    _need_cuda(logits, topk_idx, topk_gate)
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and topk_idx.dtype == torch.int32
    assert topk_gate.dtype == torch.float32 and topk_idx.numel() == T * top_k == topk_gate.numel()
    _call("cpi_router_select", _p(logits), _p(topk_idx), _p(topk_gate), c_int(T), c_int(E), c_int(top_k),
          c_int(_gate_mode(sigmoid_gate)), *_rule(rule), _stream())


def row_gates(h, w, out, bias=None):
    """out[t, e] = sigmoid(h[t] . w[e] (+ bias[e])) in float32, the router's dot products in one launch: a gate per
    token and row of w (w [E, H], out float32 [T, E])."""
    _need_cuda(h, w, out, bias)
    _rowmajor(h, "row_gates h")
    T, H = h.shape
    E = w.shape[0]
    assert w.is_contiguous() and w.shape[1] == H and out.dtype == torch.float32 and out.is_contiguous() and out.numel() == T * E
    for t0 in range(0, T, 65535):
        n = min(65535, T - t0)
        _call("cpi_router_topk", _p(h[t0:t0 + n]), c_int(dtype_code(h.dtype)), c_long(h.stride(0)), _p(w),
              c_int(dtype_code(w.dtype)), _p(out.view(T, E)[t0:t0 + n]), None, None, c_int(n), c_int(H), c_int(E), c_int(1),
              c_int(0), _p(bias), c_int(1), *_rule(None), _stream())


def moe_route(h, w, topk_idx, topk_gate, logits, group_offsets, row_token, row_scale, row_of_slot, *, top_k,
              sigmoid_gate, sorted_h=None, bias=None, rule=None) -> bool:
    """Router logits, the top-k choice and the per-expert row lists of a step; returns whether
    `sorted_h` (the activation rows in expert order) was filled too.  A step with few tokens takes two
    launches (logits, then one kernel for the rest), a larger one the separate kernels; the results
    are the same.  `sigmoid_gate`: False, True or a name of ROUTER_GATES; `bias`: float32 [experts] added to the logits."""
    _need_cuda(h, w, topk_idx, topk_gate, logits, group_offsets, row_token, row_scale, row_of_slot, sorted_h, bias)
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == w.shape[0])
    gm = _gate_mode(sigmoid_gate)
    _rowmajor(h, "router h")
    T, H = h.shape
    E = w.shape[0]
    if T <= 65535 and T * top_k <= 256 and T * E <= 4096:
        assert w.is_contiguous() and w.shape[1] == H and logits.dtype == torch.float32 and logits.is_contiguous()
        _call("cpi_router_topk", _p(h), c_int(dtype_code(h.dtype)), c_long(h.stride(0)), _p(w),
              c_int(dtype_code(w.dtype)), _p(logits), None, None, c_int(T), c_int(H), c_int(E), c_int(top_k),
              c_int(gm), _p(bias), c_int(0), *_rule(None), _stream())
        rc = load().cpi_moe_route_small(_p(logits), c_int(T), c_int(E), c_int(top_k), c_int(gm),
                                        _p(topk_idx), _p(topk_gate), _p(group_offsets), _p(row_token), _p(row_scale),
                                        _p(row_of_slot), _p(h), c_long(h.stride(0) * h.element_size()), _p(sorted_h),
                                        c_int(H * h.element_size()), *_rule(rule), _stream())
        if rc == 0:
            global launch_count
            launch_count += 1
            return sorted_h is not None
        if rc > 0:
            raise KernelError(load().cpi_last_error().decode())
        # too large or unaligned for the one-launch kernel: select here, lists below
        _call("cpi_router_select", _p(logits), _p(topk_idx), _p(topk_gate), c_int(T), c_int(E), c_int(top_k),
              c_int(gm), *_rule(rule), _stream())
    else:
        router_topk(h, w, topk_idx, topk_gate, top_k=top_k, sigmoid_gate=sigmoid_gate, logits_out=logits, bias=bias,
                    rule=rule)
    moe_lists(topk_idx, topk_gate, group_offsets, row_token, row_scale, row_of_slot, n_tokens=T, top_k=top_k,
              n_experts=E)
    return False


def moe_lists(topk_idx, topk_gate, group_offsets, row_token, row_scale, row_of_slot, *, n_tokens, top_k,
              n_experts):
    _need_cuda(topk_idx, topk_gate, group_offsets, row_token, row_scale, row_of_slot)
    _call("cpi_moe_lists", _p(topk_idx), _p(topk_gate), _p(group_offsets), _p(row_token), _p(row_scale),
          _p(row_of_slot), c_int(n_tokens), c_int(top_k), c_int(n_experts), _stream())


def moe_combine(residual, y, row_of_slot, *, top_k):
    """residual[t] += y[row_of_slot[t, 0]] + ... + y[row_of_slot[t, top_k - 1]]."""
    _need_cuda(residual, y, row_of_slot)
    T, H = residual.shape
    assert residual.dtype == torch.float32 and residual.is_contiguous() and y.is_contiguous()
    _call("cpi_moe_combine", _p(residual), _p(y), c_int(dtype_code(y.dtype)), _p(row_of_slot), c_int(T),
          c_int(top_k), c_int(H), _stream())


def swiglu(gate_up, out):
    _need_cuda(gate_up, out)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.is_contiguous() and out.is_contiguous()
    _call("cpi_swiglu", _p(gate_up), _p(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(I), _stream())


def argmax(logits, out):
    _need_cuda(logits, out)
    _rowmajor(logits, "argmax logits")
    assert logits.dtype == torch.float32 and out.dtype == torch.int32
    R, V = logits.shape
    _call("cpi_argmax", _p(logits), c_long(logits.stride(0)), c_int(R), c_int(V), _p(out), _stream())


def sample(logits, work, temperature, top_k, top_p, uniform, out):
    _need_cuda(logits, work, temperature, top_k, top_p, uniform, out)
    _rowmajor(logits, "sample logits")
    R, V = logits.shape
    assert logits.dtype == torch.float32 and work.dtype == torch.float32 and work.numel() >= R * V
    assert temperature.dtype == torch.float32 and top_k.dtype == torch.int32 and top_p.dtype == torch.float32
    assert uniform.dtype == torch.float32 and out.dtype == torch.int32
    _call("cpi_sample", _p(logits), c_long(logits.stride(0)), _p(work), c_int(R), c_int(V), _p(temperature),
          _p(top_k), _p(top_p), _p(uniform), _p(out), _stream())


def repetition_penalty(logits, ids, id_offsets, penalty):
    _need_cuda(logits, ids, id_offsets, penalty)
    R, V = logits.shape
    _call("cpi_repetition_penalty", _p(logits), c_long(logits.stride(0)), c_int(R), c_int(V), _p(ids),
          _p(id_offsets), _p(penalty), _stream())


def ban_tokens(logits, ids, id_offsets):
    _need_cuda(logits, ids, id_offsets)
    R, V = logits.shape
    _call("cpi_ban_tokens", _p(logits), c_long(logits.stride(0)), c_int(R), c_int(V), _p(ids), _p(id_offsets),
          _stream())
