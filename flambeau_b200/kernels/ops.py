"""Tensor-level wrappers of the kernel launchers.

Each wrapper checks devices, dtypes and strides, then launches on torch's
current CUDA stream.  Constants (eps, theta-derived tables, head sizes, window,
scale) arrive as arguments; nothing here knows a model.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .library import KernelError, check, lib

_CODES = {torch.float32: 0, torch.bfloat16: 1}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32 or bfloat16)") from None


try:                                   # the raw handle of torch's current stream, without building a Stream object
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:                 # a torch without it: the public way, a few microseconds slower per launch
    _raw_stream = None


def current_stream() -> int:
    """The CUDA stream the kernels are queued on: torch's current stream of the current device."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_stream = current_stream


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must live on the GPU; there is no CPU path")


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _rows(t: torch.Tensor) -> int:
    """Row stride (elements) of a 2-d tensor whose rows are dense."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"expected a 2-d tensor with dense rows, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


def _i32(t, what):
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32")


# ---------------------------------------------------------------------------

def embedding(table: torch.Tensor, ids: torch.Tensor, x: torch.Tensor, status: torch.Tensor,
              scale: float = 1.0) -> None:
    """x[t] = table[ids[t]] * scale, float32."""
    _cuda(table, ids, x, status)
    _i32(ids, "token ids")
    V, H = table.shape
    n = ids.numel()
    if x.dtype != torch.float32 or x.shape[0] < n or x.shape[1] != H or not x.is_contiguous() \
            or not table.is_contiguous():
        raise KernelError("embedding: the stream must be contiguous float32 [n, width]")
    check(lib().fb_embedding(table.data_ptr(), dtype_code(table), ids.data_ptr(), x.data_ptr(), n, H, V,
                             float(scale), status.data_ptr(), _stream()), "embedding")


def add_rms_norm(x: torch.Tensor, delta, weight: torch.Tensor, eps: float, out: torch.Tensor,
                 rows=None, n_partials: int = 1, n_rows: int | None = None, partial_stride: int = 0,
                 weight_offset: float = 0.0) -> None:
    """out[j] = rmsnorm(x[r] + sum_p delta_p[r]) * (weight + weight_offset), r = rows[j] or j; without `rows`
    the sum is also written back to x.  `delta` is [n, H]; with n_partials > 1 it is the first of that many
    slabs `partial_stride` elements apart.  weight_offset is 0 for a plain weight, 1 for a "1 + w" norm."""
    _cuda(x, delta, weight, out, rows)
    _i32(rows, "rows")
    H = x.shape[1]
    n_out = rows.numel() if rows is not None else (x.shape[0] if n_rows is None else n_rows)
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or out.shape[-1] != H \
            or weight.numel() != H or out.shape[0] < n_out:
        raise KernelError("add_rms_norm: bad shapes")
    stride = 0
    if delta is not None:
        if not delta.is_contiguous() or delta.shape[-1] != H:
            raise KernelError("add_rms_norm: delta must be contiguous with the stream's width")
        if n_partials > 1:
            stride = int(partial_stride)
            if stride <= 0:
                raise KernelError("add_rms_norm: several slabs need their stride")
    check(lib().fb_add_rmsnorm(x.data_ptr(), _ptr(delta), dtype_code(delta) if delta is not None else 0,
                               n_partials, stride, weight.data_ptr(), dtype_code(weight), out.data_ptr(),
                               dtype_code(out), _ptr(rows), n_out, H, float(eps), float(weight_offset), _stream()),
          "add_rms_norm")


def norm_add_rms_norm(x: torch.Tensor, delta: torch.Tensor, delta_weight: torch.Tensor, delta_eps: float,
                      delta_weight_offset: float, weight, eps: float, out, rows=None, n_partials: int = 1,
                      n_rows: int | None = None, partial_stride: int = 0, weight_offset: float = 0.0) -> None:
    """x[r] += rmsnorm(sum_p delta_p[r]) * (delta_weight + delta_weight_offset) (written back to x without `rows`),
    then out[j] = rmsnorm(x[r]) * (weight + weight_offset), r = rows[j] or j.  `out` (and `weight`) may be None:
    only the stream is updated.  delta is float32 [n, H], with n_partials > 1 the first of that many slabs
    `partial_stride` elements apart."""
    _cuda(x, delta, delta_weight, weight, out, rows)
    _i32(rows, "rows")
    H = x.shape[1]
    n_out = rows.numel() if rows is not None else (x.shape[0] if n_rows is None else n_rows)
    if x.dtype != torch.float32 or not x.is_contiguous() or delta.dtype != torch.float32 or not delta.is_contiguous() \
            or delta.shape[-1] != H or delta_weight.numel() != H:
        raise KernelError("norm_add_rms_norm: the stream and the delta must be contiguous float32 of one width")
    if out is not None and (not out.is_contiguous() or out.shape[-1] != H or out.shape[0] < n_out
                            or weight is None or weight.numel() != H):
        raise KernelError("norm_add_rms_norm: bad output")
    if out is None and rows is not None:
        raise KernelError("norm_add_rms_norm: nothing to do (no output, and chosen rows are not written back)")
    stride = int(partial_stride) if n_partials > 1 else 0
    if n_partials > 1 and stride <= 0:
        raise KernelError("norm_add_rms_norm: several slabs need their stride")
    check(lib().fb_norm_add_rmsnorm(x.data_ptr(), delta.data_ptr(), int(n_partials), stride, delta_weight.data_ptr(),
                                    dtype_code(delta_weight), float(delta_eps), float(delta_weight_offset),
                                    _ptr(weight), dtype_code(weight) if weight is not None else 0, _ptr(out),
                                    dtype_code(out) if out is not None else 0, _ptr(rows), n_out, H, float(eps),
                                    float(weight_offset), _stream()), "norm_add_rms_norm")


def concat_cast(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = [a[t] ; b[t]] in out's dtype; a and b are contiguous float32 [n, H]."""
    _cuda(a, b, out)
    n, H = a.shape
    if a.dtype != torch.float32 or b.dtype != torch.float32 or tuple(b.shape) != (n, H) or not a.is_contiguous() \
            or not b.is_contiguous() or tuple(out.shape) != (n, 2 * H) or not out.is_contiguous():
        raise KernelError("concat_cast: two contiguous float32 [n, H] in, one contiguous [n, 2H] out")
    check(lib().fb_concat_cast(a.data_ptr(), b.data_ptr(), out.data_ptr(), dtype_code(out), n, H, _stream()),
          "concat_cast")


def qkv_bias_cache_write(proj: torch.Tensor, bias, q_out: torch.Tensor, gate_out, cache, positions, row_seq,
                         nh: int, nkv: int, qd: int, vd: int, n_gate: int, status, n_partials: int = 1,
                         partial_stride: int = 0) -> None:
    """What follows a fused projection whose float32 rows hold [q: nh*qd | k: nkv*qd | v: nkv*vd | gate: n_gate],
    possibly as split-K shares: the shares are added, `bias` (over the q, k and v columns, optional) is added,
    q goes to q_out, k and v into their pages (pools [pages, nkv, page size, qd] and [.., vd]) when the cache view
    is writable, and gate_out (float32 [n, n_gate]) = sigmoid of the gate columns."""
    _cuda(proj, bias, q_out, gate_out, positions, row_seq, status)
    n = proj.shape[0]
    if proj.dtype != torch.float32 or q_out.shape[0] != n or q_out.shape[1] != nh * qd:
        raise KernelError("qkv_bias_cache_write: float32 projection rows and q [n, heads * size] wanted")
    if bias is not None and (bias.numel() != nh * qd + nkv * qd + nkv * vd or not bias.is_contiguous()):
        raise KernelError("qkv_bias_cache_write: the bias covers the q, k and v columns")
    if n_gate and (gate_out is None or gate_out.dtype != torch.float32 or not gate_out.is_contiguous()
                   or tuple(gate_out.shape) != (n, n_gate)):
        raise KernelError("qkv_bias_cache_write: the gate wants contiguous float32 [n, gates]")
    k_pool, v_pool = cache.k_pool, cache.v_pool
    n_pages = k_pool.shape[0]
    if tuple(k_pool.shape) != (n_pages, nkv, cache.page_size, qd) or tuple(v_pool.shape) != (n_pages, nkv, cache.page_size, vd) \
            or not k_pool.is_contiguous() or not v_pool.is_contiguous() or k_pool.dtype != q_out.dtype \
            or v_pool.dtype != q_out.dtype:
        raise KernelError("qkv_bias_cache_write: pools must be contiguous [pages, kv heads, page size, size] in q's dtype")
    check(lib().fb_qkv_bias_cache_write(
        proj.data_ptr(), _rows(proj), int(n_partials), int(partial_stride), _ptr(bias),
        dtype_code(bias) if bias is not None else 0, q_out.data_ptr(), _rows(q_out), dtype_code(q_out),
        _ptr(gate_out), positions.data_ptr(), row_seq.data_ptr(), cache.block_table.data_ptr(),
        cache.block_table.stride(0), _ptr(cache.table_base), k_pool.data_ptr(), v_pool.data_ptr(), cache.page_size,
        n_pages, n, nh, nkv, qd, vd, n_gate, 1 if cache.writable else 0, status.data_ptr(), _stream()),
        "qkv_bias_cache_write")


def diff_attention_simt(q, out, gate, cache, positions, row_seq, nh: int, nkv: int, kd: int, vd: int, window: int,
                        scale: float, lam: float, eps: float, out_scale: float, status) -> None:
    """Differential attention with float32 math on the CUDA cores (see csrc/diff_attention.cu): q [n, nh*2*kd],
    out [n, nh*vd], gate float32 [n, nh] or None."""
    _cuda(q, out, gate, positions, row_seq, status)
    n = q.shape[0]
    k_pool, v_pool = cache.k_pool, cache.v_pool
    n_pages = k_pool.shape[0]
    if q.shape[1] != nh * 2 * kd or tuple(out.shape) != (n, nh * vd) or tuple(k_pool.shape[1:]) != (nkv, cache.page_size, 2 * kd) \
            or tuple(v_pool.shape[1:]) != (nkv, cache.page_size, vd):
        raise KernelError("diff attention: shapes do not match the head counts")
    if not (q.dtype == out.dtype == k_pool.dtype == v_pool.dtype):
        raise KernelError("diff attention: q, out and the cache must share one dtype")
    if gate is not None and (gate.dtype != torch.float32 or tuple(gate.shape) != (n, nh) or not gate.is_contiguous()):
        raise KernelError("diff attention: the gate wants contiguous float32 [n, heads]")
    check(lib().fb_diff_attention_simt(
        q.data_ptr(), _rows(q), out.data_ptr(), _rows(out), dtype_code(q), _ptr(gate), k_pool.data_ptr(),
        v_pool.data_ptr(), cache.page_size, n_pages, cache.block_table.data_ptr(), cache.block_table.stride(0),
        _ptr(cache.table_base), positions.data_ptr(), row_seq.data_ptr(), n, nh, nkv, kd, vd, int(window),
        float(scale), float(lam), float(eps), float(out_scale), status.data_ptr(), _stream()), "diff_attention_simt")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
               magnitude: float = 1.0) -> None:
    """cos[t, i], sin[t, i] = magnitude * cos / sin(positions[t] * inv_freq[i]), the angle formed in float64."""
    _cuda(positions, inv_freq, cos, sin)
    _i32(positions, "positions")
    n, half = positions.numel(), inv_freq.numel()
    if inv_freq.dtype != torch.float64 or cos.dtype != torch.float32 or sin.dtype != torch.float32 \
            or cos.numel() < n * half or sin.numel() < n * half:
        raise KernelError("rope_table: bad arguments")
    check(lib().fb_rope_table(positions.data_ptr(), inv_freq.data_ptr(), cos.data_ptr(), sin.data_ptr(), n, half,
                              float(magnitude), _stream()), "rope_table")


def rope_kv_write(q_in, q_out, k, v, cos, sin, half: int, positions, row_seq, block_table, k_pool, v_pool,
                  page_size: int, nh: int, nkv: int, hd: int, write_kv: bool, status, n_partials: int = 1,
                  partial_stride: int = 0, table_base=None, table_head: int = 0) -> None:
    """q_out = rotate(q_in) (q_out may be q_in); with write_kv, rotate k into the cache and copy v into it.
    q_in, k, v share one dtype (the projection's output); q_out and the cache share one dtype.  With
    n_partials > 1 the inputs are split-K shares `partial_stride` elements apart and are added first.
    table_base (int32 per sequence, optional): the logical page that the first column behind the kept pages' of each
    table row stands for; table_head: how many columns in front hold a request's kept first pages."""
    _cuda(q_in, q_out, k, v, cos, sin, positions, row_seq, block_table, k_pool, v_pool, status, table_base)
    _i32(table_base, "table_base")
    n = q_in.shape[0]
    if q_in.shape[1] != nh * hd or q_out.shape[1] != nh * hd or q_out.shape[0] != n:
        raise KernelError("rope_kv_write: q widths do not match the head counts")
    if write_kv:
        if k.shape[1] != nkv * hd or v.shape[1] != nkv * hd:
            raise KernelError("rope_kv_write: k/v widths do not match the head counts")
        if k.dtype != q_in.dtype or v.dtype != q_in.dtype or k_pool.dtype != q_out.dtype or v_pool.dtype != q_out.dtype:
            raise KernelError("rope_kv_write: inputs must share one dtype; q_out and the cache another")
    n_pages = k_pool.shape[0] if write_kv else 0
    if write_kv and (tuple(k_pool.shape) != (n_pages, nkv, page_size, hd) or not k_pool.is_contiguous()
                     or tuple(v_pool.shape) != tuple(k_pool.shape) or not v_pool.is_contiguous()):
        raise KernelError("rope_kv_write: cache pools must be contiguous [pages, kv heads, page size, head size]")
    check(lib().fb_rope_kv_write(
        q_in.data_ptr(), _rows(q_in), int(n_partials), int(partial_stride), q_out.data_ptr(), _rows(q_out), _ptr(k),
        _rows(k) if k is not None else 0,
        _ptr(v), _rows(v) if v is not None else 0, dtype_code(q_in), dtype_code(q_out), _ptr(cos), _ptr(sin), half,
        _ptr(positions), _ptr(row_seq), _ptr(block_table),
        block_table.stride(0) if block_table is not None else 0, _ptr(table_base), int(table_head), _ptr(k_pool),
        _ptr(v_pool), page_size, n_pages, n, nh, nkv if write_kv else 0, hd, 1 if write_kv else 0, status.data_ptr(),
        _stream()), "rope_kv_write")


ACTIVATIONS = {"silu": 1, "gelu_tanh": 2, "gelu_pytorch_tanh": 2}      # codes of the kernels' gate activations


def activation_code(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"activation '{name}' is not implemented; known: {', '.join(sorted(ACTIVATIONS))}") from None


def gate_mul(gate_up: torch.Tensor, out: torch.Tensor, n_partials: int = 1, partial_stride: int = 0,
             activation: str = "silu") -> None:
    """out[:, c] = act(gate_up[:, 2c]) * gate_up[:, 2c+1] (gate and up alternate along a row); with
    n_partials > 1, gate_up is the first of that many split-K shares `partial_stride` elements apart, which are
    added first."""
    _cuda(gate_up, out)
    n, two_i = gate_up.shape
    I = two_i // 2
    if tuple(out.shape) != (n, I) or not out.is_contiguous():
        raise KernelError("gate_mul: bad output")
    check(lib().fb_gate_mul(gate_up.data_ptr(), _rows(gate_up), dtype_code(gate_up), int(n_partials),
                            int(partial_stride), out.data_ptr(), dtype_code(out), n, I, activation_code(activation),
                            _stream()), "gate_mul")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, n_partials: int = 1, partial_stride: int = 0) -> None:
    gate_mul(gate_up, out, n_partials, partial_stride, "silu")


PLAIN_ACTIVATIONS = {None: 0, "none": 0, "silu": 1, "gelu_tanh": 2, "relu_squared": 3}   # activations without a gate


def plain_activation_code(name) -> int:
    try:
        return PLAIN_ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"activation '{name}' is not one of {sorted(str(k) for k in PLAIN_ACTIVATIONS)}") from None


def activation(z: torch.Tensor, out: torch.Tensor, name: str, n_partials: int = 1, partial_stride: int = 0) -> None:
    """out = act(z), z possibly the first of n_partials split-K shares `partial_stride` elements apart."""
    _cuda(z, out)
    n, I = z.shape
    if tuple(out.shape) != (n, I) or not out.is_contiguous():
        raise KernelError("activation: bad output")
    check(lib().fb_activation(z.data_ptr(), _rows(z), dtype_code(z), int(n_partials), int(partial_stride),
                              out.data_ptr(), dtype_code(out), n, I, plain_activation_code(name), _stream()),
          "activation")


def add_row(x: torch.Tensor, v: torch.Tensor) -> None:
    """x[r] += v for every row of the contiguous float32 x."""
    _cuda(x, v)
    n, H = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or v.numel() != H or not v.is_contiguous():
        raise KernelError("add_row: a contiguous float32 [n, H] and a vector of H wanted")
    check(lib().fb_add_row(x.data_ptr(), v.data_ptr(), dtype_code(v), n, H, _stream()), "add_row")


def add_slabs(x: torch.Tensor, delta: torch.Tensor, n: int, n_partials: int = 1, partial_stride: int = 0) -> None:
    """x[:n] += delta[:n] (and the further shares of delta, `partial_stride` elements apart); contiguous float32."""
    _cuda(x, delta)
    if x.dtype != torch.float32 or delta.dtype != torch.float32 or not x.is_contiguous() or not delta.is_contiguous() \
            or x.shape[1] != delta.shape[-1]:
        raise KernelError("add_slabs: contiguous float32 rows of one width wanted")
    check(lib().fb_add_slabs(x.data_ptr(), delta.data_ptr(), int(n_partials), int(partial_stride), int(n), x.shape[1],
                             _stream()), "add_slabs")


def branch_norm_mix(branches, eps: float, out: torch.Tensor, n: int, weight_offset: float = 0.0) -> None:
    """out[r] = sum_b coef_b * rmsnorm(y_b[r]) * (w_b + weight_offset) for the first n rows.  `branches`: tuples
    (y float32 [n, H] or the first of its shares, n_partials, partial_stride, weight [H], coef); the weights share
    one dtype."""
    H = out.shape[1]
    B = len(branches)
    ys = (ctypes.c_void_p * B)(*[y.data_ptr() for y, *_ in branches])
    parts = (ctypes.c_int * B)(*[int(p) for _, p, *_ in branches])
    strides = (ctypes.c_longlong * B)(*[int(s) for _, _, s, *_ in branches])
    ws = (ctypes.c_void_p * B)(*[w.data_ptr() for *_, w, _ in branches])
    coefs = (ctypes.c_float * B)(*[float(c) for *_, c in branches])
    for y, _, _, w, _ in branches:
        _cuda(y, w)
        if y.dtype != torch.float32 or y.shape[-1] != H or not y.is_contiguous() or w.numel() != H \
                or w.dtype != branches[0][3].dtype:
            raise KernelError("branch_norm_mix: float32 branches of the output's width, weights of one dtype")
    if out.dtype != torch.float32 or not out.is_contiguous() or out.shape[0] < n:
        raise KernelError("branch_norm_mix: a contiguous float32 output wanted")
    check(lib().fb_branch_norm_mix(B, ys, parts, strides, ws, dtype_code(branches[0][3]), coefs, float(eps),
                                   float(weight_offset), out.data_ptr(), int(n), H, _stream()), "branch_norm_mix")


def gemm_simt_grouped(a: torch.Tensor, row_index, w: torch.Tensor, tile_group: torch.Tensor, tile: int,
                      out: torch.Tensor, activation_name=None) -> None:
    """out[m] = act(a[row_index[m]] @ w[tile_group[m // tile]]^T): w is [groups, N, K]; the rows of `out` come in
    tiles of `tile` (16 or 64) that belong to one group each (negative: skipped); row_index negative = a row of
    zeros, None = row m itself."""
    _cuda(a, row_index, w, tile_group, out)
    _i32(row_index, "row_index")
    _i32(tile_group, "tile_group")
    if w.dim() != 3 or not w.is_contiguous():
        raise KernelError("grouped gemm: weights are contiguous [groups, N, K]")
    _, N, K = w.shape
    M = out.shape[0]
    if a.shape[1] != K or out.shape[1] != N or tile_group.numel() * tile < M:
        raise KernelError("grouped gemm: shapes do not agree")
    check(lib().fb_gemm_simt_grouped(a.data_ptr(), dtype_code(a), _rows(a), _ptr(row_index), w.data_ptr(),
                                     dtype_code(w), K, N * K, tile_group.data_ptr(), int(tile), out.data_ptr(),
                                     dtype_code(out), _rows(out), M, N, K, plain_activation_code(activation_name),
                                     _stream()), "gemm_simt_grouped", (M, N, K))


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T, float32 accumulation on the CUDA cores."""
    _cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    check(lib().fb_gemm_simt(a.data_ptr(), dtype_code(a), _rows(a), w.data_ptr(), dtype_code(w), _rows(w),
                             out.data_ptr(), dtype_code(out), _rows(out), M, N, K, _stream()), "gemm_simt", (M, N, K))


def _slopes(score_slopes, nh: int) -> int:
    """The address of the per-head slopes (float32 [nh], contiguous, on the GPU), or 0 for none."""
    if score_slopes is None:
        return 0
    if not score_slopes.is_cuda or score_slopes.dtype != torch.float32 or score_slopes.numel() != nh \
            or not score_slopes.is_contiguous():
        raise KernelError(f"attention: score slopes must be {nh} contiguous float32 on the GPU, one per query head")
    return score_slopes.data_ptr()


def paged_attention_simt(q, out, k_pool, v_pool, block_table, positions, row_seq, nh: int, nkv: int, hd: int,
                         window: int, scale: float, status, table_base=None, score_slopes=None, sinks=None,
                         vd: int = 0, keep_first: int = 0, table_head: int = 0) -> None:
    """score_slopes (float32 per query head, optional): slope * (key position - query position) is added to every
    scaled score, a linear penalty on distance.  sinks (float32 per query head, optional): one more softmax slot per
    head whose score is that number, unscaled, and which has no value.  vd: the size of a value row where it is not
    the key row's (the output then has nh * vd columns).  keep_first: under a window, the keys at positions below
    this stay visible to every later query."""
    _cuda(q, out, k_pool, v_pool, block_table, positions, row_seq, status, table_base, sinks)
    _i32(table_base, "table_base")
    n = q.shape[0]
    vd = int(vd) or hd
    n_pages, pool_kv, page_size, pool_hd = k_pool.shape
    if pool_kv != nkv or pool_hd != hd or q.shape[1] != nh * hd or out.shape[1] != nh * vd or out.shape[0] != n \
            or tuple(v_pool.shape) != (n_pages, nkv, page_size, vd):
        raise KernelError("attention: shapes do not match the head counts")
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != nh or not sinks.is_contiguous()):
        raise KernelError("attention: sinks are one float32 per query head")
    if not (q.dtype == out.dtype == k_pool.dtype == v_pool.dtype):
        raise KernelError("attention: q, out and the cache must share one dtype")
    if not k_pool.is_contiguous() or not v_pool.is_contiguous():
        raise KernelError("attention: cache pools must be contiguous")
    check(lib().fb_paged_attention_simt(
        q.data_ptr(), _rows(q), out.data_ptr(), _rows(out), dtype_code(q), k_pool.data_ptr(), v_pool.data_ptr(),
        page_size, n_pages, block_table.data_ptr(), block_table.stride(0), _ptr(table_base), int(table_head),
        positions.data_ptr(), row_seq.data_ptr(), n, nh, nkv, hd, vd, int(window), int(keep_first), float(scale), _slopes(score_slopes, nh),
        _ptr(sinks), status.data_ptr(), _stream()), "paged_attention_simt")


def apply_penalties(logits, rows, tokens, counts, repetition, presence, frequency) -> None:
    _cuda(logits, rows, tokens, counts, repetition, presence, frequency)
    check(lib().fb_apply_penalties(logits.data_ptr(), _rows(logits), logits.shape[1], rows.data_ptr(),
                                   tokens.data_ptr(), counts.data_ptr(), repetition.data_ptr(),
                                   presence.data_ptr(), frequency.data_ptr(), rows.numel(), _stream()),
          "apply_penalties")


def apply_logit_bias(logits, rows, tokens, bias) -> None:
    _cuda(logits, rows, tokens, bias)
    check(lib().fb_apply_logit_bias(logits.data_ptr(), _rows(logits), logits.shape[1], rows.data_ptr(),
                                    tokens.data_ptr(), bias.data_ptr(), rows.numel(), _stream()),
          "apply_logit_bias")


def sample(logits, out, temperature=None, uniform=None, top_k=None, top_p=None, min_p=None, n=None) -> None:
    """out[r] = argmax(logits[r]) where temperature[r] <= 0 (or no temperature given), else a draw."""
    _cuda(logits, out, temperature, uniform, top_k, top_p, min_p)
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    _i32(out, "sampled tokens")
    _i32(top_k, "top_k")
    n = logits.shape[0] if n is None else n
    check(lib().fb_sample(logits.data_ptr(), _rows(logits), n, logits.shape[1], _ptr(temperature), _ptr(uniform),
                          _ptr(top_k), _ptr(top_p), _ptr(min_p), out.data_ptr(), _stream()), "sample")


# ---------------------------------------------------------------------------
# choices between kernels of one family
# ---------------------------------------------------------------------------

class _SplitScratch:
    """Float32 partial tiles and per-tile arrival counters of the split-K tensor-core product, per device.
    Kernels of one stream run in order, so one buffer serves every product of the step."""
    PARTIAL_FLOATS = 16 << 20
    COUNTERS = 8192
    _by_device: dict = {}

    @classmethod
    def get(cls, device):
        hit = cls._by_device.get(device)
        if hit is None:
            hit = (torch.empty(cls.PARTIAL_FLOATS, dtype=torch.float32, device=device),
                   torch.zeros(cls.COUNTERS, dtype=torch.int32, device=device))
            cls._by_device[device] = hit
        return hit


def tc_supported(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether the tcgen05 product takes these operands: bfloat16, 16-byte aligned, row strides of 8 elements."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype in _CODES
            and a.dim() == 2 and w.dim() == 2 and a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_SPLITS_USED = ctypes.c_int(1)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor, splits: int = 0,
            slabs: torch.Tensor | None = None) -> int:
    """out[M,N] = a[M,K] @ w[N,K]^T on the tensor cores (bfloat16 operands, float32 accumulation).
    splits = 0 lets the launcher choose the split of K.  With `slabs` (float32 [P, M, N], out = slabs[0]) each
    split writes its share into its own slab and the count of slabs to add is returned; otherwise the kernel
    adds the shares itself and 1 is returned."""
    _cuda(a, w, out, status)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: operands must be bfloat16")
    slab_stride = max_slabs = 0
    if slabs is not None:
        if slabs.dtype != torch.float32 or slabs.dim() != 3 or slabs.data_ptr() != out.data_ptr():
            raise KernelError("gemm_tc: slabs must be float32 [P, M, N] with out = slabs[0]")
        slab_stride, max_slabs = slabs.stride(0), slabs.shape[0]
    partials, counters = _SplitScratch.get(a.device)
    check(lib().fb_gemm_tc(a.data_ptr(), _rows(a), w.data_ptr(), _rows(w), out.data_ptr(), dtype_code(out),
                           _rows(out), slab_stride, max_slabs, ctypes.byref(_SPLITS_USED), M, N, K,
                           partials.data_ptr(), partials.numel(), counters.data_ptr(), counters.numel(),
                           int(splits), status.data_ptr(), _stream()), "gemm_tc", (M, N, K))
    return _SPLITS_USED.value if slabs is not None else 1


def gemm_tc_add(a: torch.Tensor, w: torch.Tensor, acc: torch.Tensor, status: torch.Tensor, max_slabs: int = 1) -> bool:
    """acc[M,N] += a[M,K] @ w[N,K]^T in float32, where the product is one the two-SM tensor-core kernel takes in
    whole tiles (hundreds of rows, and no split of K would be chosen although `max_slabs` slabs could be had): each
    element of acc gets one float32 add from the kernel's epilogue.  Returns False, having done nothing, for any
    other product: the caller then leaves the output where another kernel adds it."""
    _cuda(a, w, acc, status)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or acc.shape[0] < M or acc.shape[1] != N:
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} acc{tuple(acc.shape)} do not agree")
    if acc.dtype != torch.float32 or not tc_supported(a, w, acc) or M <= 128:
        return False
    rc = lib().fb_gemm_tc_add(a.data_ptr(), _rows(a), w.data_ptr(), _rows(w), acc.data_ptr(), _rows(acc),
                              int(max_slabs), M, N, K, status.data_ptr(), _stream())
    if rc == 0:
        return False                         # nothing was launched
    check(0 if rc == 1 else rc, "gemm_tc_add", (M, N, K))
    return True


def gemm_tc_gated(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
                  activation: str = "silu") -> None:
    """out[M, N/2] = act(g) * u where (g_0, u_0, g_1, u_1, ...) = a @ w^T: w stacks gate and up rows alternately
    and the activation runs in the product's epilogue."""
    _cuda(a, w, out, status)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] * 2 != N:
        raise KernelError(f"gated gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    partials, counters = _SplitScratch.get(a.device)
    check(lib().fb_gemm_tc_gated(a.data_ptr(), _rows(a), w.data_ptr(), _rows(w), out.data_ptr(), dtype_code(out),
                                 _rows(out), M, N, K, activation_code(activation), partials.data_ptr(),
                                 partials.numel(), counters.data_ptr(), counters.numel(), status.data_ptr(),
                                 _stream()), "gemm_tc_gated", (M, N, K))


def gemm_tc_act(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor, activation_name: str) -> None:
    """out[M, N] = act(a @ w^T) with a plain activation (PLAIN_ACTIVATIONS) in the product's epilogue."""
    _cuda(a, w, out, status)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    check(lib().fb_gemm_tc_act(a.data_ptr(), _rows(a), w.data_ptr(), _rows(w), out.data_ptr(), dtype_code(out),
                               _rows(out), M, N, K, plain_activation_code(activation_name), status.data_ptr(),
                               _stream()), "gemm_tc_act", (M, N, K))


def linear_slabs(a: torch.Tensor, w: torch.Tensor, slabs: torch.Tensor, ctx) -> int:
    """slabs[0] + ... + slabs[k-1] = a @ w^T; returns k.  The tensor-core kernel leaves the split-K shares for the
    next kernel to add; every other path writes the whole product into slabs[0]."""
    out = slabs[0]
    if slabs.shape[0] > 1 and tc_supported(a, w, out):
        return gemm_tc(a, w, out, ctx.runtime.status, slabs=slabs)
    linear(a, w, out, ctx)
    return 1


def grouped_tc_supported(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel takes a grouped product: bfloat16 operands whose rows TMA can fetch."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype in (torch.float32, torch.bfloat16)
            and a.dim() == 2 and a.stride(1) == 1 and a.stride(0) % 8 == 0 and w.shape[-1] % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous()
            and _GROUPED_TC[0])


_GROUPED_TC = [os.environ.get("FLAMBEAU_MOE_TC", "1") != "0"]


def grouped_tile(pairs: int, groups: int, tensor_cores: bool) -> int:
    """Rows of a tile of the grouped products for `pairs` rows spread over `groups` groups: small tiles while a
    group holds few rows (decoding: a tile of 16 streams an expert's weights once), larger ones as the groups fill
    (128 on the tensor cores, whose instruction takes as long for 64 columns as for 128)."""
    if pairs <= 16 * groups:
        return 16
    if tensor_cores and pairs >= 192 * groups:
        return 128
    return 64


def gather_rows(h: torch.Tensor, place_token: torch.Tensor, out: torch.Tensor, share=None, place_pair=None) -> None:
    """out[i] = h[place_token[i]], zeros where place_token[i] < 0.  With share (float32, one per (token, choice) pair)
    and place_pair (the pair of every place): out[i] = share[place_pair[i]] * h[place_token[i]]."""
    _cuda(h, place_token, out, share, place_pair)
    _i32(place_token, "place_token")
    _i32(place_pair, "place_pair")
    if (share is None) != (place_pair is None) or (share is not None and share.dtype != torch.float32):
        raise KernelError("gather_rows: float32 shares come with the pair of every place")
    rows, D = out.shape
    if h.dtype != out.dtype or h.shape[1] != D or not out.is_contiguous() or place_token.numel() < rows:
        raise KernelError("gather_rows: shapes or dtypes do not agree")
    check(lib().fb_moe_gather_rows(h.data_ptr(), _rows(h), dtype_code(h), place_token.data_ptr(), out.data_ptr(), rows,
                                   D, _ptr(share), _ptr(place_pair), _stream()), "moe_gather_rows")


def gemm_tc_grouped(a: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, tile: int, out: torch.Tensor,
                    status: torch.Tensor, activation_name=None) -> None:
    """out[m] = act(a[m] @ w[tile_group[m // tile]]^T) on the tcgen05 kernel; a [M, K] with M whole tiles."""
    _cuda(a, w, tile_group, out, status)
    _i32(tile_group, "tile_group")
    groups, N, K = w.shape
    M = out.shape[0]
    if a.shape[0] != M or a.shape[1] != K or out.shape[1] != N or tile_group.numel() * tile < M:
        raise KernelError("grouped gemm: shapes do not agree")
    check(lib().fb_gemm_tc_grouped(a.data_ptr(), _rows(a), w.data_ptr(), K, groups, tile_group.data_ptr(), int(tile),
                                   out.data_ptr(), dtype_code(out), _rows(out), M, N, K,
                                   plain_activation_code(activation_name), status.data_ptr(), _stream()),
          "gemm_tc_grouped", (M, N, K))


def gemm_tc_grouped_gated(a: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, tile: int, out: torch.Tensor,
                          status: torch.Tensor, activation: str) -> None:
    """out[m, c] = act(g_c) * u_c with (g_0, u_0, g_1, u_1, ...) = a[m] @ w[tile_group[m // tile]]^T on the tcgen05
    kernel: w [groups, 2 I, K] stacks every group's gate and up rows alternately, out has I columns."""
    _cuda(a, w, tile_group, out, status)
    _i32(tile_group, "tile_group")
    groups, N, K = w.shape
    M = out.shape[0]
    if a.shape[0] != M or a.shape[1] != K or out.shape[1] * 2 != N or tile_group.numel() * tile < M:
        raise KernelError("grouped gated gemm: shapes do not agree")
    check(lib().fb_gemm_tc_grouped_gated(a.data_ptr(), _rows(a), w.data_ptr(), K, groups, tile_group.data_ptr(),
                                         int(tile), out.data_ptr(), dtype_code(out), _rows(out), M, N, K,
                                         activation_code(activation), status.data_ptr(), _stream()),
          "gemm_tc_grouped_gated", (M, N, K))


def grouped_gated_linear(a: torch.Tensor, row_index, w: torch.Tensor, tile_group: torch.Tensor, tile: int,
                         out: torch.Tensor, activation: str, ctx, row_share=None, row_pair=None) -> None:
    """out[m] = act(gate) * up of a[row_index[m]] under the weights of the row tile's group (w [groups, 2 I, K], gate
    and up rows alternating): on the tcgen05 kernel with the activation in its epilogue for bfloat16 operands, else
    the float32-FMA grouped product followed by the activation kernel.  row_share / row_pair (with row_index): the
    fetched row is multiplied by row_share[row_pair[m]] on its way (see gather_rows)."""
    if grouped_tc_supported(a, w, out):
        with ctx.ws.scope():
            side = a
            if row_index is not None:
                side = ctx.ws.alloc((out.shape[0], a.shape[1]), a.dtype)
                gather_rows(a, row_index, side, row_share, row_pair)
            gemm_tc_grouped_gated(side, w, tile_group, tile, out, ctx.runtime.status, activation)
        return
    if tile not in (16, 64):
        raise KernelError(f"grouped gemm: the float32-FMA kernel takes tiles of 16 or 64 rows, not {tile}")
    with ctx.ws.scope():
        if row_share is not None:           # the scaled rows side by side first; the product then reads them in order
            side = ctx.ws.alloc((out.shape[0], a.shape[1]), a.dtype)
            gather_rows(a, row_index, side, row_share, row_pair)
            a, row_index = side, None
        gu = ctx.ws.alloc((out.shape[0], w.shape[1]), torch.float32)
        gemm_simt_grouped(a, row_index, w, tile_group, tile, gu, None)
        gate_mul(gu, out, activation=activation)


def grouped_linear(a: torch.Tensor, row_index, w: torch.Tensor, tile_group: torch.Tensor, tile: int,
                   out: torch.Tensor, activation_name=None, ctx=None, row_share=None, row_pair=None) -> None:
    """out[m] = act(a[row_index[m]] @ w[tile_group[m // tile]]^T) with w [groups, N, K]: the product of routed
    experts over rows that were sorted by expert and padded to whole tiles.  bfloat16 operands go to the tcgen05
    kernel (rows that have to be fetched through row_index are first laid side by side, since tensor-map copies
    take whole tiles of consecutive rows); everything else to the float32-FMA kernel, which fetches by index."""
    if ctx is not None and grouped_tc_supported(a, w, out):
        if row_index is not None:
            with ctx.ws.scope():
                side = ctx.ws.alloc((out.shape[0], a.shape[1]), a.dtype)
                gather_rows(a, row_index, side, row_share, row_pair)
                gemm_tc_grouped(side, w, tile_group, tile, out, ctx.runtime.status, activation_name)
        else:
            gemm_tc_grouped(a, w, tile_group, tile, out, ctx.runtime.status, activation_name)
        return
    if tile not in (16, 64):
        raise KernelError(f"grouped gemm: the float32-FMA kernel takes tiles of 16 or 64 rows, not {tile}")
    if row_share is not None:
        if ctx is None:
            raise KernelError("grouped gemm: rows scaled on their way need the step's scratch (ctx)")
        with ctx.ws.scope():
            side = ctx.ws.alloc((out.shape[0], a.shape[1]), a.dtype)
            gather_rows(a, row_index, side, row_share, row_pair)
            gemm_simt_grouped(side, None, w, tile_group, tile, out, activation_name)
        return
    gemm_simt_grouped(a, row_index, w, tile_group, tile, out, activation_name)


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ctx=None) -> None:
    """out = a @ w^T with the kernel that fits the dtypes and the shape: the tcgen05 kernel for bfloat16
    operands it can fetch by TMA, the float32-FMA kernel for everything else (all of the 32-bit mode)."""
    if ctx is not None and tc_supported(a, w, out):
        gemm_tc(a, w, out, ctx.runtime.status)
    else:
        gemm_simt(a, w, out)


class _AttentionScratch:
    """Float32 partial outputs of the split-key attention arrangement and its per-pair arrival counters, per
    device.  The counters must be zero between launches: the kernel leaves them so.  The buffer grows with the
    largest step seen; outgrown buffers stay alive because captured graphs may hold their addresses."""
    _by_device: dict = {}
    _outgrown: list = []

    @classmethod
    def get(cls, device, n_seqs: int, nkv: int, hd: int):
        hd_max = 32 if hd <= 32 else 64 if hd <= 64 else 128 if hd <= 128 else 256
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        pairs = n_seqs * nkv
        # 65536 counters, then one partial per slot: at most 4 resident CTAs per SM plus one slot per pair
        need = (1 << 16) + (4 * sms + pairs) * (16 * hd_max + 32)
        hit = cls._by_device.get(device)
        if hit is None or hit.numel() < need:
            if hit is not None:
                cls._outgrown.append(hit)
            floats = max(1 << 22, 1 << (need - 1).bit_length())
            hit = cls._by_device[device] = torch.zeros(floats, dtype=torch.float32, device=device)
        return hit


def prefetch_arguments(weight, budget_bytes: int = 16 << 20) -> tuple:
    """(base, rows, row stride in bytes, bytes per row) for the attention launcher's L2 hint: the first bytes of
    every row of `weight` ([rows, K], the matrix of the product that follows), `budget_bytes` in all, which the
    split-key kernel fetches into L2 when its stream of cache ends, so that the product starts on data that is
    already on the chip.  A hint: results do not depend on it; a matrix the kernel cannot take gives no hint.
    (Measured for the row-wise kernels between the products and for the products' own tails as well: there it
    costs more than it brings.)"""
    if weight is None or weight.dim() != 2 or weight.stride(1) != 1:
        return (0, 0, 0, 0)
    rows = weight.shape[0]
    row_bytes = weight.shape[1] * weight.element_size()
    per_row = min(row_bytes, max(512, (budget_bytes // max(rows, 1)) // 512 * 512)) // 16 * 16
    if per_row < 16:
        return (0, 0, 0, 0)
    return (weight.data_ptr(), rows, weight.stride(0) * weight.element_size(), per_row)


def set_gemm_pair(on: bool) -> None:
    """Products with hundreds of rows on the two-SM kernel (tcgen05 cta_group::2) where there are enough tiles
    (the default), or always on the one-SM kernel."""
    lib().fb_set_gemm_pair(1 if on else 0)


def set_attention_tc(on: bool) -> None:
    """Portions of prompts on the tcgen05 attention kernel where it takes the geometry (the default), or always on
    the mma.sync kernel."""
    lib().fb_set_attention_tc(1 if on else 0)


def mma_attention_supported(q: torch.Tensor, nh: int, nkv: int, hd: int) -> bool:
    return (q.dtype == torch.bfloat16 and hd % 8 == 0 and hd <= 256 and nh % nkv == 0 and nh // nkv <= 64
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


def paged_attention_mma(q, out, k_pool, v_pool, block_table, seq_q_start, seq_q_len, seq_pos_start, n_seqs: int,
                        max_q_len: int, max_kv_len: int, any_short: bool, any_long: bool, nh: int, nkv: int,
                        hd: int, window: int, scale: float, status, table_base=None, prefetch=None,
                        multi_seqs=None, n_multi: int = 0, score_slopes=None, sinks=None,
                        weights_float32: bool = False, keep_first: int = 0, table_head: int = 0) -> None:
    """bfloat16 attention on the tensor cores over the paged cache; sequences are described per entry of the
    step (first row, rows, first position).  any_short / any_long say whether the step holds sequences with
    rows * (nh/nkv) <= 16 / > 16 (attention_is_short), which run in different arrangements of the kernel.  table_base (int32 per
    sequence, optional): the logical page that column 0 of each table row stands for.  prefetch (optional): the
    weight matrix of the product that follows (see prefetch_arguments).  multi_seqs (int32, optional): the
    n_multi sequences of the step that bring more than one token; the kernels for portions then lay their grid over
    these instead of over every sequence.  score_slopes (float32 per query head, optional): slope * (key position -
    query position) is added to every scaled score; portions then run on the mma.sync kernel.  sinks (float32 per
    query head, optional): one more softmax slot per head, its score that number unscaled, without key or value.
    weights_float32: the softmax weights enter P V as two bfloat16 numbers each (the rounded weight and what the
    rounding left: 16 bits of mantissa, two MMAs for one) instead of rounded to bfloat16; portions then run on the
    mma.sync kernel, whose weights are in registers.  keep_first: under a window, the keys at positions below this
    stay visible to every later query (their tiles are walked ahead of the window's; portions then run on the
    mma.sync kernel)."""
    _cuda(q, out, k_pool, v_pool, block_table, seq_q_start, seq_q_len, seq_pos_start, status, table_base, multi_seqs,
          sinks)
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != nh or not sinks.is_contiguous()):
        raise KernelError("attention: sinks are one float32 per query head")
    _i32(table_base, "table_base")
    _i32(multi_seqs, "multi_seqs")
    n_pages, pool_kv, page_size, pool_hd = k_pool.shape
    if pool_kv != nkv or pool_hd != hd or q.shape[1] != nh * hd or out.shape[1] != nh * hd:
        raise KernelError("attention: shapes do not match the head counts")
    if not (q.dtype == out.dtype == k_pool.dtype == v_pool.dtype == torch.bfloat16):
        raise KernelError("attention_mma: q, out and the cache must be bfloat16")
    if not k_pool.is_contiguous() or not v_pool.is_contiguous():
        raise KernelError("attention: cache pools must be contiguous")
    scratch = _AttentionScratch.get(q.device, n_seqs, nkv * attention_kv_share(nh, nkv), hd)
    check(lib().fb_paged_attention_mma(
        q.data_ptr(), _rows(q), out.data_ptr(), _rows(out), k_pool.data_ptr(), v_pool.data_ptr(), page_size, n_pages,
        block_table.data_ptr(), block_table.stride(0), _ptr(table_base), int(table_head), seq_q_start.data_ptr(),
        seq_q_len.data_ptr(), seq_pos_start.data_ptr(), _ptr(multi_seqs), int(n_multi), n_seqs, max_q_len, max_kv_len,
        1 if any_short else 0,
        1 if any_long else 0, nh, nkv, hd, int(window), int(keep_first), float(scale), _slopes(score_slopes, nh), _ptr(sinks),
        1 if weights_float32 else 0, scratch.data_ptr(), scratch.numel(),
        *prefetch_arguments(prefetch), status.data_ptr(), _stream()), "paged_attention_mma", (n_seqs, nkv, hd))


def attention_kv_share(nh: int, nkv: int) -> int:
    """Into how many equal stretches of at most 16 heads the split-key arrangement cuts a group of nh / nkv query
    heads (1 up to 16 heads; the launcher's own number, csrc/attention_mma.cu)."""
    G = nh // nkv if nkv > 0 else 1
    if G <= 16:
        return 1
    return next((s for s in range(2, G) if G % s == 0 and G // s <= 16), G)


def attention_is_short(q_len: int, nh: int, nkv: int) -> bool:
    """Whether a sequence that brings q_len tokens runs in the split-key arrangement of paged_attention_mma (its
    tokens x the query heads of a stretch fit 16 rows) rather than in the arrangement for portions."""
    return q_len * ((nh // nkv) // attention_kv_share(nh, nkv)) <= 16


def paged_attention(ctx, q, out, cache, nh: int, nkv: int, hd: int, window: int, scale: float,
                    next_weight=None, score_slopes=None, sinks=None, vd: int = 0, weights_float32: bool = False,
                    keep_first: int = 0) -> None:
    """Attention of every row of the step over its request's cached keys: the tensor-core kernel for bfloat16
    and head sizes it takes, the float32 CUDA-core kernel otherwise (all of the 32-bit mode).  next_weight: the
    matrix of the product that follows, whose start the bfloat16 kernel may fetch into L2 (a hint)."""
    b = ctx.batch
    vd = int(vd) or hd
    if mma_attention_supported(q, nh, nkv, hd) and vd == hd:
        short = [attention_is_short(ql, nh, nkv) for ql in b.seq_q_len]
        paged_attention_mma(q, out, cache.k_pool, cache.v_pool, cache.block_table, b.seq_q_start_d, b.seq_q_len_d,
                            b.seq_pos_start_d, b.n_seqs, b.max_q_len, b.max_kv_len, any(short), not all(short),
                            nh, nkv, hd, window, scale, ctx.runtime.status, table_base=cache.table_base,
                            prefetch=next_weight, multi_seqs=b.multi_seqs_d, n_multi=b.n_multi,
                            score_slopes=score_slopes, sinks=sinks, weights_float32=weights_float32,
                            keep_first=keep_first, table_head=cache.table_head)
    else:
        paged_attention_simt(q, out, cache.k_pool, cache.v_pool, cache.block_table, b.positions, b.row_seq,
                             nh, nkv, hd, window, scale, ctx.runtime.status, table_base=cache.table_base,
                             score_slopes=score_slopes, sinks=sinks, vd=vd, keep_first=keep_first,
                             table_head=cache.table_head)


def diff_attention_mma_supported(q: torch.Tensor, nh: int, nkv: int, kd: int, vd: int) -> bool:
    """Whether the tensor-core arrangements take this geometry: bfloat16, key size (per map) a multiple of 16 up to
    128, value size a multiple of 16 up to 256."""
    return (q.dtype == torch.bfloat16 and kd % 16 == 0 and 16 <= kd <= 128 and vd % 16 == 0 and 16 <= vd <= 256
            and nh % nkv == 0 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


def diff_attention_mma(q, out, gate, cache, seq_q_start, seq_q_len, seq_pos_start, n_seqs: int, max_q_len: int,
                       max_kv_len: int, any_short: bool, any_long: bool, nh: int, nkv: int, kd: int, vd: int,
                       window: int, scale: float, lam: float, eps: float, out_scale: float, status, alloc=None) -> None:
    """Differential attention on the tensor cores (csrc/diff_attention_mma.cu).  Sequences are described per entry of
    the step (first row, rows, first position); any_short / any_long say whether the step holds sequences with
    rows * (nh / nkv) <= 16 / > 16, which run in the split-key and in the portion arrangement.  `alloc(n)` returns
    n float32 of scratch for the split arrangement's partials (default: a fresh tensor)."""
    _cuda(q, out, gate, seq_q_start, seq_q_len, seq_pos_start, status)
    k_pool, v_pool = cache.k_pool, cache.v_pool
    n_pages = k_pool.shape[0]
    n = q.shape[0]
    if q.shape[1] != nh * 2 * kd or tuple(out.shape) != (n, nh * vd) or tuple(k_pool.shape[1:]) != (nkv, cache.page_size, 2 * kd) \
            or tuple(v_pool.shape[1:]) != (nkv, cache.page_size, vd):
        raise KernelError("diff attention: shapes do not match the head counts")
    if not (q.dtype == out.dtype == k_pool.dtype == v_pool.dtype == torch.bfloat16):
        raise KernelError("diff_attention_mma: q, out and the cache must be bfloat16")
    if not k_pool.is_contiguous() or not v_pool.is_contiguous():
        raise KernelError("diff attention: cache pools must be contiguous")
    if gate is not None and (gate.dtype != torch.float32 or tuple(gate.shape) != (n, nh) or not gate.is_contiguous()):
        raise KernelError("diff attention: the gate wants contiguous float32 [n, heads]")
    splits, scratch = 1, None
    if any_short:
        max_keys = min(max_kv_len, window + 16) if window > 0 else max_kv_len
        splits = lib().fb_diff_attention_splits(n_seqs, nkv, max(1, int(max_keys)), kd, vd)
        floats = lib().fb_diff_attention_scratch_floats(n_seqs, nkv, vd, splits)
        scratch = alloc(floats) if alloc is not None else torch.empty(floats, dtype=torch.float32, device=q.device)
    check(lib().fb_diff_attention_mma(
        q.data_ptr(), _rows(q), out.data_ptr(), _rows(out), _ptr(gate), k_pool.data_ptr(), v_pool.data_ptr(),
        cache.page_size, n_pages, cache.block_table.data_ptr(), cache.block_table.stride(0), _ptr(cache.table_base),
        seq_q_start.data_ptr(), seq_q_len.data_ptr(), seq_pos_start.data_ptr(), n_seqs, max_q_len,
        1 if any_short else 0, 1 if any_long else 0, nh, nkv, kd, vd, int(window), float(scale), float(lam),
        float(eps), float(out_scale), splits, _ptr(scratch), scratch.numel() if scratch is not None else 0,
        status.data_ptr(), _stream()), "diff_attention_mma")


def diff_attention(ctx, q, out, gate, cache, nh: int, nkv: int, kd: int, vd: int, window: int, scale: float,
                   lam: float, eps: float, out_scale: float) -> None:
    """Differential attention of every row of the step over its request's cached keys and values, with the kernel
    that fits the dtype and the sizes: the tensor-core arrangements for bfloat16 and sizes they take, the
    float32-math kernel otherwise (all of the 32-bit mode)."""
    b = ctx.batch
    if diff_attention_mma_supported(q, nh, nkv, kd, vd) and scale > 0.0 and _DIFF_MMA[0]:
        G = nh // nkv
        short = [ql * G <= 16 for ql in b.seq_q_len]
        # A step of single tokens may be replayed from a CUDA graph at any context length: its split of the keys
        # (and the scratch that goes with it) is sized by the longest context the engine allows, in the eager run
        # as in the captured one, so that both take the same memory.
        longest = ctx.engine.max_seq_len if b.max_q_len == 1 else b.max_kv_len
        diff_attention_mma(q, out, gate, cache, b.seq_q_start_d, b.seq_q_len_d, b.seq_pos_start_d, b.n_seqs,
                           b.max_q_len, longest, any(short), not all(short), nh, nkv, kd, vd, window, scale, lam,
                           eps, out_scale, ctx.runtime.status,
                           alloc=lambda n: ctx.ws.alloc((n,), torch.float32))
    else:
        diff_attention_simt(q, out, gate, cache, b.positions, b.row_seq, nh, nkv, kd, vd, window, scale, lam, eps,
                            out_scale, ctx.runtime.status)


_DIFF_MMA = [os.environ.get("FLAMBEAU_DIFF_ATTN_MMA", "1") != "0"]


def set_diff_attention_mma(on: bool) -> None:
    """Differential attention in bfloat16 on the tensor-core arrangements where they take the geometry (the default),
    or always on the float32-math kernel."""
    _DIFF_MMA[0] = bool(on)


# ---------------------------------------------------------------------------
# query/key norm + rotation + cache write behind a fused projection
# ---------------------------------------------------------------------------
QK_NORM_REACH = {None: 0, "none": 0, "head": 1, "projection": 2}


def qk_norm_rope_kv_write(proj: torch.Tensor, q_weight, k_weight, reach, eps: float, weight_offset: float, cos, sin,
                          half: int, q_out: torch.Tensor, cache, positions, row_seq, nh: int, nkv: int, hd: int,
                          vd: int, status, n_partials: int = 1, partial_stride: int = 0) -> None:
    """proj: float32 rows [q: nh*hd | k: nkv*hd | v: nkv*vd] (possibly split-K shares).  q and k pass an RMS norm
    whose reach is a head ('head': weights [hd]) or the whole projection ('projection': weights [nh*hd] and
    [nkv*hd]) or none, then the rotation of the first 2*half dimensions of every head (cos/sin float32 [n, half]);
    q goes to q_out in its dtype, k and v into the cache's pages when the view is writable."""
    _cuda(proj, q_weight, k_weight, cos, sin, q_out, positions, row_seq, status)
    n = proj.shape[0]
    code = QK_NORM_REACH[reach]
    if proj.dtype != torch.float32 or tuple(q_out.shape) != (n, nh * hd):
        raise KernelError("qk_norm_rope_kv_write: float32 projection rows and q [n, heads * size] wanted")
    if code:
        want = (hd, hd) if code == 1 else (nh * hd, nkv * hd)
        if q_weight is None or k_weight is None or (q_weight.numel(), k_weight.numel()) != want \
                or q_weight.dtype != k_weight.dtype:
            raise KernelError("qk_norm_rope_kv_write: the norm weights do not fit the norm's reach")
    k_pool, v_pool = cache.k_pool, cache.v_pool
    n_pages = k_pool.shape[0]
    if tuple(k_pool.shape) != (n_pages, nkv, cache.page_size, hd) or tuple(v_pool.shape) != (n_pages, nkv, cache.page_size, vd) \
            or not k_pool.is_contiguous() or not v_pool.is_contiguous() or k_pool.dtype != q_out.dtype:
        raise KernelError("qk_norm_rope_kv_write: the cache pools do not fit the head sizes")
    check(lib().fb_qk_norm_rope_kv_write(
        proj.data_ptr(), _rows(proj), int(n_partials), int(partial_stride), _ptr(q_weight), _ptr(k_weight),
        dtype_code(q_weight) if q_weight is not None else 0, code, float(eps), float(weight_offset), _ptr(cos),
        _ptr(sin), int(half), q_out.data_ptr(), _rows(q_out), dtype_code(q_out), positions.data_ptr(),
        row_seq.data_ptr(), cache.block_table.data_ptr(), cache.block_table.stride(0), _ptr(cache.table_base),
        int(cache.table_head), k_pool.data_ptr(), v_pool.data_ptr(), cache.page_size, n_pages, n, nh, nkv, hd, vd,
        1 if cache.writable else 0, status.data_ptr(), _stream()), "qk_norm_rope_kv_write")


# ---------------------------------------------------------------------------
# gated delta rule
# ---------------------------------------------------------------------------
def gdr_prepare(proj, conv_w, taps: int, a_log, dt_bias, state, tail_off: int, batch, qkv, beta, decay, G: int,
                H: int, dk: int, dv: int, q_scale: float, unit_eps: float, n_partials: int = 1,
                partial_stride: int = 0) -> None:
    """The step's tokens made ready for the recurrence (csrc/gated_delta.cu: gdr_prepare, gdr_conv_tail).  proj:
    float32 rows [q | k | v | b | a | gate] (possibly shares); state: float32 [slots, floats per slot] with the
    convolution's tail at `tail_off`; qkv, beta, decay: float32 outputs [n, C], [n, H], [n, H]."""
    _cuda(proj, conv_w, a_log, dt_bias, state, qkv, beta, decay)
    n = proj.shape[0]
    C = 2 * G * dk + H * dv
    if proj.dtype != torch.float32 or state.dtype != torch.float32 or not state.is_contiguous() or state.dim() != 2 \
            or tuple(qkv.shape) != (n, C) or tuple(beta.shape) != (n, H) or tuple(decay.shape) != (n, H) \
            or tuple(conv_w.shape) != (C, taps) or not conv_w.is_contiguous() \
            or not (conv_w.dtype == a_log.dtype == dt_bias.dtype) \
            or any(t.dtype != torch.float32 or not t.is_contiguous() for t in (qkv, beta, decay)):
        raise KernelError("gated delta: bad shapes or dtypes")
    if state.shape[1] < tail_off + (taps - 1) * C:
        raise KernelError("gated delta: the state slot is too small for the convolution's tail")
    check(lib().fb_gdr_prepare(proj.data_ptr(), _rows(proj), int(n_partials), int(partial_stride), conv_w.data_ptr(),
                               int(taps), a_log.data_ptr(), dt_bias.data_ptr(), dtype_code(conv_w), state.data_ptr(),
                               state.stride(0), int(tail_off), batch.row_seq.data_ptr(), batch.seq_q_start_d.data_ptr(),
                               batch.seq_q_len_d.data_ptr(), batch.seq_slot_d.data_ptr(), batch.n_seqs,
                               qkv.data_ptr(), beta.data_ptr(), decay.data_ptr(), n, G, H, dk, dv, float(q_scale),
                               float(unit_eps), _stream()), "gdr_prepare")


def gdr_recurrent(qkv, beta, decay, state, batch, o, G: int, H: int, dk: int, dv: int) -> None:
    """S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q over the step's tokens of every request, the state
    [H][dk][dv] at the start of the request's slot."""
    _cuda(qkv, beta, decay, state, o)
    if o.dtype != torch.float32 or not o.is_contiguous() or o.shape[1] != H * dv or state.shape[1] < H * dk * dv:
        raise KernelError("gated delta: bad output or state")
    check(lib().fb_gdr_recurrent(qkv.data_ptr(), beta.data_ptr(), decay.data_ptr(), state.data_ptr(), state.stride(0),
                                 batch.seq_q_start_d.data_ptr(), batch.seq_q_len_d.data_ptr(),
                                 batch.seq_slot_d.data_ptr(), batch.n_seqs, o.data_ptr(), G, H, dk, dv, _stream()),
          "gdr_recurrent")


def gdr_out_norm(o, proj, gate_off: int, weight, eps: float, out, H: int, dv: int, n_partials: int = 1,
                 partial_stride: int = 0) -> None:
    """out = o / rms(o) * weight * silu(gate) per head, the gate taken from the projection rows at `gate_off`."""
    _cuda(o, proj, weight, out)
    n = o.shape[0]
    if tuple(out.shape) != (n, H * dv) or not out.is_contiguous() or weight.numel() != dv:
        raise KernelError("gated delta: bad output")
    check(lib().fb_gdr_out_norm(o.data_ptr(), proj.data_ptr(), _rows(proj), int(n_partials), int(partial_stride),
                                int(gate_off), weight.data_ptr(), dtype_code(weight), float(eps), out.data_ptr(),
                                dtype_code(out), n, H, dv, _stream()), "gdr_out_norm")


# ---------------------------------------------------------------------------
# routed experts
# ---------------------------------------------------------------------------
ROUTER_RULES = {"softmax_of_chosen": 0, "softmax_of_all": 1, "sigmoid": 2}


def moe_choose(z, bias, gate_col: int, experts: int, top: int, chosen, share, gate, n_partials: int = 1,
               partial_stride: int = 0, rule: str = "softmax_of_chosen", weight_scale: float = 1.0) -> None:
    """Per token: the `top` experts with the largest logits z[:, :experts] + bias (float32; z possibly split-K
    shares), their softmax weights, and (gate_col >= 0) gate = sigmoid(z[:, gate_col]).  rule 'softmax_of_all':
    scores = softmax(z) over all experts, the `top` largest of score + bias are chosen, and the weights are the chosen
    scores over their sum, times `weight_scale`.  rule 'sigmoid': scores = sigmoid of every logit by itself, the `top`
    largest of score + bias are chosen, and the weights are the chosen scores as they are, times `weight_scale`."""
    if rule not in ROUTER_RULES:
        raise KernelError(f"router: rule '{rule}' is not one of {sorted(ROUTER_RULES)}")
    _cuda(z, bias, chosen, share, gate)
    n = z.shape[0]
    if z.dtype != torch.float32 or tuple(chosen.shape) != (n, top) or chosen.dtype != torch.int32 \
            or tuple(share.shape) != (n, top) or share.dtype != torch.float32 or z.shape[1] < experts:
        raise KernelError("router: bad shapes")
    check(lib().fb_moe_choose(z.data_ptr(), _rows(z), int(n_partials), int(partial_stride), _ptr(bias),
                              dtype_code(bias) if bias is not None else 0, int(gate_col), n, int(experts), int(top),
                              chosen.data_ptr(), share.data_ptr(), _ptr(gate), ROUTER_RULES[rule],
                              float(weight_scale), _stream()), "moe_choose")


def moe_max_tiles(pairs: int, experts: int, tile: int) -> int:
    return pairs // tile + min(experts, pairs)


def moe_sort(chosen, experts: int, tile: int, place_token, pair_place, tile_expert, place_pair=None) -> None:
    """The (token, choice) pairs in expert order, every expert's stretch padded to whole row tiles.  place_pair
    (int32 [places], optional) receives, for every place that holds a token, the pair it stands for."""
    _cuda(chosen, place_token, pair_place, tile_expert, place_pair)
    _i32(place_pair, "place_pair")
    n, K = chosen.shape
    if place_pair is not None and place_pair.numel() < place_token.numel():
        raise KernelError("moe_sort: place_pair is shorter than place_token")
    check(lib().fb_moe_sort(chosen.data_ptr(), n * K, K, int(experts), int(tile), tile_expert.numel(),
                            place_token.data_ptr(), pair_place.data_ptr(), tile_expert.data_ptr(), _ptr(place_pair),
                            _stream()), "moe_sort")


def moe_combine(expert_out, pair_place, share, shared_out, shared_partials: int, shared_partial_stride: int, gate,
                out, n: int, pass_on=None) -> None:
    """out[t] = sum_k share[t, k] * expert_out[pair_place[t, k]] + gate[t] * sum of shared_out's shares (gate None:
    1).  pass_on ([n, D], optional): a pair without a place (an expert that has no weights) contributes
    share * pass_on[t].  share None: every pair counts once (experts whose share scaled what they read)."""
    _cuda(expert_out, pair_place, share, shared_out, gate, out, pass_on)
    if pass_on is not None and pass_on.shape[1] != out.shape[1]:
        raise KernelError("moe_combine: the rows handed on must have the output's width")
    D = out.shape[1]
    K = pair_place.shape[1]
    if expert_out.dtype != torch.float32 or out.dtype != torch.float32 or not out.is_contiguous() \
            or expert_out.shape[1] != D or (shared_out is not None and (shared_out.dtype != torch.float32
                                                                        or not shared_out.is_contiguous())):
        raise KernelError("moe_combine: float32 rows of the output's width wanted")
    check(lib().fb_moe_combine(expert_out.data_ptr(), _rows(expert_out), pair_place.data_ptr(), _ptr(share), K,
                               _ptr(shared_out), int(shared_partials), int(shared_partial_stride), _ptr(gate),
                               out.data_ptr(), int(n), D, _ptr(pass_on),
                               dtype_code(pass_on) if pass_on is not None else 0,
                               _rows(pass_on) if pass_on is not None else 0, _stream()), "moe_combine")


# ---------------------------------------------------------------------------
# a norm that centres; a weighted mean over depth; a convolution over time in front of a sublayer
# ---------------------------------------------------------------------------
def add_layer_norm(x: torch.Tensor, delta, weight: torch.Tensor, eps: float, out: torch.Tensor, rows=None,
                   n_partials: int = 1, n_rows: int | None = None, partial_stride: int = 0) -> None:
    """out[j] = (v - mean v) / sqrt(var v + eps) * weight with v = x[r] + sum_p delta_p[r], r = rows[j] or j; without
    `rows` the sum is also written back to x.  delta: float32 [n, H] or the first of n_partials slabs."""
    _cuda(x, delta, weight, out, rows)
    _i32(rows, "rows")
    H = x.shape[1]
    n_out = rows.numel() if rows is not None else (x.shape[0] if n_rows is None else n_rows)
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or out.shape[-1] != H \
            or weight.numel() != H or out.shape[0] < n_out:
        raise KernelError("add_layer_norm: bad shapes")
    stride = 0
    if delta is not None:
        if delta.dtype != torch.float32 or not delta.is_contiguous() or delta.shape[-1] != H:
            raise KernelError("add_layer_norm: delta must be contiguous float32 with the stream's width")
        if n_partials > 1:
            stride = int(partial_stride)
            if stride <= 0:
                raise KernelError("add_layer_norm: several slabs need their stride")
    check(lib().fb_add_layernorm(x.data_ptr(), _ptr(delta), int(n_partials) if delta is not None else 0, stride,
                                 weight.data_ptr(), dtype_code(weight), out.data_ptr(), dtype_code(out), _ptr(rows),
                                 n_out, H, float(eps), _stream()), "add_layer_norm")


def depth_average(x: torch.Tensor, delta, n_partials: int, partial_stride: int, history: torch.Tensor, count: int,
                  weights: torch.Tensor, n: int) -> None:
    """history[count - 1] = x + sum of delta's slabs; x = sum_{j < count} weights[j] * history[j], over the first n
    rows.  x float32 [>= n, H] contiguous; history float32 [slots, rows, H] contiguous."""
    _cuda(x, delta, history, weights)
    H = x.shape[1]
    if x.dtype != torch.float32 or not x.is_contiguous() or history.dtype != torch.float32 \
            or not history.is_contiguous() or history.shape[-1] != H or history.shape[1] < n \
            or not 1 <= count <= history.shape[0] or weights.numel() < count or not weights.is_contiguous():
        raise KernelError("depth_average: bad shapes")
    if delta is not None and (delta.dtype != torch.float32 or not delta.is_contiguous() or delta.shape[-1] != H):
        raise KernelError("depth_average: delta must be contiguous float32 with the stream's width")
    check(lib().fb_depth_average(x.data_ptr(), _ptr(delta), int(n_partials) if delta is not None else 0,
                                 int(partial_stride) if n_partials > 1 else 0, history.data_ptr(), history.stride(0),
                                 int(count), weights.data_ptr(), dtype_code(weights), int(n) * H, _stream()),
          "depth_average")


def time_conv(h: torch.Tensor, wt: torch.Tensor, state, tail_off: int, batch, out: torch.Tensor, n: int) -> None:
    """out[t] = h[t] + sum_j wt[j] * h[t - taps + 1 + j] per request (csrc/time_conv.cu); h float32 [n, D]; wt float32
    [taps, D] (the weights tap by tap); state float32 [slots, floats] with the kept inputs [taps - 1, D] at tail_off,
    updated for the next step."""
    _cuda(h, wt, state, out)
    taps, D = wt.shape
    if h.dtype != torch.float32 or not h.is_contiguous() or h.shape[1] != D or not out.is_contiguous() \
            or out.shape[1] != D or out.shape[0] < n or h.shape[0] < n or not wt.is_contiguous() \
            or wt.dtype != torch.float32:
        raise KernelError("time_conv: bad shapes")
    if taps > 1 and (state is None or state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous()
                     or state.shape[1] < tail_off + (taps - 1) * D):
        raise KernelError("time_conv: the state slot is too small for the kept inputs")
    check(lib().fb_time_conv(h.data_ptr(), wt.data_ptr(), int(taps), _ptr(state),
                             state.stride(0) if state is not None else 0, int(tail_off), batch.row_seq.data_ptr(),
                             batch.seq_q_start_d.data_ptr(), batch.seq_q_len_d.data_ptr(), batch.seq_slot_d.data_ptr(),
                             batch.n_seqs, out.data_ptr(), dtype_code(out), int(n), D, _stream()), "time_conv")


# ---------------------------------------------------------------------------
# gated linear attention
# ---------------------------------------------------------------------------
def gla_prepare(proj, w2, b2, tau: float, q_scale: float, qkv, decay, H: int, dk: int, dv: int, n_partials: int = 1,
                partial_stride: int = 0) -> None:
    """The step's tokens made ready for the recurrence (csrc/linear_attention.cu): proj float32 rows
    [q | k | v | gate | middle] (possibly shares); w2 [H * dk, R], b2 [H * dk]; qkv float32 [n, 2 H dk + H dv];
    decay float32 [n, H dk]."""
    _cuda(proj, w2, b2, qkv, decay)
    n = proj.shape[0]
    R = w2.shape[1]
    if proj.dtype != torch.float32 or tuple(w2.shape) != (H * dk, R) or b2.numel() != H * dk or w2.dtype != b2.dtype \
            or not w2.is_contiguous() or not b2.is_contiguous() or tuple(qkv.shape) != (n, 2 * H * dk + H * dv) \
            or tuple(decay.shape) != (n, H * dk) \
            or any(t.dtype != torch.float32 or not t.is_contiguous() for t in (qkv, decay)):
        raise KernelError("linear attention: bad shapes or dtypes")
    check(lib().fb_gla_prepare(proj.data_ptr(), _rows(proj), int(n_partials), int(partial_stride), w2.data_ptr(),
                               b2.data_ptr(), dtype_code(w2), R, float(tau), float(q_scale), qkv.data_ptr(),
                               decay.data_ptr(), n, H, dk, dv, _stream()), "gla_prepare")


def gla_recurrent(qkv, decay, state, batch, o, H: int, dk: int, dv: int) -> None:
    """S <- diag(alpha) S + k v^T; o = S^T q over the step's tokens of every request, the state [H][dv][dk] at the
    start of the request's slot."""
    _cuda(qkv, decay, state, o)
    if o.dtype != torch.float32 or not o.is_contiguous() or o.shape[1] != H * dv or state.dtype != torch.float32 \
            or state.dim() != 2 or not state.is_contiguous() or state.shape[1] < H * dk * dv:
        raise KernelError("linear attention: bad output or state")
    check(lib().fb_gla_recurrent(qkv.data_ptr(), decay.data_ptr(), state.data_ptr(), state.stride(0),
                                 batch.seq_q_start_d.data_ptr(), batch.seq_q_len_d.data_ptr(),
                                 batch.seq_slot_d.data_ptr(), batch.n_seqs, int(qkv.shape[0]), o.data_ptr(), H, dk, dv,
                                 _stream()),
          "gla_recurrent")


# ---------------------------------------------------------------------------
# latent attention
# ---------------------------------------------------------------------------
ROTARY_PAIRING = {"neighbours": 0, "halves": 1}      # which dimensions form pair i: (2i, 2i + 1) or (i, i + half)


def mla_latents(proj, Rq: int, wq, cq, kv_off: int, Rc: int, r: int, wkv, eps: float, cos, sin, half: int, cache,
                positions, row_seq, status, n_partials: int = 1, partial_stride: int = 0,
                pairing: str = "neighbours") -> None:
    """cq = rmsnorm(proj[:, :Rq]) * wq; with a writable cache also the token's cache row [rmsnorm(proj[:, kv_off:
    kv_off + Rc]) * wkv | rot(proj[:, kv_off + Rc : kv_off + Rc + r])] (csrc/latent_attention.cu)."""
    _cuda(proj, wq, cq, wkv, cos, sin, positions, row_seq, status)
    n = proj.shape[0]
    if proj.dtype != torch.float32 or wq.numel() != Rq or tuple(cq.shape) != (n, Rq) or not cq.is_contiguous():
        raise KernelError("latent attention: bad shapes")
    pool = cache.k_pool if cache is not None and cache.writable else None
    if pool is not None:
        if tuple(pool.shape[1:]) != (1, cache.page_size, Rc + r) or not pool.is_contiguous() or pool.dtype != cq.dtype \
                or wkv.numel() != Rc or wkv.dtype != wq.dtype or proj.shape[1] < kv_off + Rc + r:
            raise KernelError("latent attention: the cache rows do not fit the latent")
    check(lib().fb_mla_latents(
        proj.data_ptr(), _rows(proj), int(n_partials), int(partial_stride), Rq, wq.data_ptr(), cq.data_ptr(), kv_off,
        Rc, r, _ptr(wkv), dtype_code(wq), float(eps), _ptr(cos), _ptr(sin), half, ROTARY_PAIRING[pairing],
        _ptr(positions), _ptr(row_seq),
        _ptr(cache.block_table) if pool is not None else 0, cache.block_table.stride(0) if pool is not None else 0,
        _ptr(cache.table_base) if pool is not None else 0, _ptr(pool), dtype_code(cq),
        cache.page_size if pool is not None else 1, pool.shape[0] if pool is not None else 0, n, status.data_ptr(),
        _stream()), "mla_latents")


def head_linear(a, a_head: int, w, out, o_head: int, n: int, n_partials: int = 1, partial_stride: int = 0, gate=None,
                gate_off: int = 0, gate_partials: int = 1, gate_partial_stride: int = 0, cos=None, sin=None,
                half: int = 0, rot: int = 0, pairing: str = "neighbours") -> None:
    """out[t, h*o_head + c] = sum_k w[h, c, k] * a[t, h*a_head + k] for every head h (w [H, N, K]); `a` may be the
    first of float32 shares.  gate (float32 rows, possibly shares): the result is multiplied by
    sigmoid(gate[t, gate_off + h*N + c]).  rot > 0: columns K .. K+rot of a's head go, their first 2*half dimensions
    turned pairwise by (cos, sin), to columns N .. N+rot of out's head; `pairing` says which dimensions form a pair
    (ROTARY_PAIRING)."""
    _cuda(a, w, out, gate, cos, sin)
    H, N, K = w.shape
    if not w.is_contiguous() or a.shape[0] < n or out.shape[0] < n:
        raise KernelError("head_linear: bad shapes")
    check(lib().fb_head_linear(a.data_ptr(), dtype_code(a), _rows(a), int(a_head), int(n_partials), int(partial_stride),
                               w.data_ptr(), dtype_code(w), out.data_ptr(), dtype_code(out), _rows(out), int(o_head),
                               _ptr(gate), _rows(gate) if gate is not None else 0, int(gate_partials),
                               int(gate_partial_stride), int(gate_off), _ptr(cos), _ptr(sin), int(half), int(rot),
                               ROTARY_PAIRING[pairing], int(n), H, N, K, _stream()), "head_linear", (n * H, N, K))


def rope_neighbours(x, cos, sin, half: int, heads: int, head_dim: int) -> None:
    """In place on float32 rows [n, heads * head_dim]: dimensions (2i, 2i + 1), i < half, of every head turned by the
    tables' angles."""
    _cuda(x, cos, sin)
    if x.dtype != torch.float32 or x.shape[1] < heads * head_dim:
        raise KernelError("rope_neighbours: float32 rows of heads * head_dim wanted")
    check(lib().fb_rope_neighbours(x.data_ptr(), _rows(x), cos.data_ptr(), sin.data_ptr(), int(half), int(heads),
                                   int(head_dim), x.shape[0], _stream()), "rope_neighbours")


# ---------------------------------------------------------------------------
# an output gate on a mixer's heads; several residual streams
# ---------------------------------------------------------------------------
def sigmoid_gate(a: torch.Tensor, gate: torch.Tensor, n: int, n_partials: int = 1, partial_stride: int = 0) -> None:
    """a[t, c] *= sigmoid(sum of the shares of gate[t, c]) in place for the first n rows; gate is a float32 view
    [n, width of a] (columns of a wider product as a rule), the first of n_partials shares."""
    _cuda(a, gate)
    if gate.dtype != torch.float32 or gate.shape[1] != a.shape[1] or a.shape[0] < n or gate.shape[0] < n:
        raise KernelError("sigmoid_gate: float32 gate columns of the rows' width wanted")
    check(lib().fb_sigmoid_gate(a.data_ptr(), _rows(a), dtype_code(a), gate.data_ptr(), _rows(gate), int(n_partials),
                                int(partial_stride), int(n), a.shape[1], _stream()), "sigmoid_gate")


def hc_step(streams: torch.Tensor, y, n_partials: int, partial_stride: int, mix, out_w, in_w, norm_weight, eps: float,
            weight_offset: float, out, n: int, rows=None, write_back: bool = True) -> None:
    """One pass over the residual streams (float32 [S, n_all, D]) between two sublayers: with y (float32 [n, D], the
    first of n_partials shares) every stream becomes sum_s mix[s, t] x_s + out_w[t] y (written back unless told
    otherwise); then u = sum_t in_w[t] x_t (in_w None: ones) and out = rmsnorm(u) * (norm_weight + weight_offset), or
    u itself (float32) where norm_weight is None; out None: only the write.  rows (int32, optional): only those rows
    are formed, nothing is written back.  mix [S, S] ([from, to]), out_w [S], in_w [S]: float32."""
    _cuda(streams, y, mix, out_w, in_w, norm_weight, out, rows)
    _i32(rows, "rows")
    S, n_all, D = streams.shape
    for t in (mix, out_w, in_w):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError("hc_step: the streams' weights are contiguous float32")
    if streams.dtype != torch.float32 or streams.stride(2) != 1 or streams.stride(1) != D \
            or (y is not None and (y.dtype != torch.float32 or not y.is_contiguous() or y.shape[-1] != D)) \
            or (mix is not None and mix.numel() != S * S) or (out_w is not None and out_w.numel() != S) \
            or (in_w is not None and in_w.numel() != S) or (norm_weight is not None and norm_weight.numel() != D):
        raise KernelError("hc_step: bad shapes")
    n_out = rows.numel() if rows is not None else int(n)
    if out is not None and (not out.is_contiguous() or out.shape[-1] != D or out.shape[0] < n_out
                            or (norm_weight is None and out.dtype != torch.float32)):
        raise KernelError("hc_step: the output is contiguous rows of the streams' width (float32 without a norm)")
    if rows is not None:
        write_back = False
    check(lib().fb_hc_step(streams.data_ptr(), streams.stride(0), S, _ptr(y), int(n_partials), int(partial_stride),
                           _ptr(mix), _ptr(out_w), _ptr(in_w), _ptr(norm_weight),
                           dtype_code(norm_weight) if norm_weight is not None else 0, float(eps), float(weight_offset),
                           _ptr(out), dtype_code(out) if out is not None else 0, _ptr(rows), 1 if write_back else 0,
                           n_out, D, _stream()), "hc_step")
