"""Python faces of the CUDA kernels: each takes torch tensors on a CUDA device,
checks what the kernel assumes, and launches on torch's current stream.

The libraries are compiled and loaded on first use (``csrc/build.py``).  There is
no CPU or library fallback here: a tensor that is not on a CUDA device is an error.
``launches`` counts the kernels launched through this module (a captured CUDA
graph replays its launches without passing through here; the graph runner adds
its own count).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .csrc.build import load_library

launches = 0

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operand is not on a CUDA device (there is no CPU path)")


def _check(lib, name: str, rc: int):
    global launches
    if rc != 0:
        fn = getattr(lib, "kllm_last_error_" + name)
        fn.restype = ctypes.c_char_p
        raise KernelError(f"{name}: {fn().decode(errors='replace')} (code {rc})")
    launches += 1


def _i32(t: Optional[torch.Tensor], what: str):
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{what} must be a contiguous int32 tensor")


def _f64(t: Optional[torch.Tensor], what: str):
    if t is not None and (t.dtype != torch.float64 or not t.is_contiguous()):
        raise KernelError(f"{what} must be a contiguous float64 tensor")


def embed(out_x: torch.Tensor, table: torch.Tensor, ids: torch.Tensor,
          last_token: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """out_x[t,:] = float32(table[ids[t],:]) * scale; out_x float32 [n, d].  With ``last_token``
    (int32, one entry per request slot) an id -(s + 1) means last_token[s], the token
    that ``sample`` stored there."""
    _cuda(out_x, table, ids, last_token)
    _i32(ids, "ids"); _i32(last_token, "last_token")
    n, d = out_x.shape
    if out_x.dtype != torch.float32 or not out_x.is_contiguous() or not table.is_contiguous():
        raise KernelError("embed: residual stream must be contiguous float32")
    if table.shape[1] != d or ids.numel() != n:
        raise KernelError("embed: shapes do not agree")
    lib = load_library("embedding")
    rc = lib.kllm_embed(_p(out_x), _p(table), _p(ids), _p(last_token), n, d, table.shape[0], ctypes.c_float(scale),
                        dtype_code(table.dtype), _stream())
    _check(lib, "embedding", rc)


def gather_rows(out: torch.Tensor, src: torch.Tensor, rows: torch.Tensor) -> None:
    """out[r,:] = src[rows[r],:] for contiguous 2-D tensors of one dtype."""
    _cuda(out, src, rows)
    _i32(rows, "rows")
    if out.dtype != src.dtype or not out.is_contiguous() or not src.is_contiguous() or out.shape[1] != src.shape[1]:
        raise KernelError("gather_rows: operands do not agree")
    lib = load_library("embedding")
    rc = lib.kllm_gather_rows(_p(out), _p(src), _p(rows), rows.numel(),
                              ctypes.c_int64(src.shape[1] * src.element_size()), _stream())
    _check(lib, "embedding", rc)


def gated_slice(gate: torch.Tensor, table: torch.Tensor, offset: int, ids: torch.Tensor,
                last_token: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[n, P] in the table's dtype: gelu_tanh(gate[t, j]) * table[ids[t], offset + j], ``gate`` float32 [n, P]
    with dense rows, ``table`` contiguous [vocab, columns]: a slice of each token's row of a second embedding
    table, gated (csrc/embedding.cu).  Ids as in ``embed``."""
    _cuda(gate, table, ids, last_token)
    _i32(ids, "ids"); _i32(last_token, "last_token")
    n, P = gate.shape
    if gate.dtype != torch.float32 or gate.stride(1) != 1 or not table.is_contiguous() or ids.numel() != n \
            or offset < 0 or offset + P > table.shape[1]:
        raise KernelError("gated_slice: gate float32 [n, P] with dense rows, table contiguous with columns offset .. offset + P")
    out = torch.empty((n, P), dtype=table.dtype, device=gate.device)
    lib = load_library("embedding")
    rc = lib.kllm_gated_slice(_p(out), _p(gate), ctypes.c_int64(gate.stride(0)), _p(table), ctypes.c_int64(table.shape[1]),
                              int(offset), P, _p(ids), _p(last_token), n, table.shape[0], dtype_code(table.dtype), _stream())
    _check(lib, "embedding", rc)
    return out


def add_rmsnorm(x: torch.Tensor, res: Optional[torch.Tensor], out: torch.Tensor, gain: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """x (+)= res in float32, out = rmsnorm(x) * gain.

    ``rows`` given: out[r] comes from row rows[r] of x (+ res) and x is not written.
    """
    _cuda(x, res, out, gain, rows)
    _i32(rows, "rows")
    d = x.shape[1]
    if x.dtype != torch.float32 or gain.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("add_rmsnorm: x and gain must be float32, contiguous")
    if res is not None and (res.dtype not in (out.dtype, torch.float32) or not res.is_contiguous()
                            or res.shape != x.shape):
        raise KernelError("add_rmsnorm: res must match x in shape and be float32 or of out's dtype")
    if gain.numel() != d or out.shape[1] != d:
        raise KernelError("add_rmsnorm: widths do not agree")
    n_rows = out.shape[0]
    if rows is None and n_rows != x.shape[0]:
        raise KernelError("add_rmsnorm: row counts do not agree")
    if rows is not None and rows.numel() != n_rows:
        raise KernelError("add_rmsnorm: rows and out do not agree")
    lib = load_library("norm")
    rc = lib.kllm_add_rmsnorm(_p(x), _p(res), _p(out), _p(gain), _p(rows), n_rows, d,
                              ctypes.c_float(eps), dtype_code(out.dtype),
                              dtype_code(res.dtype if res is not None else out.dtype), _stream())
    _check(lib, "norm", rc)


def add_layernorm(x: torch.Tensor, res: Optional[torch.Tensor], out: torch.Tensor, gain: torch.Tensor,
                  bias: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """x (+)= res in float32, out = (x - mean) / sqrt(var + eps) * gain + bias; ``rows`` as in
    ``add_rmsnorm`` (csrc/norm.cu)."""
    _cuda(x, res, out, gain, bias, rows)
    _i32(rows, "rows")
    d = x.shape[1]
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or out.shape[1] != d:
        raise KernelError("add_layernorm: x must be contiguous float32, out contiguous of the same width")
    for t in (gain, bias):
        if t.dtype != torch.float32 or t.numel() != d or not t.is_contiguous():
            raise KernelError("add_layernorm: gain and bias must be contiguous float32 [d]")
    if res is not None and (res.dtype not in (out.dtype, torch.float32) or not res.is_contiguous() or res.shape != x.shape):
        raise KernelError("add_layernorm: res must match x in shape and be float32 or of out's dtype")
    n_rows = out.shape[0]
    if (rows is None and n_rows != x.shape[0]) or (rows is not None and rows.numel() != n_rows):
        raise KernelError("add_layernorm: row counts do not agree")
    lib = load_library("norm")
    rc = lib.kllm_add_layernorm(_p(x), _p(res), _p(out), _p(gain), _p(bias), _p(rows), n_rows, d, ctypes.c_float(eps),
                                dtype_code(out.dtype), dtype_code(res.dtype if res is not None else out.dtype), _stream())
    _check(lib, "norm", rc)


def rmsnorm_add(x: torch.Tensor, y: torch.Tensor, gain: torch.Tensor, eps: float,
                out: Optional[torch.Tensor] = None, gain2: Optional[torch.Tensor] = None, eps2: float = 0.0) -> None:
    """x += rmsnorm(y) * gain, all float32 [n, d]: a norm on a sublayer's output as it joins
    the residual stream.  With ``out`` [n, d] (model dtype) and ``gain2`` also
    out = rmsnorm(x) * gain2 of the updated rows, the norm in front of the next sublayer; with
    ``out`` alone the updated rows themselves in out's dtype (a next sublayer that reads the
    stream as it is)."""
    _cuda(x, y, gain, out, gain2)
    d = x.shape[1]
    for t in (x, y):
        if t.dtype != torch.float32 or not t.is_contiguous() or t.shape != x.shape:
            raise KernelError("rmsnorm_add: x and y must be contiguous float32 of one shape")
    if gain.dtype != torch.float32 or gain.numel() != d:
        raise KernelError("rmsnorm_add: gain must be float32 [d]")
    if out is not None and (not out.is_contiguous() or out.shape != x.shape or (
            gain2 is not None and (gain2.dtype != torch.float32 or gain2.numel() != d))):
        raise KernelError("rmsnorm_add: out contiguous like x, a second norm's gain float32 [d]")
    lib = load_library("norm")
    rc = lib.kllm_rmsnorm_add(_p(x), _p(y), _p(gain), ctypes.c_float(eps), _p(out), _p(gain2), ctypes.c_float(eps2),
                              x.shape[0], d, dtype_code(out.dtype if out is not None else torch.float32), _stream())
    _check(lib, "norm", rc)


def qknorm_append(q_out: torch.Tensor, qkv: torch.Tensor, q_gain: torch.Tensor, k_gain: Optional[torch.Tensor],
                  eps: float, temp_coef: float, temp_every: int, positions: torch.Tensor, token_req: torch.Tensor,
                  block_table: Optional[torch.Tensor], kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor],
                  n_heads: int, n_kv: int, head_dim: int, v_head_dim: int, rot: int = 0,
                  freq: Optional[torch.Tensor] = None) -> None:
    """RMS norm of the whole query projection and of the whole key projection (float32
    ``qkv`` [n, H*dk + G*dk + G*dv]), the queries' temperature 1 + coef * ln(floor((p + 1) /
    every) + 1), then with ``rot`` > 0 the rotation of the first ``rot`` values of every query and
    key head (pair (i, i + rot / 2) turns by position * freq[i]; ``freq`` float64 [rot / 2]), q stored
    in ``q_out`` [n, H*dk] (model dtype) and k, v written to the paged
    caches [pages, G, page_size, dk] / [pages, G, page_size, dv] (csrc/qknorm_append.cu).
    With ``kcache`` None ``qkv`` holds queries only and nothing is stored."""
    _cuda(q_out, qkv, q_gain, k_gain, positions, token_req, block_table, kcache, vcache, freq)
    _i32(positions, "positions"); _i32(token_req, "token_req"); _i32(block_table, "block_table"); _f64(freq, "freq")
    if rot and (freq is None or freq.numel() != rot // 2 or rot % 2 or rot > head_dim):
        raise KernelError("qknorm_append: an even rotary width within the head, one frequency per rotated pair")
    n = qkv.shape[0]
    Q, K, V = n_heads * head_dim, n_kv * head_dim, n_kv * v_head_dim
    if qkv.dtype != torch.float32 or qkv.stride(1) != 1 or qkv.shape[1] != (Q + K + V if kcache is not None else Q):
        raise KernelError("qknorm_append: the projections must be float32 [n, q + k + v] with dense rows")
    if q_out.shape != (n, Q) or not q_out.is_contiguous():
        raise KernelError("qknorm_append: q_out must be contiguous [n, heads * head_dim]")
    if q_gain.dtype != torch.float32 or q_gain.numel() != Q:
        raise KernelError("qknorm_append: the query gain must be float32 [heads * head_dim]")
    page_size = max_blocks = 0
    if kcache is not None:
        if k_gain is None or k_gain.dtype != torch.float32 or k_gain.numel() != K:
            raise KernelError("qknorm_append: the key gain must be float32 [kv heads * head_dim]")
        page_size, max_blocks = kcache.shape[2], block_table.shape[1]
        if (kcache.dtype != q_out.dtype or vcache.dtype != q_out.dtype or not kcache.is_contiguous()
                or not vcache.is_contiguous() or tuple(kcache.shape[1:]) != (n_kv, page_size, head_dim)
                or tuple(vcache.shape[1:]) != (n_kv, page_size, v_head_dim) or vcache.shape[0] != kcache.shape[0]):
            raise KernelError("qknorm_append: caches must be [pages, kv heads, page_size, size] in q_out's dtype")
    lib = load_library("qknorm_append")
    rc = lib.kllm_qknorm_append(_p(q_out), _p(qkv), ctypes.c_int64(qkv.stride(0)), _p(q_gain), _p(k_gain),
                                ctypes.c_float(eps), ctypes.c_float(temp_coef), int(temp_every or 1), _p(positions),
                                _p(token_req), _p(block_table), max_blocks, _p(kcache), _p(vcache), n, n_heads, n_kv,
                                head_dim, v_head_dim, page_size, int(rot or 0), _p(freq if rot else None),
                                dtype_code(q_out.dtype), _stream())
    _check(lib, "qknorm_append", rc)


def latent_norm_append(q_out: torch.Tensor, proj: torch.Tensor, q_gain: torch.Tensor, kv_gain: Optional[torch.Tensor],
                       eps: float, positions: torch.Tensor, token_req: torch.Tensor,
                       block_table: Optional[torch.Tensor], cache: Optional[torch.Tensor]) -> None:
    """RMS norms of the two low-rank latents of a step's tokens (csrc/latent.cu): ``proj`` float32
    [n, Rq + R] is the stacked down-projection's result; the query latent goes to ``q_out`` [n, Rq]
    (model dtype), the key/value latent into the paged store ``cache`` [pages, 1, page_size, R] at
    each token's position.  With ``cache`` None ``proj`` holds the query latents alone."""
    _cuda(q_out, proj, q_gain, kv_gain, positions, token_req, block_table, cache)
    _i32(positions, "positions"); _i32(token_req, "token_req"); _i32(block_table, "block_table")
    n, Rq = q_out.shape
    R = page_size = max_blocks = 0
    if cache is not None:
        R, page_size, max_blocks = cache.shape[3], cache.shape[2], block_table.shape[1]
        if cache.dtype != q_out.dtype or not cache.is_contiguous() or cache.shape[1] != 1:
            raise KernelError("latent_norm_append: the store must be contiguous [pages, 1, page_size, R] in q_out's dtype")
        if kv_gain is None or kv_gain.dtype != torch.float32 or kv_gain.numel() != R or not kv_gain.is_contiguous():
            raise KernelError("latent_norm_append: the key/value gain must be float32 [R]")
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or proj.shape != (n, Rq + R):
        raise KernelError("latent_norm_append: the projections must be float32 [n, Rq + R] with dense rows")
    if not q_out.is_contiguous() or q_gain.dtype != torch.float32 or q_gain.numel() != Rq or not q_gain.is_contiguous():
        raise KernelError("latent_norm_append: q_out contiguous [n, Rq], the query gain float32 [Rq]")
    lib = load_library("latent")
    rc = lib.kllm_latent_norm_append(_p(q_out), _p(proj), ctypes.c_int64(proj.stride(0)), _p(q_gain), _p(kv_gain),
                                     ctypes.c_float(eps), _p(positions), _p(token_req), _p(block_table), max_blocks,
                                     _p(cache), n, Rq, R, page_size, dtype_code(q_out.dtype), _stream())
    _check(lib, "latent", rc)


def latent_rope_append(q_plain: torch.Tensor, q_full: torch.Tensor, proj: torch.Tensor, kv_gain: Optional[torch.Tensor],
                       eps: float, freq: Optional[torch.Tensor], amplitude: float, positions: torch.Tensor,
                       token_req: torch.Tensor, block_table: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                       n_heads: int, dk: int, dr: int, rank: int) -> None:
    """What lies between the stacked projection and the attention of a layer that attends through a
    latent plus one rotated key part (csrc/latent.cu): ``proj`` float32 [n, >= H (dk + dr) + R + dr]
    holds per token the heads' queries (dk plain, dr rotated values each), the latent and the rotated
    key part.  ``q_plain`` [n, H dk] gets the plain query values, ``q_full`` [n, H (R + dr)] the rotated
    query parts in the tail of every head's row, the paged store ``cache`` [pages, 1, page_size,
    R + dr] the RMS-normed latent times ``kv_gain`` and the rotated key part.  ``freq`` float64
    [dr / 2]: pair (i, i + dr / 2) turns by position * freq[i]; cos and sin are multiplied by
    ``amplitude``.  With ``cache`` None only the queries are produced."""
    _cuda(q_plain, q_full, proj, kv_gain, freq, positions, token_req, block_table, cache)
    _i32(positions, "positions"); _i32(token_req, "token_req"); _i32(block_table, "block_table"); _f64(freq, "freq")
    n = proj.shape[0]
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or \
            proj.shape[1] < n_heads * (dk + dr) + (rank + dr if cache is not None else 0):
        raise KernelError("latent_rope_append: the projections must be float32 [n, >= H (dk + dr) (+ R + dr with a store)] "
                          "with dense rows")
    if (tuple(q_plain.shape) != (n, n_heads * dk) or tuple(q_full.shape) != (n, n_heads * (rank + dr))
            or not q_plain.is_contiguous() or not q_full.is_contiguous() or q_plain.dtype != q_full.dtype):
        raise KernelError("latent_rope_append: q_plain [n, H dk] and q_full [n, H (R + dr)] contiguous, of one dtype")
    if dr and (freq is None or freq.numel() != dr // 2):
        raise KernelError("latent_rope_append: one frequency per rotated pair")
    page_size = max_blocks = 0
    if cache is not None:
        page_size, max_blocks = cache.shape[2], block_table.shape[1]
        if cache.dtype != q_plain.dtype or not cache.is_contiguous() or cache.shape[1] != 1 or cache.shape[3] != rank + dr:
            raise KernelError("latent_rope_append: the store must be contiguous [pages, 1, page_size, R + dr] in q's dtype")
        if kv_gain is None or kv_gain.dtype != torch.float32 or kv_gain.numel() != rank or not kv_gain.is_contiguous():
            raise KernelError("latent_rope_append: the latent's gain must be float32 [R]")
    lib = load_library("latent")
    rc = lib.kllm_latent_rope_append(_p(q_plain), _p(q_full), _p(proj), ctypes.c_int64(proj.stride(0)), _p(kv_gain),
                                     ctypes.c_float(eps), _p(freq), ctypes.c_float(amplitude), _p(positions),
                                     _p(token_req), _p(block_table), max_blocks, _p(cache), n, n_heads, dk, dr, rank,
                                     page_size, dtype_code(q_plain.dtype), _stream())
    _check(lib, "latent", rc)


def headnorm_rope_append(q_out: torch.Tensor, qkv: torch.Tensor, bias: Optional[torch.Tensor],
                         q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                         freq: Optional[torch.Tensor], amplitude: float, rot: int, positions: torch.Tensor,
                         token_req: torch.Tensor, block_table: Optional[torch.Tensor], kcache: Optional[torch.Tensor],
                         vcache: Optional[torch.Tensor], q_heads: int, k_heads: int, v_heads: int, dk: int, dv: int) -> None:
    """Bias, RMS norm per head with a gain [dk] that all heads share, rotation of the first ``rot`` values
    of every query and key head, and the cache write, in one kernel (csrc/qk_headnorm.cu).  ``qkv`` float32
    [n, (q_heads + k_heads) dk + v_heads dv]; ``bias`` float32 of a row's length or None; ``q_gain`` /
    ``k_gain`` float32 [dk] or None (no norm); ``freq`` float64 [rot / 2] (pair (i, i + rot / 2) turns by
    position * freq[i], cos and sin times ``amplitude``); ``q_out`` [n, q_heads dk] in the model dtype;
    caches [pages, k_heads, page_size, dk] and [pages, v_heads, page_size, dv].  With ``kcache`` None ``qkv``
    holds queries only."""
    _cuda(q_out, qkv, bias, q_gain, k_gain, freq, positions, token_req, block_table, kcache, vcache)
    _i32(positions, "positions"); _i32(token_req, "token_req"); _i32(block_table, "block_table"); _f64(freq, "freq")
    n = qkv.shape[0]
    width = q_heads * dk + ((k_heads * dk + v_heads * dv) if kcache is not None else 0)
    if qkv.dtype != torch.float32 or qkv.stride(1) != 1 or qkv.shape[1] < width:
        raise KernelError("headnorm_rope_append: the projections must be float32 with dense rows of q, k and v")
    if tuple(q_out.shape) != (n, q_heads * dk) or not q_out.is_contiguous():
        raise KernelError("headnorm_rope_append: q_out must be contiguous [n, q_heads * dk]")
    if bias is not None and (bias.dtype != torch.float32 or not bias.is_contiguous() or bias.numel() < width):
        raise KernelError("headnorm_rope_append: the bias must be float32 of a row's length")
    for g in (q_gain, k_gain):
        if g is not None and (g.dtype != torch.float32 or not g.is_contiguous() or g.numel() != dk):
            raise KernelError("headnorm_rope_append: a gain must be float32 [dk]")
    if rot and (freq is None or freq.numel() != rot // 2):
        raise KernelError("headnorm_rope_append: one frequency per rotated pair")
    page_size = max_blocks = 0
    if kcache is not None:
        page_size, max_blocks = kcache.shape[2], block_table.shape[1]
        if (kcache.dtype != q_out.dtype or vcache.dtype != q_out.dtype or not kcache.is_contiguous()
                or not vcache.is_contiguous() or tuple(kcache.shape[1:]) != (k_heads, page_size, dk)
                or tuple(vcache.shape[1:]) != (v_heads, page_size, dv) or vcache.shape[0] != kcache.shape[0]):
            raise KernelError("headnorm_rope_append: caches must be [pages, heads, page_size, size] in q_out's dtype")
    lib = load_library("qk_headnorm")
    rc = lib.kllm_headnorm_rope_append(_p(q_out), _p(qkv), ctypes.c_int64(qkv.stride(0)), _p(bias), _p(q_gain), _p(k_gain),
                                       ctypes.c_float(eps), _p(freq), ctypes.c_float(amplitude), int(rot), _p(positions),
                                       _p(token_req), _p(block_table), max_blocks, _p(kcache), _p(vcache), n, q_heads,
                                       k_heads, v_heads, dk, dv, page_size, dtype_code(q_out.dtype), _stream())
    _check(lib, "qk_headnorm", rc)


def maps_combine(out: torch.Tensor, a: torch.Tensor, kv_heads: int, group: int, dv: int, lam: float, eps: float,
                 post: float) -> None:
    """out [n, G gs dv] = (a1 - lam a2) / rms(a1 - lam a2 over dv) * post for every head, from the two
    attention maps of a differential attention: ``a`` float32 [n, G, 2, gs, dv] (csrc/qk_headnorm.cu)."""
    _cuda(out, a)
    n = a.shape[0]
    if a.dtype != torch.float32 or not a.is_contiguous() or a.shape[1] != kv_heads * 2 * group * dv:
        raise KernelError("maps_combine: the maps must be contiguous float32 [n, G * 2 * gs * dv]")
    if tuple(out.shape) != (n, kv_heads * group * dv) or not out.is_contiguous():
        raise KernelError("maps_combine: out must be contiguous [n, G * gs * dv]")
    lib = load_library("qk_headnorm")
    rc = lib.kllm_maps_combine(_p(out), _p(a), n, kv_heads, group, dv, ctypes.c_float(lam), ctypes.c_float(eps),
                               ctypes.c_float(post), dtype_code(out.dtype), _stream())
    _check(lib, "qk_headnorm", rc)


def sigmoid_gate(out: torch.Tensor, a: torch.Tensor, gate: torch.Tensor) -> None:
    """out = a * sigmoid(gate): a and out in the model dtype, gate float32 logits; dense rows, strided rows
    allowed (csrc/activation.cu)."""
    _cuda(out, a, gate)
    if gate.dtype != torch.float32 or a.dtype != out.dtype or a.shape != out.shape or gate.shape != out.shape:
        raise KernelError("sigmoid_gate: a and out of one dtype and shape, gate float32 of that shape")
    for t in (out, a, gate):
        if t.stride(1) != 1:
            raise KernelError("sigmoid_gate: operands must have dense rows")
    n, f = out.shape
    lib = load_library("activation")
    rc = lib.kllm_sigmoid_gate(_p(out), ctypes.c_int64(out.stride(0)), _p(a), ctypes.c_int64(a.stride(0)), _p(gate),
                               ctypes.c_int64(gate.stride(0)), n, f, dtype_code(out.dtype), _stream())
    _check(lib, "activation", rc)


def streams_step(streams: torch.Tensor, *, init: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None,
                 mix: Optional[torch.Tensor] = None, out_w: Optional[torch.Tensor] = None,
                 in_w: Optional[torch.Tensor] = None, gain: Optional[torch.Tensor] = None, eps: float = 0.0,
                 normed: Optional[torch.Tensor] = None, total: Optional[torch.Tensor] = None) -> None:
    """One pass over S residual streams ``streams`` float32 [S, n, d] (csrc/streams.cu), in this
    order: with ``init`` [n, d] the streams become S copies of it; with ``y`` [n, d] (a sublayer's
    float32 output) every stream t becomes sum_s mix[s, t] x_s + out_w[t] y; with ``in_w`` [S] the
    row sum_t in_w[t] x_t is RMS-normed with ``gain`` and stored in ``normed`` [n, d] (model
    dtype); with ``total`` [n, d] the sum of the streams is stored there."""
    _cuda(streams, init, y, mix, out_w, in_w, gain, normed, total)
    if streams.dtype != torch.float32 or streams.dim() != 3 or not streams.is_contiguous():
        raise KernelError("streams_step: the streams must be contiguous float32 [S, n, d]")
    S, n, d = streams.shape
    for t, shape, what in ((init, (n, d), "init"), (y, (n, d), "y"), (total, (n, d), "total"), (mix, (S, S), "mix"),
                           (out_w, (S,), "out_w"), (in_w, (S,), "in_w"), (gain, (d,), "gain")):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape) != shape):
            raise KernelError(f"streams_step: {what} must be contiguous float32 {shape}")
    if normed is not None and (not normed.is_contiguous() or tuple(normed.shape) != (n, d)):
        raise KernelError("streams_step: normed must be contiguous [n, d]")
    if (y is not None and (mix is None or out_w is None)) or (in_w is not None and (gain is None or normed is None)):
        raise KernelError("streams_step: a write needs mix and out_w, a read needs gain and normed")
    lib = load_library("streams")
    rc = lib.kllm_streams_step(_p(streams), ctypes.c_int64(n * d), _p(init), _p(y), _p(mix), _p(out_w), _p(in_w),
                               _p(gain), ctypes.c_float(eps), _p(normed), _p(total), n, d, S,
                               dtype_code(normed.dtype if normed is not None else torch.float32), _stream())
    _check(lib, "streams", rc)


def rope_append(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos_sin: Optional[torch.Tensor],
                positions: torch.Tensor, token_req: torch.Tensor, block_table: Optional[torch.Tensor],
                kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor],
                n_heads: int, n_kv: int, head_dim: int) -> None:
    """Rotate q in place; write rotated k and v into the paged cache.

    q, k, v are 2-D views (rows may be strided, the last dim is dense); caches are
    [pages, n_kv, page_size, head_dim].  With kcache None only q is rotated; with
    cos_sin None nothing is rotated and k, v are only stored.
    """
    _cuda(q, k, v, cos_sin, positions, token_req, block_table, kcache, vcache)
    _i32(positions, "positions"); _i32(token_req, "token_req"); _i32(block_table, "block_table")
    for t in (q, k, v):
        if t.stride(1) != 1:
            raise KernelError("rope_append: q, k, v rows must be dense")
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous()):
        raise KernelError("rope_append: the cos/sin table must be contiguous float32")
    n = q.shape[0]
    rot = cos_sin.shape[1] if cos_sin is not None else 0
    if kcache is not None:
        if kcache.shape != vcache.shape or kcache.shape[1] != n_kv or kcache.shape[3] != head_dim \
                or not kcache.is_contiguous() or not vcache.is_contiguous() or kcache.dtype != q.dtype:
            raise KernelError("rope_append: cache layout must be [pages, n_kv, page_size, head_dim] in q's dtype")
        page_size, max_blocks = kcache.shape[2], block_table.shape[1]
    else:
        page_size, max_blocks = 1, 0
    lib = load_library("rope")
    rc = lib.kllm_rope_append(_p(q), ctypes.c_int64(q.stride(0)), _p(k), ctypes.c_int64(k.stride(0)),
                              _p(v), ctypes.c_int64(v.stride(0)), _p(cos_sin), _p(positions),
                              _p(token_req), _p(block_table), max_blocks, _p(kcache), _p(vcache),
                              n, n_heads, n_kv, head_dim, rot, page_size, dtype_code(q.dtype), _stream())
    _check(lib, "rope", rc)


def attention_generic(out: torch.Tensor, q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                      positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                      n_heads: int, n_kv: int, head_dim: int, window: int, scale: float,
                      score_slopes: Optional[torch.Tensor] = None, v_head_dim: Optional[int] = None,
                      sinks: Optional[torch.Tensor] = None, segment: int = 0) -> None:
    """Causal GQA attention of every new token over its request's cached keys: one warp per
    (token, head), any head size up to 512, values of their own size, optional score slopes and
    sinks (float32 [n_heads]: exp(sinks[h]) joins the denominator of head h's softmax).
    ``segment``, fewer value heads than key heads, value rows that head longer rows and a float32
    ``out`` as in ``attention_simt``."""
    _cuda(out, q, kcache, vcache, positions, token_req, block_table, score_slopes, sinks)
    vd = int(v_head_dim or head_dim)
    v_heads, v_row = _value_layout(kcache, vcache, n_kv, vd)
    if out.shape[1] != n_heads * vd:
        raise KernelError("attention: out must be [n, heads * value size]")
    _i32(positions, "positions"); _i32(token_req, "token_req"); _i32(block_table, "block_table")
    if q.stride(1) != 1 or not out.is_contiguous() or out.dtype not in (q.dtype, torch.float32) or kcache.dtype != q.dtype:
        raise KernelError("attention: operands must share a dtype; out contiguous (of that dtype or float32), q rows dense")
    if not kcache.is_contiguous() or not vcache.is_contiguous() or kcache.shape[1] != n_kv or kcache.shape[3] != head_dim:
        raise KernelError("attention: cache layout must be [pages, n_kv, page_size, head_dim]")
    n = q.shape[0]
    lib = load_library("attention_generic")
    rc = lib.kllm_attention_generic(_p(out), _p(q), ctypes.c_int64(q.stride(0)), _p(kcache), _p(vcache),
                                    _p(positions), _p(token_req), _p(block_table), block_table.shape[1],
                                    n, n_heads, n_kv, head_dim, vd, kcache.shape[2], int(window or 0),
                                    ctypes.c_float(scale), _slopes_arg(score_slopes, n_heads),
                                    _slopes_arg(sinks, n_heads, "sinks"), int(segment or 0), v_heads, v_row,
                                    int(out.dtype == torch.float32 and q.dtype != torch.float32), dtype_code(q.dtype),
                                    _stream())
    _check(lib, "attention_generic", rc)


def _value_layout(kcache, vcache, n_kv, vd):
    """(value heads, elements between value rows) of a value store [pages, value heads, page_size, row]
    beside a key store [pages, n_kv, page_size, head_dim]: the value heads divide the key heads, a
    row holds at least ``vd`` values (more when the values head a longer row)."""
    if (vcache.dim() != 4 or vcache.shape[0] != kcache.shape[0] or vcache.shape[2] != kcache.shape[2]
            or vcache.shape[1] <= 0 or n_kv % vcache.shape[1] or vcache.shape[3] < vd or not vcache.is_contiguous()
            or vcache.dtype != kcache.dtype):
        raise KernelError("attention: value store [pages, value heads, page_size, >= value size], its heads dividing "
                          "the key heads")
    return int(vcache.shape[1]), int(vcache.shape[3])


SIMT_CHUNK = 256      # keys per CTA when a decoding token's context is cut (attention_simt)


def attention_simt(out: torch.Tensor, q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, ctx,
                   block_table: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, window: int,
                   scale: float, score_slopes: Optional[torch.Tensor] = None, v_head_dim: Optional[int] = None,
                   sinks: Optional[torch.Tensor] = None, segment: int = 0, upto: Optional[int] = None) -> None:
    """Causal GQA attention of the step's tokens on the CUDA cores, float32 arithmetic
    (csrc/attention_simt.cu): the attention of the float32 path.  The requests that bring
    one token each at the head of the batch (decoding requests, which the scheduler puts
    first) have their contexts cut into chunks of SIMT_CHUNK keys, one CTA each, merged in
    chunk order; the portions after them run as tiles of up to 64 (token, head) rows.
    ``score_slopes`` (float32 [n_heads]): slope[h] * (key position - query position) is added
    to the scaled scores of head h.  ``v_head_dim``: the size of a head's values and of its
    output where it differs from the keys' (``vcache`` [pages, n_kv, page_size, v_head_dim],
    ``out`` [n, n_heads * v_head_dim]).  ``sinks`` (float32 [n_heads]): exp(sinks[h]) is one more
    term of the denominator of head h's softmax, without a key or a value.  ``segment`` C: positions
    are cut into segments of C counted from 0 and a query sees only the keys of its own segment.
    The value store may have fewer heads than the key store (``vcache`` [pages, v_heads, page_size,
    row]: n_kv / v_heads neighbouring key heads read one value head) and rows longer than
    ``v_head_dim`` (the values are then the head of each row: a store whose rows are keys and, in
    their first part, values).  ``out`` may be float32 beside bfloat16 operands.  ``upto``: only the
    first ``upto`` requests are served, which bring one token each (the caller gives the portions
    after them to another kernel)."""
    _cuda(out, q, kcache, vcache, block_table, score_slopes, sinks)
    _slopes_arg(sinks, n_heads, "sinks")
    vd = int(v_head_dim or head_dim)
    v_heads, v_row = _value_layout(kcache, vcache, n_kv, vd)
    segment = int(segment or 0)
    out_f32 = int(out.dtype == torch.float32 and q.dtype != torch.float32)
    if score_slopes is not None and (score_slopes.dtype != torch.float32 or not score_slopes.is_contiguous()
                                     or score_slopes.numel() != n_heads):
        raise KernelError("attention: score slopes must be a contiguous float32 tensor, one per head")
    _i32(block_table, "block_table"); _i32(ctx.q_start, "q_start"); _i32(ctx.start_pos, "start_pos")
    if q.stride(1) != 1 or not out.is_contiguous() or out.dtype not in (q.dtype, torch.float32) or kcache.dtype != q.dtype:
        raise KernelError("attention: operands must share a dtype; out contiguous (of that dtype or float32), q rows dense")
    if not kcache.is_contiguous() or kcache.shape[1] != n_kv or kcache.shape[3] != head_dim \
            or out.shape[1] != n_heads * vd or v_row % 4:
        raise KernelError("attention: cache layout must be [pages, n_kv, page_size, head_dim]")
    group = n_heads // max(1, n_kv)
    lib = load_library("attention_simt")
    n_req, n_tokens = ctx.n_requests, ctx.n_tokens
    singles = n_req if ctx.all_single else 0
    if upto is not None:
        n_req = n_tokens = singles = int(upto)
    elif not ctx.all_single and ctx.host_n_new:
        while singles < n_req and ctx.host_n_new[singles] == 1:
            singles += 1
    bound = ctx.split_bound or ctx.max_ctx
    if window:
        bound = min(bound, int(window))
    if segment:
        bound = min(bound, segment)
    splits = max(1, -(-bound // SIMT_CHUNK))
    common = (n_heads, n_kv, head_dim, vd, kcache.shape[2], int(window or 0), ctypes.c_float(scale))
    first = 0
    global launches
    if singles and splits > 1:
        part_o = torch.empty((singles * n_heads, splits, vd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((singles * n_heads, splits, 2), dtype=torch.float32, device=q.device)
        rc = lib.kllm_attention_simt(_p(out), _p(part_o), _p(part_ml), _p(q), ctypes.c_int64(q.stride(0)), _p(kcache),
                                     _p(vcache), _p(ctx.q_start), _p(ctx.start_pos), _p(block_table),
                                     block_table.shape[1], singles, singles, *common, 1, SIMT_CHUNK, splits,
                                     _p(score_slopes), _p(sinks), segment, v_heads, v_row, out_f32, dtype_code(q.dtype),
                                     _stream())
        _check(lib, "attention_simt", rc)
        rc = lib.kllm_attention_simt_merge(_p(out), _p(part_o), _p(part_ml), _p(ctx.positions), singles, n_heads,
                                           vd, int(window or 0), SIMT_CHUNK, splits, _p(sinks), segment, out_f32,
                                           dtype_code(q.dtype), _stream())
        _check(lib, "attention_simt", rc)
        first = singles
    if first < n_req:
        qt = max(1, 64 // group)
        rest = n_tokens - first
        rc = lib.kllm_attention_simt(_p(out), None, None, _p(q), ctypes.c_int64(q.stride(0)), _p(kcache), _p(vcache),
                                     _p(ctx.q_start[first:]), _p(ctx.start_pos[first:]), _p(block_table[first:]),
                                     block_table.shape[1], n_req - first, rest // qt + (n_req - first), *common, qt, 0, 1,
                                     _p(score_slopes), _p(sinks), segment, v_heads, v_row, out_f32, dtype_code(q.dtype),
                                     _stream())
        _check(lib, "attention_simt", rc)


def simt_fits(q: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, v_head_dim: Optional[int] = None) -> bool:
    """Whether ``attention_simt`` takes these operands: head sizes (keys, values) multiples of
    4 up to 256, at most 64 heads per kv head, rows aligned to four elements."""
    quad = 4 * q.element_size()
    vd = int(v_head_dim or head_dim)
    return (head_dim % 4 == 0 and 0 < head_dim <= 256 and vd % 4 == 0 and 0 < vd <= 256 and n_heads // max(1, n_kv) <= 64
            and q.data_ptr() % quad == 0 and q.stride(0) % 4 == 0)


TC_HEAD_DIMS = tuple(range(16, 129, 16))     # head sizes of the tensor-core attention library
WIDE_SINGLE_KEYS = 2048                      # a single token that sees at most this many keys runs as a row of the wide prefill form
TC_WIDE_HEAD_DIMS = (160, 192, 224, 256)     # ... and those that only its unfused kernels are built for
TCGEN05_HEAD_DIMS = (64, 128)                # head sizes of the tcgen05 prefill attention
PREFETCH_L2 = os.environ.get("KLLM_B200_PREFETCH", "1") != "0"   # kernels warm L2 for the kernel after them
# ... with at most this much of the next matrix: what is asked for beyond a fraction of the
# 126 MB of L2 pushes out lines that are still needed and is read from HBM twice
PREFETCH_L2_BYTES = int(float(os.environ.get("KLLM_B200_PREFETCH_MB", "24")) * 2 ** 20)
USE_TCGEN05 = os.environ.get("KLLM_B200_TCGEN05", "1") != "0"
_sm_count = {}


def tensor_core_rows(head_dim: int, group: int, dtype: torch.dtype) -> bool:
    """Whether ``attention`` runs bfloat16 rows of this size, with ``group`` heads on a kv head and values as
    wide as keys, on the ``mma.sync`` kernels (also with ``exact_weights`` or sinks)."""
    return dtype == torch.bfloat16 and (head_dim in TC_HEAD_DIMS or head_dim in TC_WIDE_HEAD_DIMS) and group <= 64


def sm_count() -> int:
    """Streaming multiprocessors of the current device (148 on a B200)."""
    dev = torch.cuda.current_device()
    if dev not in _sm_count:
        _sm_count[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sm_count[dev]


def decode_splits(n_tokens: int, n_kv: int, ctx_bound: int) -> int:
    """Into how many key ranges the decode kernel cuts a token's context.

    A CTA takes one (token, kv head, range); two CTAs fit an SM.  The ranges are
    whole 64-key tiles, as many as fill the SMs in ONE wave (a second wave of short
    CTAs would double the kernel's time), at most 16, all the same length.  When one
    range per token would be long, two are used even if that spills into a second
    wave: long CTAs hide it."""
    slots = 2 * sm_count()
    tiles = max(1, -(-ctx_bound // 64))
    base = max(1, n_tokens * n_kv)
    splits = max(1, min(slots // base, tiles, 16))
    if splits == 1 and tiles >= 16:
        splits = 2
    per = -(-tiles // splits)
    return -(-tiles // per)


def attention(out: torch.Tensor, q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, ctx,
              block_table: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, window: int,
              scale: float, score_slopes: Optional[torch.Tensor] = None, v_head_dim: Optional[int] = None,
              exact_weights: bool = False, sinks: Optional[torch.Tensor] = None, segment: int = 0) -> None:
    """Causal GQA attention of the step's tokens over the paged cache, by the
    kernel that fits: bfloat16 with a head size in TC_HEAD_DIMS runs on tensor cores
    (the decode form when every request brings one token, else the prefill form: on
    tcgen05 for head sizes 64 and 128, on mma.sync for the other multiples of 16);
    float32 and other head sizes run on the CUDA cores (``attention_simt``; head sizes
    that are no multiple of 4 and groups wider than 64 the one-warp-per-row kernel).  A mixed
    step whose first requests bring one token each (the scheduler puts decoding requests
    first) is cut in two: those tokens take the decode form, which spreads a long context
    over many CTAs, the portions after them the prefill form, in which a single token
    would walk its whole context with one CTA of 128 rows, 127 of them idle.
    ``score_slopes`` (a bias on the scores that is linear in the distance, per head) is
    taken by the CUDA-core kernel and the ``mma.sync`` kernels, not by the tcgen05 kernels.
    ``exact_weights``: the softmax weights, computed in float32, must not meet the values
    rounded to one bfloat16: the ``mma.sync`` kernels then feed them to the tensor cores as
    two bfloat16 terms (16 bits of mantissa), the CUDA-core kernel as float32.
    ``sinks`` (float32 [n_heads]): exp(sinks[h]) joins the denominator of head h's softmax, a
    term without a key or a value; taken by the CUDA-core kernels and the ``mma.sync`` kernels.
    ``segment`` (a query sees only the keys of its own segment of that many positions), values of
    another size than the keys, a value store with fewer heads than the key store or with rows that
    the values only head, and a float32 ``out`` beside bfloat16 operands are taken by the CUDA-core
    kernels and, for portions in bfloat16 with sizes in steps of 16, by the ``mma.sync`` prefill kernel."""
    group = n_heads // max(1, n_kv)
    vd = int(v_head_dim or head_dim)
    special = score_slopes is not None or exact_weights
    special = special or sinks is not None
    plain_values = vcache.shape[1] == n_kv and vcache.shape[3] == vd and out.dtype == q.dtype
    tc = (q.dtype == torch.bfloat16 and (head_dim in TC_HEAD_DIMS or head_dim in TC_WIDE_HEAD_DIMS) and vd == head_dim
          and not (special and scale <= 0) and not segment and plain_values)
    # what the plain tensor-core route refuses, the prefill kernel takes in its wide form (bfloat16 rows, sizes
    # in steps of 16): portions go there, the single tokens at the head of the batch to the CUDA cores
    # ... unless a segment or a window keeps every token's keys few: then a single token's CTA has a short walk
    # and the tensor-core kernel takes the whole step, decoding steps too
    wide = (not tc and q.dtype == torch.bfloat16 and (head_dim in TC_HEAD_DIMS or head_dim in TC_WIDE_HEAD_DIMS)
            and vd % 16 == 0 and 16 <= vd <= 256 and group <= 64 and not (special and scale <= 0)
            and vcache.dim() == 4 and vcache.shape[3] % 8 == 0)
    short = min(int(segment or (1 << 30)), int(window or (1 << 30))) <= WIDE_SINGLE_KEYS
    if wide and not short and (ctx.all_single or not ctx.host_n_new):
        wide = False
    if wide:
        singles = 0
        while not short and singles < ctx.n_requests and ctx.host_n_new[singles] == 1:
            singles += 1
        if singles:
            if not simt_fits(q, n_heads, n_kv, head_dim, vd):
                wide = False
            else:
                attention_simt(out, q, kcache, vcache, ctx, block_table, n_heads, n_kv, head_dim, window, scale,
                               score_slopes, vd, sinks, segment, upto=singles)
    if wide:
        if singles < ctx.n_requests:
            attention_prefill(out, q, kcache, vcache, ctx.q_start[singles:], ctx.start_pos[singles:],
                              block_table[singles:], ctx.n_requests - singles, n_heads, n_kv, head_dim, window, scale,
                              slopes=score_slopes, split_weights=exact_weights, sinks=sinks, v_head_dim=vd,
                              segment=segment)
        return
    if (special or vd != head_dim or segment or not plain_values) and not (tc and group <= 64):
        if not simt_fits(q, n_heads, n_kv, head_dim, vd) or vcache.shape[3] % 4:
            # head sizes that are no multiples of 4, very wide groups: one warp per (token, head)
            return attention_generic(out, q, kcache, vcache, ctx.positions, ctx.token_req, block_table, n_heads, n_kv,
                                     head_dim, window, scale, score_slopes, vd, sinks, segment)
        return attention_simt(out, q, kcache, vcache, ctx, block_table, n_heads, n_kv, head_dim, window, scale,
                              score_slopes, vd, sinks, segment)
    # the decode kernel takes 16 heads per CTA: more heads on a kv head are cut into groups of equal size
    groups = n_kv * next(s for s in range(1, group + 1) if group % s == 0 and group // s <= 16)
    if tc and ctx.all_single and group <= 64:
        return attention_decode(out, q, kcache, vcache, ctx.positions, ctx.token_req, block_table, n_heads,
                                n_kv, head_dim, window, scale,
                                decode_splits(ctx.n_tokens, groups, min(ctx.split_bound or ctx.max_ctx, window or (1 << 30))),
                                slopes=score_slopes, split_weights=exact_weights, sinks=sinks)
    singles = 0
    if tc and group <= 64 and ctx.host_n_new:
        while singles < ctx.n_requests and ctx.host_n_new[singles] == 1:
            singles += 1
    if 0 < singles < ctx.n_requests:
        # token t of the first `singles` is request t: no token-to-request table needed
        attention_decode(out[:singles], q[:singles], kcache, vcache, ctx.positions[:singles], None,
                         block_table[:singles], n_heads, n_kv, head_dim, window, scale,
                         decode_splits(singles, groups, min(ctx.max_ctx, window or (1 << 30))), slopes=score_slopes,
                         split_weights=exact_weights, sinks=sinks)
    q_start, start_pos, table, n_req = ctx.q_start, ctx.start_pos, block_table, ctx.n_requests
    if 0 < singles < ctx.n_requests:
        q_start, start_pos, table, n_req = q_start[singles:], start_pos[singles:], block_table[singles:], n_req - singles
    if tc and USE_TCGEN05 and head_dim in TCGEN05_HEAD_DIMS and group <= 128 and not special:
        return attention_prefill_tcgen05(out, q, kcache, vcache, q_start, start_pos, table,
                                         n_req, n_heads, n_kv, head_dim, window, scale,
                                         probabilities=tcgen05_form(head_dim, group, n_kv, ctx.n_tokens - singles,
                                                                    n_req, ctx.max_ctx))
    if tc and group <= 64:
        return attention_prefill(out, q, kcache, vcache, q_start, start_pos, table,
                                 n_req, n_heads, n_kv, head_dim, window, scale, slopes=score_slopes,
                                 split_weights=exact_weights, sinks=sinks)
    if simt_fits(q, n_heads, n_kv, head_dim):
        return attention_simt(out, q, kcache, vcache, ctx, block_table, n_heads, n_kv, head_dim, window, scale)
    return attention_generic(out, q, kcache, vcache, ctx.positions, ctx.token_req, block_table, n_heads, n_kv,
                             head_dim, window, scale)


def _check_attention(out, q, kcache, vcache, block_table, n_kv, head_dim):
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16:
        raise KernelError("tensor-core attention takes bfloat16 operands")
    if q.stride(1) != 1 or not out.is_contiguous() or not kcache.is_contiguous() or not vcache.is_contiguous():
        raise KernelError("attention: out and caches contiguous, q rows dense")
    if kcache.shape[1] != n_kv or kcache.shape[3] != head_dim or kcache.shape != vcache.shape:
        raise KernelError("attention: cache layout must be [pages, n_kv, page_size, head_dim]")
    _i32(block_table, "block_table")


def _slopes_arg(slopes, n_heads, what="score slopes"):
    if slopes is not None and (slopes.dtype != torch.float32 or not slopes.is_contiguous() or slopes.numel() != n_heads):
        raise KernelError(f"attention: {what} must be a contiguous float32 tensor, one per head")
    return _p(slopes)


def attention_decode(out, q, kcache, vcache, positions, token_req, block_table, n_heads, n_kv, head_dim,
                     window, scale, num_splits: int, slopes: Optional[torch.Tensor] = None,
                     split_weights: bool = False, sinks: Optional[torch.Tensor] = None) -> None:
    """Tensor-core decode attention: every token attends on its own, its keys cut
    into ``num_splits`` ranges that are merged in a fixed order.  ``slopes`` (float32 [heads]):
    slope[h] * (key position - query position) is added to the scaled scores; ``split_weights``:
    the probabilities enter the second product as two bfloat16 terms instead of one; ``sinks``
    (float32 [heads]): exp(sinks[h]) joins the denominator of head h's softmax."""
    _cuda(out, q, kcache, vcache, positions, token_req, block_table, slopes, sinks)
    _check_attention(out, q, kcache, vcache, block_table, n_kv, head_dim)
    _i32(positions, "positions"); _i32(token_req, "token_req")
    n = q.shape[0]
    part_o = part_ml = None
    if num_splits > 1:
        part_o = torch.empty((n, n_heads, num_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, n_heads, num_splits, 2), dtype=torch.float32, device=q.device)
    lib = load_library("attention_tc", {"KLLM_HD": head_dim})
    rc = lib.kllm_attention_decode(_p(out), _p(part_o), _p(part_ml), _p(q), ctypes.c_int64(q.stride(0)),
                                   _p(kcache), _p(vcache), _p(positions), _p(token_req), _p(block_table),
                                   block_table.shape[1], n, n_heads, n_kv, head_dim, kcache.shape[2],
                                   int(window or 0), ctypes.c_float(scale), int(num_splits), _slopes_arg(slopes, n_heads),
                                   int(bool(split_weights)), _slopes_arg(sinks, n_heads, "sinks"), _stream())
    _check(lib, "attention_tc", rc)
    global launches
    if num_splits > 1:
        launches += 1       # the combine kernel


def attention_decode_fused(out, q, k_new, v_new, cos_sin, kcache, vcache, positions, token_req, block_table,
                           counters, n_heads, n_kv, head_dim, window, scale, num_splits: int,
                           prefetch: Optional[torch.Tensor] = None) -> None:
    """Decode attention of one token per request with the rotary encoding, the cache
    write and the merge of the key ranges inside the kernel.  q, k_new, v_new are the
    step's unrotated projections; ``counters`` is an all-zero int32 tensor of at least
    n_tokens * n_kv elements that the kernel leaves all zero.  ``token_req`` may be None:
    token t then belongs to request t, and the kernel reads its block-table row without
    waiting for that look-up.  ``prefetch``: a contiguous tensor that a later kernel
    streams; it is requested into L2 once this kernel's own copies are on their way."""
    _cuda(out, q, k_new, v_new, cos_sin, kcache, vcache, positions, token_req, block_table, counters)
    _check_attention(out, q, kcache, vcache, block_table, n_kv, head_dim)
    _i32(positions, "positions"); _i32(token_req, "token_req"); _i32(counters, "counters")
    n = q.shape[0]
    if k_new.stride(1) != 1 or v_new.stride(1) != 1 or k_new.dtype != q.dtype or v_new.dtype != q.dtype:
        raise KernelError("attention (fused): k and v must be bfloat16 with dense rows")
    if cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous() or cos_sin.shape[1] != head_dim:
        raise KernelError("attention (fused): the cos/sin table must be float32 [positions, head_dim]")
    if counters.numel() < n * n_kv:
        raise KernelError("attention (fused): too few counters")
    part_o = part_ml = None
    if num_splits > 1:
        part_o = torch.empty((n, n_heads, num_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, n_heads, num_splits, 2), dtype=torch.float32, device=q.device)
    lib = load_library("attention_tc", {"KLLM_HD": head_dim})
    rc = lib.kllm_attention_decode_fused(
        _p(out), _p(part_o), _p(part_ml), _p(counters), _p(q), ctypes.c_int64(q.stride(0)), _p(k_new),
        ctypes.c_int64(k_new.stride(0)), _p(v_new), ctypes.c_int64(v_new.stride(0)), _p(cos_sin), _p(kcache),
        _p(vcache), _p(positions), _p(token_req), _p(block_table), block_table.shape[1], n, n_heads, n_kv,
        head_dim, kcache.shape[2], int(window or 0), ctypes.c_float(scale), int(num_splits),
        *_prefetch_args(prefetch), _stream())
    _check(lib, "attention_tc", rc)


def attention_prefill(out, q, kcache, vcache, q_start, start_pos, block_table, n_requests, n_heads, n_kv,
                      head_dim, window, scale, slopes: Optional[torch.Tensor] = None,
                      split_weights: bool = False, sinks: Optional[torch.Tensor] = None,
                      v_head_dim: Optional[int] = None, segment: int = 0) -> None:
    """Tensor-core attention of portions: request s brings rows q_start[s]..q_start[s+1]
    that start at cache position start_pos[s].  ``slopes``, ``split_weights`` and ``sinks`` as in
    ``attention_decode``.  ``v_head_dim`` (values of another size than the keys: a library of its
    own per pair of sizes), ``segment``, a value store of another shape than the key store and a
    float32 ``out`` as in ``attention_simt``."""
    _cuda(out, q, kcache, vcache, q_start, start_pos, block_table, slopes, sinks)
    vd = int(v_head_dim or head_dim)
    if q.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32) or kcache.dtype != torch.bfloat16:
        raise KernelError("tensor-core attention takes bfloat16 operands (out bfloat16 or float32)")
    if q.stride(1) != 1 or not out.is_contiguous() or not kcache.is_contiguous() or out.shape[1] != n_heads * vd:
        raise KernelError("attention: out and caches contiguous, q rows dense")
    if kcache.shape[1] != n_kv or kcache.shape[3] != head_dim:
        raise KernelError("attention: cache layout must be [pages, n_kv, page_size, head_dim]")
    v_heads, v_row = _value_layout(kcache, vcache, n_kv, vd)
    _i32(block_table, "block_table")
    _i32(q_start, "q_start"); _i32(start_pos, "start_pos")
    lib = load_library("attention_tc", {"KLLM_HD": head_dim} if vd == head_dim else {"KLLM_HD": head_dim, "KLLM_VD": vd})
    rc = lib.kllm_attention_prefill(_p(out), _p(q), ctypes.c_int64(q.stride(0)), _p(kcache), _p(vcache),
                                    _p(q_start), _p(start_pos), _p(block_table), block_table.shape[1],
                                    q.shape[0], int(n_requests), n_heads, n_kv, head_dim, kcache.shape[2],
                                    int(window or 0), ctypes.c_float(scale), _slopes_arg(slopes, n_heads),
                                    int(bool(split_weights)), _slopes_arg(sinks, n_heads, "sinks"), vd,
                                    int(segment or 0), v_heads, v_row, int(out.dtype == torch.float32), _stream())
    _check(lib, "attention_tc", rc)


def tcgen05_form(head_dim: int, group: int, n_kv: int, n_tokens: int, n_requests: int, max_ctx: int) -> str:
    """Which of the two tcgen05 attention kernels a step of portions takes ("smem" / "tmem",
    see ``attention_prefill_tcgen05``), from measurements (profiles/attn_prefill_tc5_forms.md):
    head size 128 always keeps its probabilities in tensor memory.  At head size 64 that form
    (four CTAs per SM) wins when the step is many short chains of tiles or several waves of
    CTAs, and loses to the other (two CTAs per SM, two score buffers) when one long prompt's
    longest chain is the whole kernel: all CTAs resident at once and more than 16 key tiles."""
    if head_dim != 64:
        return "tmem"
    ctas = (n_tokens // max(1, 128 // group) + n_requests) * n_kv
    tiles = -(-max_ctx // 64)
    return "tmem" if tiles <= 16 or ctas >= 6 * sm_count() else "smem"


def attention_prefill_tcgen05(out, q, kcache, vcache, q_start, start_pos, block_table, n_requests, n_heads, n_kv,
                              head_dim, window, scale, probabilities: Optional[str] = None) -> None:
    """Attention of portions on tcgen05 tensor cores with TMEM accumulators (head size
    64 or 128); same contract as ``attention_prefill``.  Two kernels, which differ in where
    the probabilities wait for the second product: ``probabilities="smem"``
    (csrc/attention_tcgen05.cu: two score buffers in tensor memory, P through shared
    memory, two CTAs of head size 64 per SM) or ``"tmem"`` (csrc/attention_tcgen05_ptmem.cu:
    P written over the scores in tensor memory and read from there, half the tensor memory
    and shared memory per CTA, four / two CTAs per SM).  Default (no step shape known): tmem
    for head size 128 (1.3 to 1.6 times faster), smem for head size 64; ``attention`` picks
    by the step's shape (``tcgen05_form``)."""
    _cuda(out, q, kcache, vcache, q_start, start_pos, block_table)
    _check_attention(out, q, kcache, vcache, block_table, n_kv, head_dim)
    _i32(q_start, "q_start"); _i32(start_pos, "start_pos")
    probabilities = probabilities or ("tmem" if head_dim == 128 else "smem")
    if probabilities not in ("smem", "tmem"):
        raise KernelError("attention (tcgen05): probabilities wait in 'smem' or in 'tmem'")
    name = "attention_tcgen05" + ("_ptmem" if probabilities == "tmem" else "")
    lib = load_library(name, {"KLLM_HD": head_dim})
    fn = lib.kllm_attention_prefill_tcgen05_ptmem if probabilities == "tmem" else lib.kllm_attention_prefill_tcgen05
    rc = fn(_p(out), _p(q), ctypes.c_int64(q.stride(0)), _p(kcache), _p(vcache), _p(q_start), _p(start_pos),
            _p(block_table), block_table.shape[1], q.shape[0], int(n_requests), n_heads, n_kv, head_dim,
            kcache.shape[2], int(window or 0), ctypes.c_float(scale), _p(status_word(q.device)), _stream())
    _check(lib, name, rc)


_status_words = {}      # device index -> int32 tensor that kernels set when a bounded wait runs out


def status_word(device) -> torch.Tensor:
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status_words[idx]


def check_status(device) -> None:
    """Raise if a kernel reported that a bounded wait (on an mbarrier) ran out; its
    results are then not valid.  Synchronises the device."""
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise KernelError(f"a kernel gave up waiting on an mbarrier (wait number {code} in its source); "
                          "its results are not valid")


TIMELINE_TAGS = {200: "attn_decode_fused", 201: "attn_decode_fused (merging CTA)"}
for _pro, _pn in ((0, "x"), (1, "norm")):
    for _epi, _en in ((0, "bf16"), (1, "f32"), (2, "add"), (3, "swiglu")):
        TIMELINE_TAGS[100 + _pro * 10 + _epi] = f"skinny_gemm {_pn}->{_en}"


def timeline():
    """Rows of the kernels' timeline tables, oldest first (only in a process started with
    KLLM_B200_TIMELINE=1, which loads the instrumented builds): a list of dicts with the
    library, the kernel, and per recorded CTA (first, middle, last of the grid) the
    nanosecond timer at the kernel's marks; see the TL_END lines in csrc for what the
    marks of a kernel mean.  Synchronises the device."""
    import numpy as np
    from .csrc.build import loaded_libraries
    torch.cuda.synchronize()
    rows = []
    for variant, lib in loaded_libraries().items():
        name = variant.split("-")[0]
        fn = getattr(lib, "kllm_timeline_" + name, None) if "KLLM_TIMELINE" in variant else None
        if fn is None:
            continue
        buf = np.zeros((512, 3, 9), dtype=np.uint64)
        if fn(buf.ctypes.data_as(ctypes.c_void_p)) != 0:
            raise KernelError(f"timeline of {variant} could not be read")
        for slot in range(512):
            ctas = [buf[slot, c, :8].astype(np.int64) for c in range(3) if buf[slot, c, 0] > 0]
            if ctas:
                tags = sorted({int(buf[slot, c, 8]) for c in range(3) if buf[slot, c, 0] > 0})
                rows.append({"library": variant, "kernel": " / ".join(TIMELINE_TAGS.get(t, str(t)) for t in tags),
                             "start": int(min(c[0] for c in ctas)), "end": int(max(c.max() for c in ctas)),
                             "marks": ctas})
    rows.sort(key=lambda r: r["start"])
    return rows


def silu_mul(out: torch.Tensor, gate: torch.Tensor, up: torch.Tensor) -> None:
    """out = silu(gate) * up; 2-D operands with dense rows (strided rows allowed);
    gate and up share a dtype, float32 or out's."""
    _cuda(out, gate, up)
    for t in (out, gate, up):
        if t.stride(1) != 1:
            raise KernelError("silu_mul: operands must have dense rows")
    if gate.dtype != up.dtype or gate.dtype not in (out.dtype, torch.float32):
        raise KernelError("silu_mul: gate and up must share a dtype, float32 or out's")
    n, f = out.shape
    lib = load_library("activation")
    rc = lib.kllm_silu_mul(_p(out), ctypes.c_int64(out.stride(0)), _p(gate), ctypes.c_int64(gate.stride(0)),
                           _p(up), ctypes.c_int64(up.stride(0)), n, f, dtype_code(out.dtype),
                           dtype_code(gate.dtype), _stream())
    _check(lib, "activation", rc)


def clamped_glu(out: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, limit: float, alpha: float) -> None:
    """out = g * sigmoid(alpha g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit);
    float32 gate and up with dense rows (strided rows allowed), out in float32 or bfloat16."""
    _cuda(out, gate, up)
    for t in (out, gate, up):
        if t.stride(1) != 1:
            raise KernelError("clamped_glu: operands must have dense rows")
    if gate.dtype != torch.float32 or up.dtype != torch.float32 or gate.shape != out.shape or up.shape != out.shape:
        raise KernelError("clamped_glu: gate and up must be float32 of out's shape")
    n, f = out.shape
    lib = load_library("activation")
    rc = lib.kllm_clamped_glu(_p(out), ctypes.c_int64(out.stride(0)), _p(gate), ctypes.c_int64(gate.stride(0)),
                              _p(up), ctypes.c_int64(up.stride(0)), n, f, ctypes.c_float(limit), ctypes.c_float(alpha),
                              dtype_code(out.dtype), _stream())
    _check(lib, "activation", rc)


def sample(out: torch.Tensor, logits: torch.Tensor, temperature: Optional[torch.Tensor],
           uniform: Optional[torch.Tensor], last_token: Optional[torch.Tensor] = None,
           slots: Optional[torch.Tensor] = None, host_out: Optional[torch.Tensor] = None) -> None:
    """out[r] = argmax (temperature[r] <= 0) or the inverse CDF of softmax(z/T) at uniform[r];
    with ``last_token`` and ``slots`` (int32 [rows]) also last_token[slots[r]] = out[r];
    with ``host_out`` (pinned host int32 [rows]) the kernel also writes the choices there itself."""
    _cuda(out, logits, temperature, uniform, last_token, slots)
    if host_out is not None and (host_out.is_cuda or not host_out.is_pinned() or host_out.dtype != torch.int32
                                 or not host_out.is_contiguous() or host_out.numel() < logits.shape[0]):
        raise KernelError("sample: host_out must be a pinned, contiguous int32 host tensor of [rows]")
    _i32(out, "out"); _i32(last_token, "last_token"); _i32(slots, "slots")
    if (last_token is None) != (slots is None) or (slots is not None and slots.numel() != logits.shape[0]):
        raise KernelError("sample: last_token and slots [rows] go together")
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with dense rows")
    for t in (temperature, uniform):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != logits.shape[0]):
            raise KernelError("sample: temperature and uniform must be float32 [rows]")
    lib = load_library("sampling")
    rc = lib.kllm_sample(_p(out), _p(logits), ctypes.c_int64(logits.stride(0)), logits.shape[0],
                         logits.shape[1], _p(temperature), _p(uniform), _p(last_token), _p(slots), _p(host_out), _stream())
    _check(lib, "sampling", rc)


SKINNY_MAX_ROWS = 16
_PRO = {"bf16": 0, "norm": 1}
_EPI = {"bf16": 0, "f32": 1, "add": 2, "swiglu": 3}


SKINNY_F32_MAX_ROWS = 8
SKINNY_F32_MAX_WIDTH = 220 * 1024 // (8 * 4) // 128 * 128      # 8 float32 rows in shared memory


def skinny_fits(n: int, k: int, dtype: torch.dtype, sliced: bool = False) -> bool:
    """Whether the weight-streaming product takes n rows of width k in this dtype
    (bfloat16: csrc/skinny_gemm.cu, up to 16 rows; float32: csrc/skinny_gemm_f32.cu, up to
    8 rows, width a multiple of 128).  ``sliced``: the caller adds into a float32 matrix
    from rows of the weights' dtype, where a width too long for shared memory is taken
    slice by slice."""
    if dtype == torch.float32:
        return 1 <= n <= SKINNY_F32_MAX_ROWS and k >= 128 and k % 128 == 0 and (sliced or k <= SKINNY_F32_MAX_WIDTH)
    if dtype != torch.bfloat16 or not (1 <= n <= SKINNY_MAX_ROWS) or k < 32 or k % 32:
        return False
    return sliced or k <= _skinny_max_width(n)


def _skinny_max_width(n: int) -> int:
    """Largest width (a multiple of 32) whose X rows, the 16 warps' partial tiles and the
    norm's gain fit the 227 KB of shared memory (smem_bytes in csrc/skinny_gemm.cu)."""
    nt = 1 if n <= 8 else 2
    room = 227 * 1024 - 16 * 16 * 8 * nt * 4
    k = room // (8 * nt * 2 + 4) // 32 * 32
    while 8 * nt * (k + (32 if (k * 2) % 128 == 0 else 0)) * 2 + k * 4 > room:
        k -= 32
    return k


def _prefetch_args(t: Optional[torch.Tensor]):
    if t is None or not PREFETCH_L2:
        return None, ctypes.c_int64(0)
    if not t.is_contiguous():
        raise KernelError("prefetch: the tensor to bring into L2 must be contiguous")
    return _p(t), ctypes.c_int64(min(t.numel() * t.element_size(), PREFETCH_L2_BYTES) // 16 * 16)


def skinny_gemm(weight: torch.Tensor, *, x: Optional[torch.Tensor] = None, x_f32: Optional[torch.Tensor] = None,
                gain: Optional[torch.Tensor] = None, eps: float = 0.0, rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None, weight_up: Optional[torch.Tensor] = None, epilogue: str = "bf16",
                out: Optional[torch.Tensor] = None, prefetch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = X @ weight^T for at most 16 rows, the weights streamed once (csrc/skinny_gemm.cu
    for bfloat16 weights, csrc/skinny_gemm_f32.cu for float32 weights: true float32 FMAs,
    at most 8 rows).

    X is either ``x`` ([n, K] in the weights' dtype) or rmsnorm(``x_f32``) * ``gain`` computed
    inside the kernel (rows ``rows`` of x_f32 when given).  ``epilogue``: "store" stores y
    [n, N] in the weights' dtype ("bf16" / "f32" name the dtype); "add" adds y into the
    float32 ``out``; "swiglu" takes ``weight`` as gate and ``weight_up`` as up matrix and
    stores silu(gate) * up [n, N] in the weights' dtype.
    ``prefetch``: a contiguous tensor that a later kernel will stream (the next weight
    matrix); the kernel asks for it to be brought into L2 before its own work.
    A width K too long for shared memory is taken in column slices, one launch each, when
    X is bfloat16 and the epilogue is "add" (the slices' sums meet in ``out``, always in
    the same order).
    """
    _cuda(weight, x, x_f32, gain, rows, weight_up, out, prefetch)
    N, K = weight.shape
    if epilogue == "store":
        epilogue = "f32" if weight.dtype == torch.float32 else "bf16"
    if weight.dtype == torch.float32:
        return _skinny_gemm_f32(weight, x, x_f32, gain, eps, rows, n_rows, weight_up, epilogue, out)
    if weight.dtype != torch.bfloat16 or weight.stride(1) != 1 or weight.stride(0) % 8:
        raise KernelError("skinny_gemm: the weight must be bfloat16 with dense rows at a stride that is a multiple of 8")
    if weight_up is not None and weight_up.stride() != weight.stride():
        raise KernelError("skinny_gemm: the up matrix must be laid out like the gate matrix")
    if x is not None and epilogue == "add" and out is not None and K % 32 == 0 and 1 <= x.shape[0] <= SKINNY_MAX_ROWS \
            and K > _skinny_max_width(x.shape[0]):
        widest = _skinny_max_width(x.shape[0])
        parts = -(-K // widest)
        width = -(-K // parts // 32) * 32
        for lo in range(0, K, width):
            hi = min(K, lo + width)
            skinny_gemm(weight[:, lo:hi], x=x[:, lo:hi], epilogue="add", out=out,
                        prefetch=prefetch if hi == K else None)
        return out
    if x is not None:
        pro, n = 0, x.shape[0]
        if x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.shape[1] != K:
            raise KernelError("skinny_gemm: x must be bfloat16 [n, K] with dense rows")
    else:
        pro = 1
        _i32(rows, "rows")
        n = rows.numel() if rows is not None else x_f32.shape[0]
        if n_rows is not None:
            n = n_rows
        if x_f32.dtype != torch.float32 or not x_f32.is_contiguous() or x_f32.shape[1] != K \
                or gain.dtype != torch.float32 or gain.numel() != K:
            raise KernelError("skinny_gemm: x_f32 [rows, K] and gain [K] must be contiguous float32")
    if not skinny_fits(n, K, torch.bfloat16):
        raise KernelError(f"skinny_gemm: {n} rows of width {K} are not supported")
    epi = _EPI[epilogue]
    if epilogue == "swiglu" and (weight_up is None or weight_up.shape != weight.shape
                                 or weight_up.dtype != torch.bfloat16):
        raise KernelError("skinny_gemm: swiglu needs an up matrix like the gate matrix")
    if out is None:
        if epilogue == "add":
            raise KernelError("skinny_gemm: 'add' needs the matrix to add into")
        out = torch.empty((n, N), dtype=torch.float32 if epilogue == "f32" else torch.bfloat16, device=weight.device)
    want = torch.float32 if epilogue in ("f32", "add") else torch.bfloat16
    if out.dtype != want or out.stride(1) != 1 or out.shape[0] < n or out.shape[1] != N:
        raise KernelError("skinny_gemm: out has the wrong dtype or shape")
    lib = load_library("skinny_gemm")
    y16 = out if want == torch.bfloat16 else None
    y32 = out if want == torch.float32 else None
    rc = lib.kllm_skinny_gemm(_p(weight), _p(weight_up), ctypes.c_int64(weight.stride(0)), N, K, n, _p(x),
                              ctypes.c_int64(x.stride(0) if x is not None else 0), _p(x_f32), _p(gain), _p(rows),
                              ctypes.c_float(eps), _p(y16), _p(y32), ctypes.c_int64(out.stride(0)), pro, epi,
                              *_prefetch_args(prefetch), _stream())
    _check(lib, "skinny_gemm", rc)
    return out


def _skinny_gemm_f32(weight, x, x_f32, gain, eps, rows, n_rows, weight_up, epilogue, out):
    """The float32 form of ``skinny_gemm`` (same arguments; no prefetch hint)."""
    N, K = weight.shape
    if weight.stride(1) != 1 or weight.stride(0) % 4:
        raise KernelError("skinny_gemm: float32 weights need dense rows at a stride that is a multiple of 4")
    if epilogue not in ("f32", "add", "swiglu"):
        raise KernelError(f"skinny_gemm: float32 weights have no epilogue {epilogue!r}")
    if x is not None:
        n = x.shape[0]
        if x.dtype != torch.float32 or x.stride(1) != 1 or x.shape[1] != K:
            raise KernelError("skinny_gemm: x must be float32 [n, K] with dense rows")
        if epilogue == "add" and out is not None and K > SKINNY_F32_MAX_WIDTH and K % 128 == 0 and n <= SKINNY_F32_MAX_ROWS:
            parts = -(-K // SKINNY_F32_MAX_WIDTH)
            width = -(-K // parts // 128) * 128
            for lo in range(0, K, width):
                hi = min(K, lo + width)
                _skinny_gemm_f32(weight[:, lo:hi], x[:, lo:hi], None, None, 0.0, None, None, None, "add", out)
            return out
        src, pro, stride = x, 0, x.stride(0)
    else:
        _i32(rows, "rows")
        n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x_f32.shape[0])
        if x_f32.dtype != torch.float32 or not x_f32.is_contiguous() or x_f32.shape[1] != K \
                or gain.dtype != torch.float32 or gain.numel() != K:
            raise KernelError("skinny_gemm: x_f32 [rows, K] and gain [K] must be contiguous float32")
        src, pro, stride = x_f32, 1, K
    if not skinny_fits(n, K, torch.float32):
        raise KernelError(f"skinny_gemm: {n} float32 rows of width {K} are not supported")
    if epilogue == "swiglu" and (weight_up is None or weight_up.shape != weight.shape or weight_up.dtype != torch.float32
                                 or weight_up.stride() != weight.stride()):
        raise KernelError("skinny_gemm: swiglu needs an up matrix like the gate matrix")
    if out is None:
        if epilogue == "add":
            raise KernelError("skinny_gemm: 'add' needs the matrix to add into")
        out = torch.empty((n, N), dtype=torch.float32, device=weight.device)
    if out.dtype != torch.float32 or out.stride(1) != 1 or out.shape[0] < n or out.shape[1] != N:
        raise KernelError("skinny_gemm: out has the wrong dtype or shape")
    lib = load_library("skinny_gemm_f32")
    rc = lib.kllm_skinny_gemm_f32(_p(weight), _p(weight_up), ctypes.c_int64(weight.stride(0)), N, K, n, _p(src),
                                  ctypes.c_int64(stride), _p(gain), _p(rows), ctypes.c_float(eps), _p(out),
                                  ctypes.c_int64(out.stride(0)), pro, {"f32": 0, "add": 1, "swiglu": 2}[epilogue], _stream())
    _check(lib, "skinny_gemm_f32", rc)
    return out


def linear_add(acc: torch.Tensor, x: torch.Tensor, weight: torch.Tensor) -> None:
    """acc += x @ weight^T through the vendor GEMM library, acc float32 (the residual
    stream), the sum formed in float32 inside the product's epilogue: what the reference
    does in a kernel of its own after cublasSgemm (backend/model.cu:97-110)."""
    _cuda(acc, x, weight)
    if torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("TF32 matmul mode is on; the float32 path must stay true 32-bit")
    if acc.dtype != torch.float32 or not acc.is_contiguous():
        raise KernelError("linear_add: the matrix added into must be contiguous float32")
    if x.dtype == torch.float32:
        torch.addmm(acc, x, weight.t(), out=acc)
    else:
        torch.addmm(acc, x, weight.t(), out_dtype=torch.float32, out=acc)


def _gemm_args(x, weight, weight_up, out, epilogue):
    return (_p(x), ctypes.c_int64(x.stride(0)), _p(weight), ctypes.c_int64(weight.stride(0)), _p(weight_up),
            x.shape[0], weight.shape[0], x.shape[1], _p(out), ctypes.c_int64(out.stride(0)), _EPI[epilogue])


def gemm_fits(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "bf16",
              weight_up: Optional[torch.Tensor] = None) -> bool:
    """Whether ``gemm`` takes these operands (bfloat16, dense rows, k and the row strides
    multiples of 8, 16-byte aligned addresses)."""
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or x.dim() != 2 or weight.dim() != 2:
        return False
    if x.stride(1) != 1 or weight.stride(1) != 1 or out.stride(1) != 1 or x.shape[1] != weight.shape[1]:
        return False
    if weight_up is not None and (weight_up.dtype != torch.bfloat16 or weight_up.shape != weight.shape
                                  or weight_up.stride() != weight.stride()):
        return False
    lib = load_library("gemm_tcgen05")
    return bool(lib.kllm_gemm_tcgen05_fits(*_gemm_args(x, weight, weight_up, out, epilogue)))


def gemm_pays(n: int, N: int, epilogue: str = "bf16", least: int = 75) -> bool:
    """Whether ``gemm``'s tiles of 128 rows x 256 accumulator columns would keep the
    tensor cores of all SMs busy for at least ``least`` percent of the product's time
    (full tiles over waves x SMs); below that the library product adapts its tiling
    better.  Same arithmetic as kllm_gemm_tcgen05_efficiency, without loading the library."""
    if not USE_TCGEN05 or n <= 0 or N <= 0:
        return False
    sms = sm_count()
    nout = 128 if epilogue == "swiglu" else 256
    tiles = -(-n // 128) * -(-N // nout)
    waves = -(-tiles // sms)
    return 100.0 * (n / 128.0) * (N / float(nout)) / (waves * sms) >= least


def gemm(x: torch.Tensor, weight: torch.Tensor, *, epilogue: str = "bf16", out: Optional[torch.Tensor] = None,
         weight_up: Optional[torch.Tensor] = None, bn: int = 0) -> torch.Tensor:
    """y = x @ weight^T on the tcgen05 tensor cores (csrc/gemm_tcgen05.cu), x bfloat16
    [n, K], weight bfloat16 [N, K].

    ``epilogue``: "bf16" / "f32" store y [n, N]; "add" adds y into the float32 ``out``;
    "swiglu" takes ``weight`` as gate and ``weight_up`` as up matrix and stores
    silu(gate) * up as bfloat16 [n, N].  ``bn``: accumulator width of a tile (0 = chosen
    by the tile count).
    """
    _cuda(x, weight, weight_up, out)
    n, N = x.shape[0], weight.shape[0]
    want = torch.float32 if epilogue in ("f32", "add") else torch.bfloat16
    if out is None:
        if epilogue == "add":
            raise KernelError("gemm: 'add' needs the matrix to add into")
        out = torch.empty((n, N), dtype=want, device=x.device)
    if out.dtype != want or out.shape[0] != n or out.shape[1] != N:
        raise KernelError("gemm: out has the wrong dtype or shape")
    if epilogue == "swiglu" and weight_up is None:
        raise KernelError("gemm: swiglu needs an up matrix like the gate matrix")
    if not gemm_fits(x, weight, out, epilogue, weight_up):
        raise KernelError(f"gemm: operands {tuple(x.shape)} x {tuple(weight.shape)} (strides {x.stride()}, "
                          f"{weight.stride()}, out {out.stride()}) are not supported")
    lib = load_library("gemm_tcgen05")
    rc = lib.kllm_gemm_tcgen05(*_gemm_args(x, weight, weight_up, out, epilogue), int(bn), _p(status_word(x.device)),
                               _stream())
    _check(lib, "gemm_tcgen05", rc)
    return out


_bmm_takes_out_dtype = None


def linear_batched(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y[b] = x[b] @ weight[b]^T in float32 for stacked operands x [B, n, K], weight [B, N, K]
    through the vendor GEMM library (one batched product; bfloat16 operands accumulate and
    come out in float32, float32 operands run as true float32)."""
    global _bmm_takes_out_dtype
    _cuda(x, weight)
    if torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("TF32 matmul mode is on; the float32 path must stay true 32-bit")
    wt = weight.transpose(1, 2)
    if x.dtype == torch.float32:
        return torch.bmm(x, wt)
    if _bmm_takes_out_dtype is None:
        try:
            y = torch.bmm(x, wt, out_dtype=torch.float32)
            _bmm_takes_out_dtype = True
            return y
        except (TypeError, RuntimeError):
            _bmm_takes_out_dtype = False
    if _bmm_takes_out_dtype:
        return torch.bmm(x, wt, out_dtype=torch.float32)
    return torch.stack([torch.mm(x[i], wt[i], out_dtype=torch.float32) for i in range(x.shape[0])])


def linear_per_head(x: torch.Tensor, weight: torch.Tensor, transposed: bool = False,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[t, h, :] = weight[h] @ x[t, h, :] for every head h: x [n, H * a] contiguous, weight
    [H, b, a] (``transposed``: weight [H, a, b], used as weight[h]^T), y [n, H * b] in x's dtype.
    One batched product of the vendor GEMM library over the heads, reading x and writing y in
    place at their head strides (bfloat16 operands accumulate in float32; float32 operands
    run as true float32).  x may also be a view [n, H, a] with dense rows of a wider tensor (the
    head of every head's row)."""
    _cuda(x, weight)
    if torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("TF32 matmul mode is on; the float32 path must stay true 32-bit")
    n, H = x.shape[0], weight.shape[0]
    a = weight.shape[1] if transposed else weight.shape[2]
    b = weight.shape[2] if transposed else weight.shape[1]
    if x.dim() == 3:
        if x.dtype != weight.dtype or tuple(x.shape) != (n, H, a) or x.stride(2) != 1:
            raise KernelError("linear_per_head: a view x must be [n, heads, a] with dense rows, in the weights' dtype")
    elif x.dtype != weight.dtype or not x.is_contiguous() or x.shape[1] != H * a:
        raise KernelError("linear_per_head: x must be contiguous [n, heads * a] in the weights' dtype")
    x = x if x.dim() == 3 else x.view(n, H, a)
    if out is not None:
        # the heads' results into a view [n, H, b] of a wider row (rows dense in b)
        if tuple(out.shape) != (n, H, b) or out.dtype != x.dtype or out.stride(2) != 1:
            raise KernelError("linear_per_head: out must be a view [n, heads, b] in x's dtype with dense rows")
        y3 = out.transpose(0, 1)
        if out.stride(0) % 8 == 0 and out.stride(1) % 8 == 0 and out.data_ptr() % 16 == 0:
            torch.bmm(x.transpose(0, 1), weight if transposed else weight.transpose(1, 2), out=y3)
        else:
            y3.copy_(torch.bmm(x.transpose(0, 1), weight if transposed else weight.transpose(1, 2)))
        return out
    y = torch.empty((n, H * b), dtype=x.dtype, device=x.device)
    torch.bmm(x.transpose(0, 1), weight if transposed else weight.transpose(1, 2),
              out=y.view(n, H, b).transpose(0, 1))
    return y


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, small_ok: bool = False) -> torch.Tensor:
    """y = x @ weight^T through the vendor GEMM library (cuBLAS, via torch.mm), as
    the reference does for every projection (backend/model.cu:496-503).

    float32 operands run as true float32 (the reduced-precision TF32 mode stays
    off); bfloat16 operands accumulate in float32.  ``small_ok`` with a float32 result: a step
    of a few rows (``skinny_fits``) takes this repository's weight-streaming product instead,
    which reads the matrix once at the speed of HBM; which of the two runs depends on the row
    count alone.
    """
    _cuda(x, weight)
    if (small_ok and out is None and out_dtype == torch.float32 and x.dtype == weight.dtype and x.dim() == 2
            and x.stride(1) == 1 and weight.stride(1) == 1 and skinny_fits(x.shape[0], x.shape[1], x.dtype)
            and weight.stride(0) % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0):
        return skinny_gemm(weight, x=x, epilogue="f32")
    if torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("TF32 matmul mode is on; the float32 path must stay true 32-bit")
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    if out is not None:
        return torch.mm(x, weight.t(), out=out)
    return torch.mm(x, weight.t())


# ---- recurrent mixer (csrc/wkv.cu) ---------------------------------------------------

def wkv_shift_mix(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, prev_off: int, ctx) -> torch.Tensor:
    """[n_mix, n, d] = h + (h_prev - h) * mu[m]: h [n, d] in the model dtype, mu float32
    [n_mix, d]; h_prev is the row before in the same request, for a request's first row of
    the step what ``state[slot, prev_off : prev_off + d]`` holds, which is then replaced by the
    request's last row."""
    _cuda(h, mu, state)
    n, d = h.shape
    if not h.is_contiguous() or mu.dtype != torch.float32 or not mu.is_contiguous() or mu.shape[1] != d:
        raise KernelError("wkv_shift_mix: h contiguous [n, d], mu float32 [mixes, d]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or prev_off + d > state.shape[1]:
        raise KernelError("wkv_shift_mix: the state must be float32 [slots, size] with room for a row at prev_off")
    out = torch.empty((mu.shape[0], n, d), dtype=h.dtype, device=h.device)
    lib = load_library("wkv")
    rc = lib.kllm_wkv_shift_mix(_p(out), _p(h), _p(mu), _p(state), ctypes.c_int64(state.stride(0)),
                                ctypes.c_int64(prev_off), _p(ctx.q_start), _p(ctx.token_req), _p(ctx.state_slots), n, d,
                                mu.shape[0], dtype_code(h.dtype), _stream())
    _check(lib, "wkv", rc)
    return out


def _f32_rows(t: torch.Tensor, cols: int, what: str):
    if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or t.shape[1] != cols:
        raise KernelError(f"{what} must be float32 [n, {cols}] with dense rows")


def wkv_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, w0: torch.Tensor, u: torch.Tensor,
             state: torch.Tensor, ctx, heads: int, size: int) -> torch.Tensor:
    """The recurrence o_j = sum_i r_i (S_ij + u_i k_i v_j), S_ij <- w_i S_ij + k_i v_j with
    w = exp(-exp(z + w0)), per head over every request's rows in order; S [heads, size, size]
    is the head of ``state[slot]`` (float32) and is carried on.  All operands float32."""
    _cuda(r, k, v, z, w0, u, state)
    A = heads * size
    for t, what in ((r, "r"), (k, "k"), (v, "v"), (z, "z")):
        _f32_rows(t, A, "wkv_scan: " + what)
    if w0.dtype != torch.float32 or u.dtype != torch.float32 or w0.numel() != A or u.numel() != A \
            or not w0.is_contiguous() or not u.is_contiguous():
        raise KernelError("wkv_scan: w0 and u must be contiguous float32 [heads * size]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < A * size:
        raise KernelError("wkv_scan: the state must be float32 [slots, >= heads * size * size]")
    o = torch.empty((r.shape[0], A), dtype=torch.float32, device=r.device)
    lib = load_library("wkv")
    rc = lib.kllm_wkv_scan(_p(o), ctypes.c_int64(o.stride(0)), _p(r), ctypes.c_int64(r.stride(0)), _p(k),
                           ctypes.c_int64(k.stride(0)), _p(v), ctypes.c_int64(v.stride(0)), _p(z),
                           ctypes.c_int64(z.stride(0)), _p(w0), _p(u), _p(state), ctypes.c_int64(state.stride(0)),
                           _p(ctx.q_start), _p(ctx.state_slots), r.shape[0], ctx.n_requests, heads, size, _stream())
    _check(lib, "wkv", rc)
    return o


def wkv_decay_outer(low: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """z = tanh(low) @ w2^T in float32: low float32 [n, R] (the inner half of the decay's
    low-rank product), w2 [A, R] in the model dtype; R is a handful."""
    _cuda(low, w2)
    n, R = low.shape
    if low.dtype != torch.float32 or low.stride(1) != 1 or not w2.is_contiguous() or w2.shape[1] != R:
        raise KernelError("wkv_decay_outer: low float32 [n, R] with dense rows, w2 contiguous [A, R]")
    z = torch.empty((n, w2.shape[0]), dtype=torch.float32, device=low.device)
    lib = load_library("wkv")
    rc = lib.kllm_wkv_decay_outer(_p(z), _p(low), ctypes.c_int64(low.stride(0)), _p(w2), n, w2.shape[0], R,
                                  dtype_code(w2.dtype), _stream())
    _check(lib, "wkv", rc)
    return z


def wkv_gate_norm(o: torch.Tensor, g: torch.Tensor, gain: torch.Tensor, eps: float, heads: int, size: int,
                  dtype: torch.dtype) -> torch.Tensor:
    """y = o / rms(o over each head's ``size`` values) * gain * silu(g), stored in ``dtype``."""
    _cuda(o, g, gain)
    A = heads * size
    _f32_rows(o, A, "wkv_gate_norm: o"); _f32_rows(g, A, "wkv_gate_norm: g")
    if gain.dtype != torch.float32 or gain.numel() != A or not gain.is_contiguous():
        raise KernelError("wkv_gate_norm: gain must be contiguous float32 [heads * size]")
    y = torch.empty((o.shape[0], A), dtype=dtype, device=o.device)
    lib = load_library("wkv")
    rc = lib.kllm_wkv_gate_norm(_p(y), _p(o), ctypes.c_int64(o.stride(0)), _p(g), ctypes.c_int64(g.stride(0)), _p(gain),
                                o.shape[0], heads, size, ctypes.c_float(eps), dtype_code(dtype), _stream())
    _check(lib, "wkv", rc)
    return y


_UNARY = {"relu2": 0, "tanh": 1, "copy": 2, "gelu": 3, "gelu_tanh": 4, "softcap": 5}


def unary(x: torch.Tensor, op: str, dtype: torch.dtype, arg: float = 0.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """f(x) elementwise of a float32 matrix with dense rows, stored in ``dtype``; ``op``:
    "relu2" (the square of relu), "tanh", "copy" (the value itself: a change of dtype), "gelu" (with the
    error function), "gelu_tanh" (its tanh form) or "softcap" (arg * tanh(x / arg)).  ``out``: where to
    store (x itself for a float32 result in place)."""
    _cuda(x, out)
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("unary: the input must be a float32 matrix with dense rows")
    if out is None:
        out = torch.empty(x.shape, dtype=dtype, device=x.device)
    elif out.dtype != dtype or out.shape != x.shape or out.stride(1) != 1:
        raise KernelError("unary: out must have x's shape, dense rows and the named dtype")
    lib = load_library("activation")
    rc = lib.kllm_unary(_p(out), ctypes.c_int64(out.stride(0)), _p(x), ctypes.c_int64(x.stride(0)), x.shape[0],
                        x.shape[1], _UNARY[op], ctypes.c_float(arg), dtype_code(dtype), _stream())
    _check(lib, "activation", rc)
    return out


# ---- linear attention with a fixed decay per head (csrc/lightning.cu) -------------------

def lightning_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, ctx,
                   heads: int, dk: int, dv: int) -> torch.Tensor:
    """o float32 [n, heads * dv] of the recurrence S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head, with
    q, k, v = silu of the float32 projections given here (rows of heads * dk, heads * dk, heads * dv values, dense,
    at their own row strides); ``state`` float32 [slots, >= heads * dk * dv] holds S as [heads, dk, dv] per
    request slot and is carried on; every request's rows are taken in order."""
    _cuda(q, k, v, decay, state)
    _f32_rows(q, heads * dk, "lightning_scan: q"); _f32_rows(k, heads * dk, "lightning_scan: k")
    _f32_rows(v, heads * dv, "lightning_scan: v")
    if decay.dtype != torch.float32 or decay.numel() != heads or not decay.is_contiguous():
        raise KernelError("lightning_scan: one float32 decay per head")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < heads * dk * dv:
        raise KernelError("lightning_scan: the state must be float32 [slots, >= heads * dk * dv]")
    _i32(ctx.q_start, "q_start"); _i32(ctx.state_slots, "state_slots")
    o = torch.empty((q.shape[0], heads * dv), dtype=torch.float32, device=q.device)
    lib = load_library("lightning")
    if not ctx.all_single:
        # portions: the chunks' own sums in parallel, then the state's walk (two kernels; see csrc/lightning.cu)
        n = q.shape[0]
        work = torch.empty((3, n, heads * max(dk, dv)), dtype=torch.float32, device=q.device)
        rc = lib.kllm_lightning_scan_portions(_p(o), ctypes.c_int64(o.stride(0)), _p(q), ctypes.c_int64(q.stride(0)), _p(k),
                                              ctypes.c_int64(k.stride(0)), _p(v), ctypes.c_int64(v.stride(0)), _p(decay),
                                              _p(state), ctypes.c_int64(state.stride(0)), _p(ctx.q_start),
                                              _p(ctx.state_slots), n, ctx.n_requests, n // 32 + ctx.n_requests, heads, dk,
                                              dv, _p(work[0]), _p(work[1]), _p(work[2]), _stream())
        if rc != -3:
            _check(lib, "lightning", rc)
            global launches
            launches += 1
            return o
    rc = lib.kllm_lightning_scan(_p(o), ctypes.c_int64(o.stride(0)), _p(q), ctypes.c_int64(q.stride(0)), _p(k),
                                 ctypes.c_int64(k.stride(0)), _p(v), ctypes.c_int64(v.stride(0)), _p(decay), _p(state),
                                 ctypes.c_int64(state.stride(0)), _p(ctx.q_start), _p(ctx.state_slots), q.shape[0],
                                 ctx.n_requests, heads, dk, dv, _stream())
    _check(lib, "lightning", rc)
    return o


def lightning_gate_norm(o: torch.Tensor, g: torch.Tensor, gain: torch.Tensor, eps: float, dtype: torch.dtype) -> torch.Tensor:
    """y = o / rms(o over the whole row) * gain * sigmoid(g), stored in ``dtype``; o, g float32 [n, width] with dense rows."""
    _cuda(o, g, gain)
    width = o.shape[1]
    _f32_rows(o, width, "lightning_gate_norm: o"); _f32_rows(g, width, "lightning_gate_norm: g")
    if gain.dtype != torch.float32 or gain.numel() != width or not gain.is_contiguous() or g.shape[0] != o.shape[0]:
        raise KernelError("lightning_gate_norm: gain must be contiguous float32 [width], g as many rows as o")
    y = torch.empty((o.shape[0], width), dtype=dtype, device=o.device)
    lib = load_library("lightning")
    rc = lib.kllm_lightning_gate_norm(_p(y), _p(o), ctypes.c_int64(o.stride(0)), _p(g), ctypes.c_int64(g.stride(0)),
                                      _p(gain), o.shape[0], width, ctypes.c_float(eps), dtype_code(dtype), _stream())
    _check(lib, "lightning", rc)
    return y


# ---- attention with scores mixed across the heads (csrc/attention_mixed.cu) ---------------

_mixed_tile_rows = {}
MIXED_MMA = os.environ.get("KLLM_B200_MIXED_MMA", "1") != "0"     # bfloat16 portions on the tensor-core forms
MIXED_CLUSTER = os.environ.get("KLLM_B200_MIXED_CLUSTER", "1") != "0"   # ... of which the cluster form goes first


def attention_mixed(out: torch.Tensor, q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, mix: torch.Tensor,
                    ctx, block_table: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, v_head_dim: int,
                    window: int, scale: float, sinks: Optional[torch.Tensor] = None) -> None:
    """Causal grouped attention of the step's tokens over the paged cache whose scaled scores are mixed across the
    heads before mask and softmax: s_h = sum_g mix[h, g] * scale * q_g . k_kv(g); ``mix`` float32 [H, H]; ``window``
    W > 0: a query sees the last W keys, its own included; ``sinks`` (float32 [H]): exp(sinks[h]) joins the
    denominator of head h.  Scores, mixing, weights and sums are float32 in both dtypes.  Two forms: on the CUDA
    cores, single tokens as tiles of one row and portions as tiles of up to eight rows of one request (float32, and
    every decoding step); on the tensor cores (mma.sync, bfloat16 steps that hold a portion, head sizes in steps of
    16), tiles of 16 rows by a block of heads, the weights entering the second product as two bfloat16 terms: either
    the blocks of heads of a tile form a thread-block cluster and read each other's raw scores from distributed
    shared memory (heads in 2 to 8 equal blocks), or every block computes all heads' raw scores itself."""
    _cuda(out, q, kcache, vcache, mix, block_table, sinks)
    _i32(block_table, "block_table"); _i32(ctx.q_start, "q_start"); _i32(ctx.start_pos, "start_pos")
    _slopes_arg(sinks, n_heads, "sinks")
    n = q.shape[0]
    if (q.stride(1) != 1 or q.shape[1] != n_heads * head_dim or not out.is_contiguous() or out.dtype != q.dtype
            or tuple(out.shape) != (n, n_heads * v_head_dim) or kcache.dtype != q.dtype or vcache.dtype != q.dtype):
        raise KernelError("attention_mixed: q [n, H dk] with dense rows, out contiguous [n, H dv], one dtype with the caches")
    page_size = kcache.shape[2]
    if (not kcache.is_contiguous() or not vcache.is_contiguous() or tuple(kcache.shape[1:]) != (n_kv, page_size, head_dim)
            or tuple(vcache.shape) != (kcache.shape[0], n_kv, page_size, v_head_dim)):
        raise KernelError("attention_mixed: caches [pages, kv heads, page_size, size]")
    if mix.dtype != torch.float32 or not mix.is_contiguous() or tuple(mix.shape) != (n_heads, n_heads):
        raise KernelError("attention_mixed: the mixing matrix must be contiguous float32 [heads, heads]")
    lib = load_library("attention_mixed")
    key = (n_heads, n_kv, head_dim, v_head_dim)
    if (MIXED_MMA and q.dtype == torch.bfloat16 and not ctx.all_single and q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0):
        tiles = ctx.n_tokens // 16 + ctx.n_requests
        args = (_p(out), _p(q), ctypes.c_int64(q.stride(0)), _p(kcache), _p(vcache), _p(mix), _p(sinks), _p(ctx.q_start),
                _p(ctx.start_pos), _p(block_table), block_table.shape[1], ctx.n_requests, int(tiles), n_heads, n_kv, head_dim,
                v_head_dim, page_size, int(window or 0), ctypes.c_float(scale), _stream())
        # first the form in which the blocks of heads of a tile share their raw scores across a cluster of CTAs
        if MIXED_CLUSTER and lib.kllm_attention_mixed_cluster_fits(*key):
            rc = lib.kllm_attention_mixed_cluster(*args)
            if rc != -3:
                _check(lib, "attention_mixed", rc)
                return
        if lib.kllm_attention_mixed_mma_fits(*key):
            rc = lib.kllm_attention_mixed_mma(*args)
            _check(lib, "attention_mixed", rc)
            return
    if key not in _mixed_tile_rows:
        _mixed_tile_rows[key] = int(lib.kllm_attention_mixed_tile_rows(*key))
    rows = _mixed_tile_rows[key]
    if rows <= 0:
        raise KernelError(f"attention_mixed: {n_heads} heads of sizes {head_dim}, {v_head_dim} do not fit a CTA's shared memory")
    if ctx.all_single:
        rows = 1
    tiles = ctx.n_requests if rows == 1 else ctx.n_tokens // rows + ctx.n_requests
    # single tokens: the keys a token sees are cut into ranges of whole key tiles, one CTA each, as many as fill the
    # SMs once, at least two tiles a range; a second kernel joins them in range order
    splits, part_o, part_ml = 1, None, None
    if ctx.all_single:
        bound = ctx.split_bound or ctx.max_ctx
        if window:
            bound = min(bound, int(window))
        tile_keys = int(lib.kllm_attention_mixed_tile_keys(n_heads, n_kv, head_dim, v_head_dim, 1))
        splits = max(1, min(-(-bound // (2 * tile_keys)), sm_count() // max(1, ctx.n_requests), 32))
        if splits > 1:
            part_o = torch.empty((n, splits, n_heads * v_head_dim), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((n, splits, n_heads, 2), dtype=torch.float32, device=q.device)
    rc = lib.kllm_attention_mixed(_p(out), _p(q), ctypes.c_int64(q.stride(0)), _p(kcache), _p(vcache), _p(mix), _p(sinks),
                                  _p(ctx.q_start), _p(ctx.start_pos), _p(block_table), block_table.shape[1],
                                  ctx.n_requests, int(tiles), int(rows), n_heads, n_kv, head_dim, v_head_dim, page_size,
                                  int(window or 0), ctypes.c_float(scale), int(splits), _p(part_o), _p(part_ml),
                                  dtype_code(q.dtype), _stream())
    _check(lib, "attention_mixed", rc)
    if splits > 1:
        global launches
        launches += 1           # the merging kernel


# ---- routed experts (csrc/moe.cu) ------------------------------------------------------

_GATED_ACT = {"silu": 0, "clamped": 1}

def moe_route(h: torch.Tensor, router: torch.Tensor, top: int, score: str = "sigmoid", renormalize: bool = False,
              groups: int = 1, keep: int = 1):
    """(idx int32 [n, top], weights float32 [n, top]): logits router @ h in float32, scores by
    ``score`` ("sigmoid" or "softmax"), the ``top`` largest, the lower index among equals.  With
    ``groups`` > 1 the experts form that many equal groups of neighbours, a group scores as its best
    expert, and only experts of the ``keep`` best groups can be chosen."""
    _cuda(h, router)
    n, d = h.shape
    if not h.is_contiguous() or router.dtype != torch.float32 or not router.is_contiguous() or router.shape[1] != d:
        raise KernelError("moe_route: h contiguous [n, d], router float32 [experts, d]")
    if score not in ("sigmoid", "softmax"):
        raise KernelError(f"moe_route: unknown score {score!r}")
    idx = torch.empty((n, top), dtype=torch.int32, device=h.device)
    wt = torch.empty((n, top), dtype=torch.float32, device=h.device)
    lib = load_library("moe")
    rc = lib.kllm_moe_route(_p(idx), _p(wt), _p(h), _p(router), n, d, router.shape[0], int(top),
                            int(score == "softmax"), int(bool(renormalize)), int(groups or 1), int(keep or 1),
                            dtype_code(h.dtype), _stream())
    _check(lib, "moe", rc)
    return idx, wt


def moe_sort(idx: torch.Tensor, experts: int):
    """(offsets int32 [experts + 1], perm int32 [rows]): the flattened (token, choice) pairs
    ordered by expert; sorted row r is pair perm[r], expert e owns rows offsets[e] ..
    offsets[e + 1]."""
    _cuda(idx)
    _i32(idx, "idx")
    rows = idx.numel()
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=idx.device)
    perm = torch.empty(rows, dtype=torch.int32, device=idx.device)
    rank = torch.empty(rows, dtype=torch.int32, device=idx.device)
    lib = load_library("moe")
    rc = lib.kllm_moe_sort(_p(offsets), _p(perm), _p(rank), _p(idx), rows, int(experts), _stream())
    _check(lib, "moe", rc)
    return offsets, perm


def moe_gemm(a: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, perm: torch.Tensor, wt: torch.Tensor, top: int,
             gated: bool, scale_in: bool = False, scale_out: bool = False, activation: str = "silu",
             limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """The experts' products over rows sorted by expert (``moe_sort``).  ``gated``: a is the
    layer's input [tokens, K], w [E, 2N, K] (gate rows, then up rows); returns silu(gate) * up
    [rows, N] in a's dtype, sorted order, the input row times its weight when ``scale_in``.
    Otherwise a is [rows, K] in sorted order, w [E, N, K]; returns float32 [rows, N] with row
    token * top + choice, times its weight when ``scale_out``.  ``activation`` of the gated
    form: "silu" (silu(g) * u) or "clamped" (with g' = min(g, limit) and u' = clamp(u, -limit,
    limit): g' * sigmoid(alpha g') * (u' + 1))."""
    _cuda(a, w, offsets, perm, wt)
    if activation not in _GATED_ACT or (activation == "clamped" and not limit > 0):
        raise KernelError(f"moe_gemm: activation {activation!r} (silu, or clamped with a positive limit)")
    _i32(offsets, "offsets"); _i32(perm, "perm")
    rows = perm.numel()
    E, N, K = w.shape
    if gated:
        N //= 2
    if a.dtype != w.dtype or a.stride(1) != 1 or a.shape[1] != K or not w.is_contiguous():
        raise KernelError("moe_gemm: a [., K] with dense rows and w [E, ., K] contiguous, of one dtype")
    if wt.dtype != torch.float32 or not wt.is_contiguous() or wt.numel() != rows:
        raise KernelError("moe_gemm: one float32 weight per (token, choice)")
    c = torch.empty((rows, N), dtype=a.dtype if gated else torch.float32, device=a.device)
    lib = load_library("moe")
    rc = lib.kllm_moe_gemm(_p(c), _p(a), ctypes.c_int64(a.stride(0)), _p(w), _p(offsets), _p(perm), _p(wt), rows, E,
                           int(top), N, K, int(gated), int(scale_in), int(scale_out), _GATED_ACT[activation],
                           ctypes.c_float(limit), ctypes.c_float(alpha), dtype_code(a.dtype), _stream())
    _check(lib, "moe", rc)
    return c


MOE_TCGEN05_ROWS = 64      # rows per expert on average from which a step's experts run on the tcgen05 kernel


def moe_gemm_tcgen05_pays(a: torch.Tensor, w: torch.Tensor, rows: int, gated: bool, scale_in: bool) -> bool:
    """Whether ``moe_gemm_tcgen05`` takes these operands and the step is large enough for tiles of 128
    rows per expert: bfloat16, no weight on the experts' inputs (TMA brings the rows to the tensor
    cores as they are), rows and matrices in whole 16-byte pieces and at least as wide as one 64-column k
    block (a layer's two products have the same two widths, so one answer holds for both)."""
    E, N, K = w.shape
    if gated:
        N //= 2
    return (USE_TCGEN05 and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and not scale_in and E <= 512
            and rows >= 512 and rows >= MOE_TCGEN05_ROWS * E and K % 8 == 0 and N % 8 == 0 and min(K, N) >= 64
            and w.is_contiguous()
            and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def moe_gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, perm: torch.Tensor, wt: torch.Tensor,
                     top: int, gated: bool, scale_out: bool = False, activation: str = "silu", limit: float = 0.0,
                     alpha: float = 1.0) -> torch.Tensor:
    """``moe_gemm`` for large steps in bfloat16 on the tcgen05 tensor cores (csrc/moe_gemm_tcgen05.cu), same
    operands and results; the weights may act on the experts' outputs only.  The gated form first gathers
    the layer's input into sorted order, one row per (token, choice)."""
    _cuda(a, w, offsets, perm, wt)
    if activation not in _GATED_ACT or (activation == "clamped" and not limit > 0):
        raise KernelError(f"moe_gemm: activation {activation!r} (silu, or clamped with a positive limit)")
    _i32(offsets, "offsets"); _i32(perm, "perm")
    rows = perm.numel()
    E, N, K = w.shape
    if gated:
        N //= 2
    if not moe_gemm_tcgen05_pays(a, w, rows, gated, False) or a.shape[1] != K:
        raise KernelError("moe_gemm_tcgen05: operands not taken (bfloat16, rows of whole 16-byte pieces, a large step)")
    if wt.dtype != torch.float32 or not wt.is_contiguous() or wt.numel() != rows:
        raise KernelError("moe_gemm: one float32 weight per (token, choice)")
    lib = load_library("moe_gemm_tcgen05")
    if gated:
        xs = torch.empty((rows, K), dtype=a.dtype, device=a.device)
        rc = lib.kllm_moe_gather_sorted(_p(xs), _p(a), ctypes.c_int64(a.stride(0)), _p(perm), rows, int(top), K, _stream())
        _check(lib, "moe_gemm_tcgen05", rc)
        a = xs
    elif not a.is_contiguous() or a.shape[0] != rows:
        raise KernelError("moe_gemm_tcgen05: the sorted rows must be contiguous")
    c = torch.empty((rows, N), dtype=a.dtype if gated else torch.float32, device=a.device)
    rc = lib.kllm_moe_gemm_tcgen05(_p(c), _p(a), _p(w), _p(offsets), _p(perm), _p(wt), rows, E, N, K, int(gated),
                                   int(scale_out), _GATED_ACT[activation], ctypes.c_float(limit), ctypes.c_float(alpha),
                                   _p(status_word(a.device)), _stream())
    _check(lib, "moe_gemm_tcgen05", rc)
    return c


def moe_combine(parts: torch.Tensor, top: int, shared: Optional[torch.Tensor] = None,
                gate: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """y[t] = sum of parts[t * top + j] over j in order; float32.  With ``shared`` (float32
    [n, d], the output of an expert that every token runs) also + shared[t] * sigmoid(gate[t]),
    ``gate`` being a float32 column of one logit per token (None: the rows are added as they are).
    ``scale`` multiplies the sum over j (one weight that all of a token's choices share)."""
    _cuda(parts, shared, gate)
    if top == 1 and shared is None and scale == 1.0:
        return parts            # nothing to add up: the rows themselves
    n, d = parts.shape[0] // top, parts.shape[1]
    if not parts.is_contiguous() or parts.dtype != torch.float32:
        raise KernelError("moe_combine: the experts' rows must be contiguous float32")
    if shared is not None and (shared.dtype != torch.float32 or not shared.is_contiguous() or shared.shape != (n, d)):
        raise KernelError("moe_combine: the shared expert's rows must be contiguous float32 [n, d]")
    if gate is not None and (shared is None or gate.dtype != torch.float32 or gate.dim() != 2 or gate.shape[0] != n):
        raise KernelError("moe_combine: the gate is a float32 column [n, 1] beside a shared expert")
    y = torch.empty((n, d), dtype=torch.float32, device=parts.device)
    lib = load_library("moe")
    rc = lib.kllm_moe_combine(_p(y), _p(parts), n, d, int(top), _p(shared), _p(gate),
                              ctypes.c_int64(gate.stride(0) if gate is not None else 0), ctypes.c_float(scale), _stream())
    _check(lib, "moe", rc)
    return y


def moe_table_route(token_ids: torch.Tensor, table: torch.Tensor, experts: int, weight: float,
                    last_token: Optional[torch.Tensor] = None):
    """(idx int32 [n, top], weights float32 [n, top]) from a table int32 [vocab, top] that gives
    every token id its experts; every pair gets ``weight``.  An id -(s + 1) stands for
    ``last_token[s]`` (a choice of the step before that is still on the device)."""
    _cuda(token_ids, table, last_token)
    _i32(token_ids, "token_ids"); _i32(table, "table"); _i32(last_token, "last_token")
    n, (vocab, top) = token_ids.numel(), table.shape
    idx = torch.empty((n, top), dtype=torch.int32, device=table.device)
    wt = torch.empty((n, top), dtype=torch.float32, device=table.device)
    lib = load_library("moe")
    rc = lib.kllm_moe_table_route(_p(idx), _p(wt), _p(token_ids), _p(last_token), _p(table), n, vocab, int(experts),
                                  top, ctypes.c_float(weight), _stream())
    _check(lib, "moe", rc)
    return idx, wt
