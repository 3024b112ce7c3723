"""Wrappers and kernel choice for latent attention (``csrc/latent_attention.cu``, ``csrc/latent_attention_mma.cu``).

Queries and results are head-major, [H, rows, width], so that the per-head products with the key and value
up-projections are grouped matrix products (one group per head).  ``rows`` is the number of tokens, rounded up to
whole 128-row tiles where the tcgen05 grouped product runs."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong
from typing import Optional

import torch

from . import _check, _dt, _i32, _ptr, _stream, gemm_tiled, lib
from .layer_ops import _act_args, _f32

TILE = 128


def prepare(proj: torch.Tensor, q_off: int, kv_off: int, norm_w: torch.Tensor, eps: float, freq: Optional[torch.Tensor],
            pairing: str, amp: float, positions, tok_entry, block_table, cache: torch.Tensor, page_size: int,
            q_plain: torch.Tensor, q_rot: torch.Tensor, n_tokens: int, H: int, D: int, R: int, C: int,
            write_cache: bool = True, q_src: Optional[torch.Tensor] = None) -> None:
    """From the input product (float32 [T, >= ...]): the normed latent and the rotated key part go to the token's
    page, the plain query parts to q_plain [H, rows, D], the rotated ones to q_rot float32 [H, rows, R].  ``freq``: the
    rotary table in float64 (the angle is formed in 64-bit).  ``q_src`` (float32 [T, >= q_off + H (D + R)]): the
    queries come from this array instead of ``proj`` (a product of their own)."""
    if q_src is None:
        q_src = proj
    assert q_src.dtype == torch.float32 and q_src.stride(1) == 1 and q_src.shape[0] == proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and cache.is_contiguous() and cache.shape[-1] == C + R
    assert cache.shape[1] == 1 and q_plain.dtype == cache.dtype and q_plain.is_contiguous() and q_rot.dtype == torch.float32
    rows = q_plain.shape[1]
    assert tuple(q_plain.shape) == (H, rows, D) and tuple(q_rot.shape) == (H, rows, R) and q_rot.is_contiguous()
    assert freq is None or (freq.dtype == torch.float64 and freq.is_contiguous())
    rot = 0 if freq is None else 2 * freq.numel()
    _check(lib().infero_latent_prepare_from(
        _ptr(proj), c_int(proj.stride(0)), _ptr(q_src), c_int(q_src.stride(0)), c_int(q_off), c_int(kv_off), _ptr(_f32(norm_w, "norm_w")), c_float(eps),
        _ptr(freq), c_int(rot), c_int(1 if pairing == "adjacent" else 0), c_float(amp),
        _ptr(_i32(positions, "positions")), _ptr(_i32(tok_entry, "tok_entry")), _ptr(_i32(block_table, "block_table")),
        c_int(block_table.shape[1]), c_int(page_size), _ptr(cache), c_int(_dt(cache)), c_int(1 if write_cache else 0),
        _ptr(q_plain), _ptr(q_rot), c_longlong(rows), c_int(n_tokens), c_int(H), c_int(D), c_int(R), c_int(C), _stream()))


def grouped_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Can the tcgen05 grouped product take a [H, rows, K] x w [H, N, K]?"""
    from .tc_gemm import supported
    return (a.dtype == torch.bfloat16 and a.shape[1] % TILE == 0 and supported(a.view(-1, a.shape[2]), w.view(-1, w.shape[2])))


_TILE_HEAD = {}


def _tile_heads(H: int, rows: int, device) -> torch.Tensor:
    """tile -> head for [H, rows] in 128-row tiles, followed by the number of rows in use."""
    key = (H, rows, str(device))
    t = _TILE_HEAD.get(key)
    if t is None:
        per = rows // TILE
        # (made by device operations: a step that is being captured into a graph may meet a new size)
        t = torch.cat([torch.arange(H * per, dtype=torch.int32, device=device) // per,
                       torch.full((1,), H * rows, dtype=torch.int32, device=device)])
        if len(_TILE_HEAD) > 256:
            _TILE_HEAD.clear()
        _TILE_HEAD[key] = t
    return t


def per_head_product(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, n_rows: int) -> None:
    """out[n] = a[n] @ w[n]^T for every head n; a [H, rows, K], w [H, N, K], out float32 [H, rows, N].  The tcgen05
    grouped product where it applies (bf16, whole tiles), else one product per head on the first ``n_rows`` rows."""
    H, rows, Kd = a.shape
    N = w.shape[1]
    assert out.dtype == torch.float32 and tuple(out.shape) == (H, rows, N) and w.is_contiguous() and a.is_contiguous()
    if grouped_ok(a, w):
        from .tc_gemm import sm_count
        _check(lib().infero_gemm_tc_grouped(_ptr(a), _ptr(w), _ptr(out), c_int(0), c_int(H * rows), c_int(N), c_int(Kd),
                                            c_int(Kd), c_int(N), _ptr(_tile_heads(H, rows, a.device)), c_int(H),
                                            c_int(sm_count(a.device)), *_act_args(None), _stream()))
        return
    for n in range(H):
        gemm_tiled(a[n, :n_rows], w[n], None, out[n, :n_rows])


def attention(ctx, q_lat: torch.Tensor, q_rot: torch.Tensor, out: torch.Tensor, kv, table, n_tokens: int, H: int, C: int,
              R: int, scale: float) -> None:
    """Causal softmax attention of every token over its request's cached latent rows: q_lat float32 [H, rows, C],
    q_rot float32 [H, rows, R], out [H, rows, C] of the cache's type."""
    cache = kv.k
    rows = q_lat.shape[1]
    assert q_lat.dtype == torch.float32 and q_rot.dtype == torch.float32 and q_lat.is_contiguous() and q_rot.is_contiguous()
    assert out.dtype == cache.dtype and out.is_contiguous() and tuple(out.shape) == (H, rows, C) and cache.is_contiguous()
    from . import latent_mma
    if latent_mma.run(ctx, q_lat, q_rot, out, kv, table, n_tokens, H, C, R, scale):
        return
    _check(lib().infero_latent_attention_generic(
        _ptr(q_lat), _ptr(q_rot), c_longlong(rows), _ptr(out), _ptr(cache), c_int(_dt(cache)),
        _ptr(_i32(table, "block_table")), c_int(table.shape[1]), _ptr(_i32(ctx.tok_entry, "tok_entry")),
        _ptr(_i32(ctx.positions, "positions")), c_int(0), c_int(n_tokens), c_int(H), c_int(C), c_int(R),
        c_int(kv.page_size), c_float(scale), _stream()))


def finish(val: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, n_tokens: int, H: int, V: int) -> None:
    """out[t, n * V + v] = val[n, t, v] * sigmoid(gate[t, n]); val float32 [H, rows, V], gate float32 [T, H] (a column
    slice is fine) or None."""
    assert val.dtype == torch.float32 and val.is_contiguous() and out.stride(1) == 1 and out.shape[1] == H * V
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[1] == H)
    _check(lib().infero_latent_finish(_ptr(val), c_longlong(val.shape[1]), _ptr(gate), c_int(gate.stride(0) if gate is not None else 0),
                                      _ptr(out), c_int(out.stride(0)), c_int(_dt(out)), c_int(n_tokens), c_int(H), c_int(V),
                                      _stream()))
