"""Wrappers of the kernels behind the gated post-norm block, the HGRN2 and differential-attention mixers
and the mixture-of-experts feed-forward (``csrc/gated_norm.cu``, ``hgrn2.cu``, ``diff_attention.cu``,
``moe.cu``).  Small vectors (biases, norm weights, convolution taps) are float32 on both precisions."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong
from typing import Optional

import torch

from . import _check, _dt, _i32, _ptr, _stream, lib


def _f32(t: Optional[torch.Tensor], name: str) -> Optional[torch.Tensor]:
    if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
        raise TypeError(f"{name} must be a contiguous float32 tensor")
    return t


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out (bf16) = x (float32), elementwise."""
    assert x.dtype == torch.float32 and out.dtype == torch.bfloat16 and x.is_contiguous() and out.is_contiguous()
    assert x.numel() == out.numel()
    _check(lib().infero_cast_rows_bf16(_ptr(x), _ptr(out), c_longlong(x.numel()), _stream()))


def gated_scalar_norm_add(x: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor],
                          gate_bias: Optional[torch.Tensor], norm_w: torch.Tensor, eps: float,
                          h_out: Optional[torch.Tensor] = None) -> None:
    """z = y * sigmoid(gate + gate_bias) (z = y without a gate); x += z / sqrt(mean(z^2) + eps) * norm_w[0];
    ``h_out`` (bf16) receives the new x.  x, y, gate float32 (y and gate may be column slices)."""
    T, d = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and y.shape == (T, d) and y.stride(1) == 1
    _f32(norm_w, "norm_w"), _f32(gate_bias, "gate_bias")
    assert y.dtype == torch.float32 and (gate is None or (gate.dtype == torch.float32 and gate.shape == (T, d) and gate.stride(1) == 1))
    assert h_out is None or (h_out.dtype == torch.bfloat16 and h_out.is_contiguous() and h_out.shape == (T, d))
    _check(lib().infero_gated_scalar_norm_add(_ptr(x), _ptr(y), c_int(y.stride(0)), _ptr(gate),
                                              c_int(gate.stride(0) if gate is not None else 0), _ptr(gate_bias),
                                              _ptr(norm_w), c_float(eps), _ptr(h_out), c_int(T), c_int(d), _stream()))


def hgrn2_scan(proj: torch.Tensor, q_off: int, f_off: int, v_off: int, f_bias: torch.Tensor, lower: torch.Tensor,
               out_w: torch.Tensor, eps: float, state: torch.Tensor, entry_q_start: torch.Tensor,
               entry_q_len: torch.Tensor, entry_slot: torch.Tensor, out: torch.Tensor, n_entries: int,
               H: int, D: int, V: int, q_lens=None) -> None:
    """The recurrence of every request of the step over its new tokens; see csrc/hgrn2.cu.
    proj float32 [T, >= ...] (row stride free); state float32 [slots, H, D, V]; out [T, H*V].
    ``q_lens``: the host's copy of ``entry_q_len``; with it, long portions run by chunks side by side."""
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and state.dtype == torch.float32 and state.is_contiguous()
    assert tuple(state.shape[1:]) == (H, D, V) and out.shape[1] == H * V and out.stride(1) == 1
    _f32(f_bias, "f_bias"), _f32(lower, "lower"), _f32(out_w, "out_w")
    max_chunks, any_short, chunk_state, chunk_decay, chunk0 = 0, 1, None, None, None
    if q_lens is not None:
        chunk, long_ = _hgrn2_sizes()
        counts = [(-(-int(n) // chunk) if int(n) >= long_ else 0) for n in q_lens]
        max_chunks = max(counts, default=0)
        if max_chunks:
            any_short = int(any(c == 0 for c in counts))
            firsts, total = [], 0
            for c in counts:
                firsts.append(total)
                total += c
            host = torch.empty(len(firsts), dtype=torch.int32, pin_memory=True)     # (pinned: the copy is asynchronous)
            host.numpy()[:] = firsts
            chunk0 = host.to(proj.device, non_blocking=True)
            chunk_state = torch.empty((total, H, D, V), dtype=torch.float32, device=proj.device)
            chunk_decay = torch.empty((total, H, D), dtype=torch.float32, device=proj.device)
    _check(lib().infero_hgrn2_scan(_ptr(proj), c_int(proj.stride(0)), c_int(q_off), c_int(f_off), c_int(v_off),
                                   _ptr(f_bias), _ptr(lower), _ptr(out_w), c_float(eps), _ptr(state),
                                   _ptr(_i32(entry_q_start, "entry_q_start")), _ptr(_i32(entry_q_len, "entry_q_len")),
                                   _ptr(_i32(entry_slot, "entry_slot")), _ptr(out), c_int(_dt(out)), c_int(out.stride(0)),
                                   c_int(n_entries), c_int(H), c_int(D), c_int(V), c_int(max_chunks), _ptr(chunk_state),
                                   _ptr(chunk_decay), _ptr(chunk0), c_int(any_short), _stream()))


_HGRN2_SIZES = []


def _hgrn2_sizes():
    if not _HGRN2_SIZES:
        _HGRN2_SIZES.extend([int(lib().infero_hgrn2_chunk()), int(lib().infero_hgrn2_long())])
    return _HGRN2_SIZES


def qkv_prepare(proj: torch.Tensor, conv_w: Optional[torch.Tensor], taps: int, conv_state: Optional[torch.Tensor],
                q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float,
                inv_freq: Optional[torch.Tensor], positions, tok_entry, entry_q_start, entry_slot, block_table,
                q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int, n_q_units: int,
                n_k_units: int, G: int, D: int, V: int, write_cache: bool = True, q_pad: bool = False) -> None:
    """Convolution over time (``conv_w`` float32 [taps, channels]), per-map RMS norm, adjacent-pair rotary, q to
    ``q_out``, k and v to their pages; see csrc/diff_attention.cu.  ``q_pad``: q_out is [T, n_q_units * 2 D], every map a query as wide as a key row
    with zeros in the other map's columns."""
    T = q_out.shape[0]
    assert q_out.shape[1] == n_q_units * D * (2 if q_pad else 1)
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and q_out.stride(1) == 1
    assert k_cache.dtype == q_out.dtype == v_cache.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape[-1] == (n_k_units // G) * D and v_cache.shape[-1] == V and k_cache.shape[1] == G
    _f32(conv_w, "conv_w"), _f32(conv_state, "conv_state"), _f32(q_norm, "q_norm"), _f32(k_norm, "k_norm")
    assert conv_w is None or tuple(conv_w.shape) == (taps, (n_q_units + n_k_units) * D + G * V)
    rot = 0 if inv_freq is None else 2 * inv_freq.numel()
    _check(lib().infero_qkv_prepare(
        _ptr(proj), c_int(proj.stride(0)), _ptr(conv_w), c_int(taps), _ptr(conv_state), _ptr(q_norm), _ptr(k_norm),
        c_float(eps), _ptr(_f32(inv_freq, "inv_freq")), c_int(rot), _ptr(_i32(positions, "positions")),
        _ptr(_i32(tok_entry, "tok_entry")), _ptr(_i32(entry_q_start, "entry_q_start")),
        _ptr(_i32(entry_slot, "entry_slot")), _ptr(_i32(block_table, "block_table")), c_int(block_table.shape[1]),
        _ptr(q_out), c_int(q_out.stride(0)), _ptr(k_cache), _ptr(v_cache), c_int(_dt(q_out)), c_int(page_size),
        c_int(T), c_int(n_q_units), c_int(n_k_units), c_int(G), c_int(D), c_int(V), c_int(1 if write_cache else 0),
        c_int(1 if q_pad else 0), _stream()))


def diff_combine(maps: torch.Tensor, out: torch.Tensor, H: int, V: int, lam: float, eps: float, out_scale: float) -> None:
    """maps [T, H*2*V] (per head the two maps' attention results) -> out [T, H*V]: a1 - lam a2, weightless RMS norm
    over V, times out_scale."""
    T = maps.shape[0]
    assert maps.dtype == out.dtype and maps.stride(1) == 1 and out.stride(1) == 1 and maps.shape[1] == 2 * H * V
    _check(lib().infero_diff_combine(_ptr(maps), c_int(maps.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(_dt(out)),
                                     c_int(T), c_int(H), c_int(V), c_float(lam), c_float(eps), c_float(out_scale), _stream()))


def conv_state_update(proj: torch.Tensor, conv_state: torch.Tensor, taps: int, entry_q_start, entry_q_len,
                      entry_slot, n_entries: int, channels: int) -> None:
    """The last taps - 1 product rows of every request become its state (float32 [slots, taps-1, channels])."""
    assert conv_state.dtype == torch.float32 and conv_state.is_contiguous()
    assert tuple(conv_state.shape[1:]) == (taps - 1, channels)
    _check(lib().infero_conv_state_update(_ptr(proj), c_int(proj.stride(0)), _ptr(conv_state), c_int(taps),
                                          _ptr(_i32(entry_q_start, "entry_q_start")),
                                          _ptr(_i32(entry_q_len, "entry_q_len")), _ptr(_i32(entry_slot, "entry_slot")),
                                          c_int(n_entries), c_int(channels), _stream()))


def diff_attention_generic(q, out, k_cache, v_cache, block_table, tok_entry, positions, H: int, G: int, D: int,
                           V: int, page_size: int, window: Optional[int], scale: float, lam: float, eps: float,
                           out_scale: float) -> None:
    """One warp per (token, head): two causal softmaxes over the same values, a1 - lam a2, weightless RMS
    norm over V, times out_scale.  q [T, H*2*D], out [T, H*V], caches of q's dtype."""
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_cache.dtype == v_cache.dtype
    _check(lib().infero_diff_attention_generic(
        _ptr(q), c_int(q.stride(0)), _ptr(out), c_int(out.stride(0)), _ptr(k_cache), _ptr(v_cache), c_int(_dt(q)),
        _ptr(_i32(block_table, "block_table")), c_int(block_table.shape[1]), _ptr(_i32(tok_entry, "tok_entry")),
        _ptr(_i32(positions, "positions")), c_int(T), c_int(H), c_int(G), c_int(D), c_int(V), c_int(page_size),
        c_int(window or 0), c_float(scale), c_float(lam), c_float(eps), c_float(out_scale), _stream()))


def moe_select(logits: torch.Tensor, E: int, top: int, gate_col: int = -1):
    """From float32 logits [T, >= E] (row stride free): (top_idx int32 [T, top], top_w float32 [T, top], gate float32
    [T] or None): the ``top`` largest of the first E columns, softmax over those alone; gate = sigmoid(column
    ``gate_col``).  See csrc/moe.cu."""
    T = logits.shape[0]
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[1] >= E
    idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    gate = torch.empty(T, dtype=torch.float32, device=logits.device) if gate_col >= 0 else None
    _check(lib().infero_moe_select(_ptr(logits), c_int(logits.stride(0)), c_int(gate_col), _ptr(idx), _ptr(w), _ptr(gate),
                                   c_int(T), c_int(E), c_int(top), _stream()))
    return idx, w, gate


GLU_KINDS = {"swiglu": 0, "glu_clamped": 1}


def _act_args(act):
    """(kind, limit, alpha) of a gated activation as the kernels take it; None: silu(g) * u."""
    if act is None:
        return c_int(0), c_float(0.0), c_float(1.0)
    kind, limit, alpha = act
    return c_int(GLU_KINDS[kind]), c_float(limit), c_float(alpha)


def moe_experts_streamed(h, gate_up, down, top_idx, top_w, shared, shared_gate, y, act=None) -> None:
    """y[t] = sum_c top_w[t, c] * expert_{top_idx[t, c]}(h[t]) (+ shared_gate[t] * shared[t]); every (token,
    choice) streams its expert's rows.  gate_up [E, 2 ff, d] (rows alternate gate_j, up_j), down [E, d, ff]."""
    T, d = h.shape
    E, ff2, _ = gate_up.shape
    ff, top = ff2 // 2, top_idx.shape[1]
    assert gate_up.dtype == h.dtype == down.dtype and gate_up.is_contiguous() and down.is_contiguous()
    assert tuple(down.shape) == (E, d, ff) and y.dtype == torch.float32 and y.is_contiguous() and y.shape == (T, d)
    scratch = torch.empty((T * top, ff), dtype=h.dtype, device=h.device)
    _check(lib().infero_moe_experts_streamed(_ptr(h), c_int(h.stride(0)), _ptr(gate_up), _ptr(down), c_int(_dt(h)),
                                             _ptr(_i32(top_idx, "top_idx")), _ptr(_f32(top_w, "top_w")),
                                             _ptr(_f32(shared, "shared")), _ptr(_f32(shared_gate, "shared_gate")),
                                             _ptr(scratch), _ptr(y), c_int(T), c_int(d), c_int(ff), c_int(top),
                                             *_act_args(act), _stream()))


def moe_experts_grouped(h, gate_up, down, top_idx, top_w, shared, shared_gate, y, act=None) -> None:
    """The same result as ``moe_experts_streamed`` by grouped tensor-core products (bf16): the (token, choice)
    pairs are sorted by expert into 64-row tiles; see csrc/moe_grouped.cu."""
    T, d = h.shape
    E, ff2, _ = gate_up.shape
    ff, top = ff2 // 2, top_idx.shape[1]
    assert h.dtype == torch.bfloat16 and gate_up.dtype == torch.bfloat16 and down.dtype == torch.bfloat16
    assert gate_up.is_contiguous() and down.is_contiguous() and tuple(down.shape) == (E, d, ff)
    assert y.dtype == torch.float32 and y.is_contiguous() and y.shape == (T, d) and h.stride(1) == 1
    tiles = int(lib().infero_moe_grouped_tiles(c_int(T * top), c_int(E)))
    R = tiles * int(lib().infero_moe_grouped_tile_rows(c_int(T * top), c_int(E)))
    dev = h.device
    ints = torch.empty(2 * R + tiles + 1, dtype=torch.int32, device=dev)
    sorted_pair, a_rows, tile_expert = ints[:R], ints[R:2 * R], ints[2 * R:]
    scratch = torch.empty((R, ff), dtype=torch.bfloat16, device=dev)
    part = torch.empty((T * top, d), dtype=torch.float32, device=dev)
    _check(lib().infero_moe_experts_grouped(_ptr(h), c_int(h.stride(0)), _ptr(gate_up), _ptr(down),
                                            _ptr(_i32(top_idx, "top_idx")), _ptr(_f32(top_w, "top_w")),
                                            _ptr(_f32(shared, "shared")), _ptr(_f32(shared_gate, "shared_gate")),
                                            _ptr(sorted_pair), _ptr(a_rows), _ptr(tile_expert), _ptr(scratch), _ptr(part),
                                            _ptr(y), c_int(T), c_int(d), c_int(ff), c_int(E), c_int(top), *_act_args(act),
                                            _stream()))


def moe_experts_tc(h, gate_up, down, top_idx, top_w, shared, shared_gate, y, act=None) -> None:
    """The same result by grouped products on the tcgen05 kernel: the tokens' rows are copied into expert order in
    tiles of 128 rows, two grouped products (the first with the SwiGLU epilogue) run over them, and the rows of a
    token's choices are added up in ascending order; see csrc/moe_grouped.cu and ``infero_gemm_tc_grouped``."""
    from .tc_gemm import sm_count
    T, d = h.shape
    E, ff2, _ = gate_up.shape
    ff, top = ff2 // 2, top_idx.shape[1]
    assert h.dtype == torch.bfloat16 and gate_up.dtype == torch.bfloat16 and down.dtype == torch.bfloat16
    assert gate_up.is_contiguous() and down.is_contiguous() and tuple(down.shape) == (E, d, ff)
    assert y.dtype == torch.float32 and y.is_contiguous() and y.shape == (T, d) and h.stride(1) == 1
    tiles = int(lib().infero_moe_tc_tiles(c_int(T * top), c_int(E)))
    R, dev = tiles * 128, h.device
    ints = torch.empty(2 * R + tiles + 1 + T * top, dtype=torch.int32, device=dev)
    sorted_pair, a_rows, tile_expert, pair_row = ints[:R], ints[R:2 * R], ints[2 * R:2 * R + tiles + 1], ints[2 * R + tiles + 1:]
    xs = torch.empty((R, d), dtype=torch.bfloat16, device=dev)
    _check(lib().infero_moe_tc_prepare(_ptr(h), c_int(h.stride(0)), _ptr(_i32(top_idx, "top_idx")), _ptr(sorted_pair),
                                       _ptr(a_rows), _ptr(tile_expert), _ptr(pair_row), _ptr(xs), c_int(T), c_int(d),
                                       c_int(E), c_int(top), _stream()))
    scratch = torch.empty((R, ff), dtype=torch.bfloat16, device=dev)
    sms = sm_count(dev)
    _check(lib().infero_gemm_tc_grouped(_ptr(xs), _ptr(gate_up), _ptr(scratch), c_int(1), c_int(R), c_int(2 * ff), c_int(d),
                                        c_int(d), c_int(ff), _ptr(tile_expert), c_int(E), c_int(sms), *_act_args(act),
                                        _stream()))
    rows = torch.empty((R, d), dtype=torch.float32, device=dev)
    _check(lib().infero_gemm_tc_grouped(_ptr(scratch), _ptr(down), _ptr(rows), c_int(0), c_int(R), c_int(d), c_int(ff),
                                        c_int(ff), c_int(d), _ptr(tile_expert), c_int(E), c_int(sms), *_act_args(None),
                                        _stream()))
    _check(lib().infero_moe_tc_combine(_ptr(rows), _ptr(pair_row), _ptr(_f32(top_w, "top_w")), _ptr(_f32(shared, "shared")),
                                       _ptr(_f32(shared_gate, "shared_gate")), _ptr(y), c_int(T), c_int(d), c_int(top),
                                       _stream()))


def moe_select_grouped(logits: torch.Tensor, correction: Optional[torch.Tensor], E: int, top: int, groups: int = 1,
                       keep: int = 1):
    """From float32 logits [T, >= E]: s = softmax over the E experts; the ``top`` largest of s + correction among the
    ``keep`` best of ``groups`` groups of neighbouring experts; (top_idx int32 [T, top], top_w float32 [T, top]) with
    top_w = s of the chosen over their sum.  See csrc/moe.cu."""
    T = logits.shape[0]
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[1] >= E
    assert correction is None or correction.numel() == E
    idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    _check(lib().infero_moe_select_grouped(_ptr(logits), c_int(logits.stride(0)), _ptr(_f32(correction, "correction")),
                                           _ptr(idx), _ptr(w), c_int(T), c_int(E), c_int(top), c_int(groups), c_int(keep),
                                           _stream()))
    return idx, w


def _product_in(v):
    """(pointer source, dtype tag, splits, split stride, shape) of a product given as a tensor or as partial sums."""
    from . import Partials
    if isinstance(v, Partials):
        assert v.bias is None
        return v.data, 0, v.splits, v.split_stride, tuple(v.shape)
    assert v.is_contiguous()
    return v, _dt(v), 1, 0, tuple(v.shape)


def glu_act(gate_up, out: torch.Tensor, act=None) -> None:
    """out[t, j] = glu(g[t, 2j], g[t, 2j + 1]) for g = gate_up (a tensor or ``Partials``; gate and up alternate along a
    row); ``act`` = (kind, limit, alpha), None: silu(g) * u."""
    T, ff = out.shape
    data, dt, splits, stride, shape = _product_in(gate_up)
    assert shape == (T, 2 * ff) and out.is_contiguous()
    _check(lib().infero_glu_act(_ptr(data), c_int(dt), c_int(splits), c_longlong(stride), _ptr(out), c_int(_dt(out)), c_int(T),
                                c_int(ff), *_act_args(act), _stream()))


def relu2(v, out: torch.Tensor) -> None:
    """out = max(v, 0)^2, v a tensor or ``Partials`` of out's shape."""
    T, ff = out.shape
    data, dt, splits, stride, shape = _product_in(v)
    assert shape == (T, ff) and out.is_contiguous()
    _check(lib().infero_relu2(_ptr(data), c_int(dt), c_int(splits), c_longlong(stride), _ptr(out), c_int(_dt(out)), c_int(T),
                              c_int(ff), _stream()))


def add_layernorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                  rows: Optional[torch.Tensor] = None) -> None:
    """x += delta (float32, if given); out = layer norm of x (weight, no bias).  With ``rows`` only those rows are
    normalised and x is left as it is."""
    d = x.shape[1]
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape[1] == d
    assert delta is None or (delta.dtype == torch.float32 and delta.is_contiguous() and delta.shape == x.shape)
    n = out.shape[0]
    assert n == (x.shape[0] if rows is None else rows.numel()) and weight.numel() == d
    _check(lib().infero_add_layernorm(_ptr(x), _ptr(delta), _ptr(_f32(weight, "weight")), c_float(eps), _ptr(out),
                                      c_int(_dt(out)), _ptr(None if rows is None else _i32(rows, "rows")), c_int(n), c_int(d),
                                      _stream()))


def hyper_step(xs: torch.Tensor, y, mix: Optional[torch.Tensor], w_out: Optional[torch.Tensor],
               w_in: Optional[torch.Tensor], norm_w: Optional[torch.Tensor], eps: float, h_out: Optional[torch.Tensor],
               u_out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """One pass over the streams xs (float32 [T, S, d]) of every token: with ``y`` (float32 [T, d], or a product left as
    ``Partials``) the update xs[r] <- sum_s mix[s, r] xs[s] + w_out[r] y; with ``w_in`` and ``norm_w`` the next
    sublayer's input h_out = layer norm(sum_s w_in[s] xs[s]); with ``u_out`` (float32) and no norm the weighted sum itself
    (w_in None: the plain sum).  ``rows``: work on these tokens only."""
    from . import Partials
    T, S, d = xs.shape
    assert xs.dtype == torch.float32 and xs.is_contiguous()
    splits, split_stride, y_stride = 1, 0, 0
    if isinstance(y, Partials):
        assert y.bias is None and tuple(y.shape) == (T, d)
        y, splits, split_stride, y_stride = y.data, y.splits, y.split_stride, d
    elif y is not None:
        assert y.dtype == torch.float32 and y.shape == (T, d) and y.stride(1) == 1
        y_stride = y.stride(0)
    n = T if rows is None else rows.numel()
    for o in (h_out, u_out):
        assert o is None or (o.is_contiguous() and tuple(o.shape) == (n, d))
    assert u_out is None or u_out.dtype == torch.float32
    _check(lib().infero_hyper_step(_ptr(xs), _ptr(y), c_int(y_stride), c_int(splits), c_longlong(split_stride),
                                   _ptr(_f32(mix, "mix")), _ptr(_f32(w_out, "w_out")), _ptr(_f32(w_in, "w_in")),
                                   _ptr(_f32(norm_w, "norm_w")), c_float(eps), _ptr(h_out),
                                   c_int(_dt(h_out) if h_out is not None else 0), _ptr(u_out),
                                   _ptr(None if rows is None else _i32(rows, "rows")), c_int(n), c_int(S), c_int(d), _stream()))


def streams_fill(x: torch.Tensor, xs: torch.Tensor) -> None:
    """xs[t, s] = x[t] for every stream s."""
    T, S, d = xs.shape
    assert x.dtype == xs.dtype == torch.float32 and x.is_contiguous() and xs.is_contiguous() and tuple(x.shape) == (T, d)
    _check(lib().infero_streams_fill(_ptr(x), _ptr(xs), c_int(T), c_int(S), c_int(d), _stream()))


# ---- normed attention, gated linear recurrence (csrc/qk_prepare.cu, rglru.cu) ------------------------------------
def qk_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, norm_mode: int, q_norm_w, k_norm_w, eps: float,
               freq64: Optional[torch.Tensor], amp: float, positions, tok_entry, block_table, page_size: int,
               q_out: torch.Tensor, k_cache, v_cache, H: int, G: int, D: int, V: int, write_cache: bool = True) -> None:
    """From the 32-bit product row of every token (``proj`` [T, >= ...], columns ``q_off`` / ``k_off`` / ``v_off``; a
    negative ``v_off``: the values are the keys as projected) to normed, rotated queries in ``q_out`` [T, H*D] and keys and
    values in the token's page.  ``norm_mode`` 0 none, 1 weighted RMS over the whole projection before the rotation,
    2 unit RMS per head after it, 3 weighted RMS per head before it (weights of D numbers shared by the heads).
    ``freq64`` float64 [rot/2] (None: no rotation), ``amp`` multiplies cos and sin."""
    T = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and q_out.stride(1) == 1 and q_out.shape == (T, H * D)
    rot = 0
    if freq64 is not None:
        assert freq64.dtype == torch.float64 and freq64.is_contiguous()
        rot = 2 * freq64.numel()
    if write_cache:
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == q_out.dtype == v_cache.dtype
        assert k_cache.shape[1:] == (G, page_size, D) and v_cache.shape[1:] == (G, page_size, V)
    if norm_mode == 1:
        assert q_norm_w.numel() == H * D and (not write_cache or k_norm_w.numel() == G * D)
        assert k_norm_w is None or k_norm_w.dtype == q_norm_w.dtype
    if norm_mode == 3:
        assert q_norm_w.numel() == D and (not write_cache or k_norm_w.numel() == D)
        assert k_norm_w is None or k_norm_w.dtype == q_norm_w.dtype
    _check(lib().infero_qk_prepare(
        _ptr(proj), c_int(proj.stride(0)), c_int(q_off), c_int(k_off), c_int(v_off), c_int(norm_mode), _ptr(q_norm_w),
        _ptr(k_norm_w), c_int(_dt(q_norm_w) if q_norm_w is not None else 0), c_float(eps), _ptr(freq64), c_int(rot),
        c_float(amp), _ptr(_i32(positions, "positions")), _ptr(_i32(tok_entry, "tok_entry")),
        _ptr(_i32(block_table, "block_table")), c_int(block_table.shape[1]), c_int(page_size), _ptr(q_out),
        c_int(q_out.stride(0)), _ptr(k_cache if write_cache else None), _ptr(v_cache if write_cache else None),
        c_int(_dt(q_out)), c_int(1 if write_cache else 0), c_int(T), c_int(H), c_int(G), c_int(D), c_int(V), _stream()))


def head_gate(a: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, H: int, V: int, scale: float = 1.0) -> None:
    """out[t, h*V + v] = a[t, h*V + v] * sigmoid(gate[t, h]) * scale (no gate: only the factor); gate float32, a column
    slice allowed; ``out`` may be ``a`` or a column slice of a wider array."""
    T = a.shape[0]
    assert a.shape == (T, H * V) and out.shape == (T, H * V) and a.stride(1) == 1 and out.stride(1) == 1 and a.dtype == out.dtype
    assert gate is None or (gate.dtype == torch.float32 and gate.shape == (T, H) and gate.stride(1) == 1)
    _check(lib().infero_head_gate(_ptr(a), c_int(a.stride(0)), _ptr(gate), c_int(gate.stride(0) if gate is not None else 0),
                                  _ptr(out), c_int(out.stride(0)), c_int(_dt(a)), c_int(T), c_int(H), c_int(V), c_float(scale),
                                  _stream()))


def rglru(proj: torch.Tensor, y_off: int, x_off: int, conv_w: torch.Tensor, conv_b: Optional[torch.Tensor], w_gates: torch.Tensor,
          ra_b: torch.Tensor, ri_b: torch.Tensor, lam: torch.Tensor, slope: float, state: torch.Tensor, tok_entry,
          entry_q_start, entry_q_len, entry_slot, n_entries: int, out: torch.Tensor, scale: float = 1.0,
          max_q_len: int = 1, tensor_cores: bool = False, conv_wt: Optional[torch.Tensor] = None) -> None:
    """The gated linear recurrence of every request of the step over its new tokens; see csrc/rglru.cu.  ``proj`` float32
    [T, >= ...] holds the gate branch at ``y_off`` and the recurrent branch at ``x_off`` (C columns each, biases added);
    ``conv_w`` float32 [C, taps]; ``w_gates`` [blocks, 2 C/blocks, C/blocks] (float32 or bf16): per block the rows of Ra,
    then those of Ri; ``state`` float32 [slots, taps, C] (rows 0..taps-2 the convolution's last inputs, row taps-1 the
    recurrent state); ``out`` [T, C] (a column slice allowed) receives S * gelu_tanh(y) * scale.  ``max_q_len``: the
    longest portion of the step.  ``tensor_cores``: the gate products of a long bf16 step run as one grouped
    tensor-core product over all blocks, from u rounded to bf16 (32-bit sums); otherwise they are 32-bit throughout.
    ``conv_wt``: ``conv_w`` laid out tap-major, float32 [taps, C], as the kernels read it (made here when absent)."""
    T = proj.shape[0]
    C, taps = conv_w.shape
    blocks, two_bs, bs = w_gates.shape
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and out.shape == (T, C) and out.stride(1) == 1
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (taps, C)
    assert blocks * bs == C and two_bs == 2 * bs and w_gates.is_contiguous()
    _f32(conv_w, "conv_w"), _f32(conv_b, "conv_b"), _f32(ra_b, "ra_b"), _f32(ri_b, "ri_b"), _f32(lam, "lam")
    if conv_wt is None:
        conv_wt = conv_w.t().contiguous()
    assert conv_wt.dtype == torch.float32 and conv_wt.is_contiguous() and tuple(conv_wt.shape) == (taps, C)
    L = lib()
    if int(max_q_len) == 1 and w_gates.dtype == torch.bfloat16 and bs % 8 == 0 and bs <= 256:
        # a step of single tokens: one launch for convolution, gate products and the state's update
        rc = L.infero_rglru_step(_ptr(proj), c_int(proj.stride(0)), c_int(y_off), c_int(x_off), _ptr(conv_wt), _ptr(conv_b),
                                 c_int(taps), _ptr(w_gates), _ptr(ra_b), _ptr(ri_b), _ptr(lam), c_float(slope), _ptr(state),
                                 _ptr(_i32(entry_q_start, "entry_q_start")), _ptr(_i32(entry_q_len, "entry_q_len")),
                                 _ptr(_i32(entry_slot, "entry_slot")), _ptr(out), c_int(out.stride(0)), c_int(_dt(out)),
                                 c_int(n_entries), c_int(C), c_int(blocks), c_float(scale), _stream())
        if rc != 2:
            _check(rc)
            return
    u = torch.empty((T, C), dtype=torch.float32, device=proj.device)
    u16 = None
    rows = -(-T // 128) * 128
    if tensor_cores and T > 256 and w_gates.dtype == torch.bfloat16:
        from . import latent_attention as LA
        u16 = torch.empty((blocks, rows, bs), dtype=torch.bfloat16, device=proj.device)
        if not LA.grouped_ok(u16, w_gates):
            u16 = None
    _check(L.infero_rglru_conv(_ptr(proj), c_int(proj.stride(0)), c_int(x_off), _ptr(conv_wt), _ptr(conv_b), c_int(taps),
                               _ptr(state), _ptr(_i32(tok_entry, "tok_entry")), _ptr(_i32(entry_q_start, "entry_q_start")),
                               _ptr(_i32(entry_slot, "entry_slot")), _ptr(u), _ptr(u16), c_int(blocks), c_longlong(rows), c_int(T),
                               c_int(C), _stream()))
    if u16 is not None:
        # one grouped product over all blocks: [blocks, rows, bs] x [blocks, 2 bs, bs]^T -> [blocks, rows, 2 bs]
        gates = torch.empty((blocks, rows, 2 * bs), dtype=torch.float32, device=proj.device)
        LA.per_head_product(u16, w_gates, gates, T)
        g_tok, g_blk = 2 * bs, rows * 2 * bs
    else:
        gates = torch.empty((T, 2 * C), dtype=torch.float32, device=proj.device)
        _check(L.infero_rglru_gates(_ptr(u), _ptr(w_gates), c_int(_dt(w_gates)), _ptr(gates), c_int(T), c_int(C), c_int(blocks),
                                    _stream()))
        g_tok, g_blk = 2 * C, 2 * bs
    _check(L.infero_rglru_scan(_ptr(proj), c_int(proj.stride(0)), c_int(y_off), c_int(x_off), _ptr(u), _ptr(gates),
                               c_longlong(g_tok), c_longlong(g_blk), _ptr(ra_b), _ptr(ri_b), _ptr(lam), c_float(slope),
                               c_int(taps), _ptr(state), _ptr(_i32(entry_q_start, "entry_q_start")),
                               _ptr(_i32(entry_q_len, "entry_q_len")), _ptr(_i32(entry_slot, "entry_slot")), _ptr(out),
                               c_int(out.stride(0)), c_int(_dt(out)),
                               c_int(n_entries), c_int(C), c_int(blocks), c_int(max(1, int(max_q_len))), c_float(scale), _stream()))


# ---- state-space recurrence (csrc/ssd.cu), gated group norm ---------------------------------------------------------
def ssd_state_floats(heads: int, N: int, P: int, groups: int, taps: int) -> int:
    """Floats of one request's state: the convolution's last taps - 1 inputs, then S [heads, N, P]."""
    return (taps - 1) * (heads * P + 2 * groups * N) + heads * N * P


def ssd(proj: torch.Tensor, z_off: int, x_off: int, dt_off: int, conv_w: torch.Tensor, conv_b: Optional[torch.Tensor],
        dt_bias: torch.Tensor, a_log: torch.Tensor, skip: torch.Tensor, norm_w: torch.Tensor, eps: float, norm_groups: int,
        state: torch.Tensor, tok_entry, entry_q_start, entry_q_len, entry_slot, n_entries: int, out: torch.Tensor,
        heads: int, groups: int, N: int, P: int, scale: float = 1.0, max_q_len: int = 1) -> None:
    """The state-space recurrence of every request of the step over its new tokens, and the gated, grouped norm of its
    result; see csrc/ssd.cu.  ``proj`` float32 [T, >= ...] holds [z | x B C | dt] at ``z_off`` / ``x_off`` / ``dt_off``;
    ``conv_w`` float32 [CH, taps] over the CH = heads P + 2 groups N channels of [x | B | C]; ``state`` float32
    [slots, floats] (``ssd_state_floats``); ``out`` [T, heads * P] (a column slice allowed) receives
    rms_parts(y * silu(z)) * norm_w * scale.  ``max_q_len``: the longest portion of the step."""
    from .tc_gemm import sm_count
    T = proj.shape[0]
    CH, taps = conv_w.shape
    inner = heads * P
    assert CH == inner + 2 * groups * N and proj.dtype == torch.float32 and proj.stride(1) == 1
    assert out.shape == (T, inner) and out.stride(1) == 1
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == ssd_state_floats(heads, N, P, groups, taps)
    _f32(conv_w, "conv_w"), _f32(conv_b, "conv_b"), _f32(dt_bias, "dt_bias"), _f32(a_log, "a_log"), _f32(skip, "skip"), _f32(norm_w, "norm_w")
    dev = proj.device
    L = lib()
    u = torch.empty((T, CH), dtype=torch.float32, device=dev)
    qs, ql, sl = _ptr(_i32(entry_q_start, "entry_q_start")), _ptr(_i32(entry_q_len, "entry_q_len")), _ptr(_i32(entry_slot, "entry_slot"))
    _check(L.infero_ssd_conv(_ptr(proj), c_int(proj.stride(0)), c_int(x_off), _ptr(conv_w), _ptr(conv_b), c_int(taps), _ptr(state),
                             c_longlong(state.stride(0)), _ptr(_i32(tok_entry, "tok_entry")), qs, ql, sl, _ptr(u), c_int(T),
                             c_int(n_entries), c_int(CH), _stream()))
    y = torch.empty((T, inner), dtype=torch.float32, device=dev)
    L.infero_ssd_scan_scratch.restype = c_longlong
    need = int(L.infero_ssd_scan_scratch(c_int(n_entries), c_int(int(max_q_len)), c_int(heads), c_int(N), c_int(P)))
    scratch = torch.empty(need, dtype=torch.float32, device=dev) if need else None
    _check(L.infero_ssd_scan(_ptr(u), _ptr(proj), c_int(proj.stride(0)), c_int(dt_off), _ptr(dt_bias), _ptr(a_log), _ptr(skip),
                             _ptr(state), c_longlong(state.stride(0)), c_int(taps), qs, ql, sl, _ptr(y), c_int(n_entries),
                             c_int(max(1, int(max_q_len))), c_int(heads), c_int(groups), c_int(N), c_int(P), _ptr(scratch),
                             c_int(sm_count(dev)), _stream()))
    gated_group_norm(y, proj[:, z_off:z_off + inner], norm_w, eps, norm_groups, out, scale)


def gated_group_norm(y: torch.Tensor, gate: Optional[torch.Tensor], weight: torch.Tensor, eps: float, parts: int,
                     out: torch.Tensor, scale: float = 1.0) -> None:
    """out = v / sqrt(mean over each of ``parts`` equal parts of v^2 + eps) * weight * scale with v = y * silu(gate)
    (v = y without a gate).  y, gate float32 [T, n] (column slices allowed); out [T, n] of any element type."""
    T, n = y.shape
    assert y.dtype == torch.float32 and y.stride(1) == 1 and out.shape == (T, n) and out.stride(1) == 1
    assert gate is None or (gate.dtype == torch.float32 and gate.shape == (T, n) and gate.stride(1) == 1)
    assert weight.numel() == n
    _check(lib().infero_gated_group_norm(_ptr(y), c_int(y.stride(0)), _ptr(gate), c_int(gate.stride(0) if gate is not None else 0),
                                         _ptr(_f32(weight, "weight")), c_float(eps), c_float(scale), _ptr(out),
                                         c_int(out.stride(0)), c_int(_dt(out)), c_int(T), c_int(n), c_int(parts), _stream()))


# ---- experts chosen by scores, ungated experts (csrc/moe.cu, csrc/moe_grouped.cu) -----------------------------------
def moe_select_scored(logits, E: int, top: int, renorm: bool = False):
    """From float32 logits [T, >= E] (a tensor, or ``Partials``: split-K sums that are added up here): scores
    sigmoid(logit); the ``top`` largest (lowest index wins a tie); (top_idx int32 [T, top], top_w float32 [T, top]) with
    top_w the chosen scores, over their sum where ``renorm``."""
    from . import Partials
    splits, split_stride = 1, 0
    if isinstance(logits, Partials):
        assert logits.bias is None
        splits, split_stride, logits = logits.splits, logits.split_stride, logits.data[0]
    T = logits.shape[0]
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[1] >= E
    idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    _check(lib().infero_moe_select_scored(_ptr(logits), c_int(logits.stride(0)), c_int(splits), c_longlong(split_stride),
                                          _ptr(idx), _ptr(w), c_int(T), c_int(E), c_int(top), c_int(1 if renorm else 0),
                                          _stream()))
    return idx, w


def moe_plain_streamed(h, up, down, top_idx, top_w, weight_input: bool, shared, y) -> None:
    """y[t] = sum_c expert_c(w_c h[t]) (``weight_input``) or sum_c w_c expert_c(h[t]), expert = down(relu(up x)^2),
    (+ shared[t]); every (token, choice) streams its expert's rows.  up [E, ff, d], down [E, d, ff].  ``shared``:
    float32 [T, d], or ``Partials`` of that shape (split-K sums, added up where they are used), or None."""
    from . import Partials
    sh_splits, sh_stride = 1, 0
    if isinstance(shared, Partials):
        assert shared.bias is None and tuple(shared.shape) == tuple(h.shape)
        sh_splits, sh_stride, shared = shared.splits, shared.split_stride, shared.data[0]
    T, d = h.shape
    E, ff, _ = up.shape
    top = top_idx.shape[1]
    assert up.dtype == h.dtype == down.dtype and up.is_contiguous() and down.is_contiguous() and h.stride(1) == 1
    assert tuple(down.shape) == (E, d, ff) and y.dtype == torch.float32 and y.is_contiguous() and y.shape == (T, d)
    scratch = torch.empty((T * top, ff), dtype=h.dtype, device=h.device)
    _check(lib().infero_moe_experts_plain_streamed(_ptr(h), c_int(h.stride(0)), _ptr(up), _ptr(down), c_int(_dt(h)),
                                                   _ptr(_i32(top_idx, "top_idx")), _ptr(_f32(top_w, "top_w")),
                                                   c_int(1 if weight_input else 0), _ptr(_f32(shared, "shared")),
                                                   c_int(sh_splits), c_longlong(sh_stride), _ptr(scratch), _ptr(y), c_int(T),
                                                   c_int(d), c_int(ff), c_int(top), _stream()))


def moe_plain_tc(h, up, down, top_idx, top_w, weight_input: bool, shared, y) -> None:
    """The same result by grouped products on the tcgen05 kernel (bf16): the tokens' rows are copied into expert order
    in tiles of 128 rows, times their pair's weight where it multiplies the expert's input; the first grouped product
    applies the squared relu in its epilogue; the rows of a token's choices are added up in ascending order."""
    from .tc_gemm import sm_count
    T, d = h.shape
    E, ff, _ = up.shape
    top = top_idx.shape[1]
    assert h.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and down.dtype == torch.bfloat16
    assert up.is_contiguous() and down.is_contiguous() and tuple(down.shape) == (E, d, ff)
    assert y.dtype == torch.float32 and y.is_contiguous() and y.shape == (T, d) and h.stride(1) == 1
    L = lib()
    tiles = int(L.infero_moe_tc_tiles(c_int(T * top), c_int(E)))
    R, dev = tiles * 128, h.device
    ints = torch.empty(2 * R + tiles + 1 + T * top, dtype=torch.int32, device=dev)
    sorted_pair, a_rows, tile_expert, pair_row = ints[:R], ints[R:2 * R], ints[2 * R:2 * R + tiles + 1], ints[2 * R + tiles + 1:]
    xs = torch.empty((R, d), dtype=torch.bfloat16, device=dev)
    _f32(top_w, "top_w")
    _check(L.infero_moe_tc_prepare_scaled(_ptr(h), c_int(h.stride(0)), _ptr(_i32(top_idx, "top_idx")), _ptr(sorted_pair),
                                          _ptr(a_rows), _ptr(tile_expert), _ptr(pair_row), _ptr(xs), c_int(T), c_int(d),
                                          c_int(E), c_int(top), _ptr(top_w if weight_input else None), _stream()))
    act = torch.empty((R, ff), dtype=torch.bfloat16, device=dev)
    sms = sm_count(dev)
    _check(L.infero_gemm_tc_grouped(_ptr(xs), _ptr(up), _ptr(act), c_int(2), c_int(R), c_int(ff), c_int(d), c_int(d),
                                    c_int(ff), _ptr(tile_expert), c_int(E), c_int(sms), *_act_args(None), _stream()))
    rows = torch.empty((R, d), dtype=torch.float32, device=dev)
    _check(L.infero_gemm_tc_grouped(_ptr(act), _ptr(down), _ptr(rows), c_int(0), c_int(R), c_int(d), c_int(ff), c_int(ff),
                                    c_int(d), _ptr(tile_expert), c_int(E), c_int(sms), *_act_args(None), _stream()))
    _check(L.infero_moe_tc_combine(_ptr(rows), _ptr(pair_row), _ptr(None if weight_input else top_w), _ptr(_f32(shared, "shared")),
                                   _ptr(None), _ptr(y), c_int(T), c_int(d), c_int(top), _stream()))
