"""Choice of kernel for the experts of a mixture-of-experts feed-forward.

Few tokens: every (token, choice) streams the rows of its expert (bound by the bytes of the chosen experts).
More tokens on the bf16 path: grouped tensor-core products over the (token, choice) pairs sorted by expert, so an
expert's matrices are read once per tile of rows: on the tcgen05 product kernel (tiles of 128 rows) when an expert
gets about a tile's worth of pairs, on a warp-level kernel with tiles of 64 rows below that.  The 32-bit path
always streams."""
from __future__ import annotations

import os

import torch

from . import layer_ops as L

GROUPED_FROM = int(os.environ.get("INFERO_MOE_GROUPED_FROM", "5"))     # tokens from which the grouped path runs
TC_PAIRS_PER_EXPERT = int(os.environ.get("INFERO_MOE_TC_FROM", "96"))  # pairs per expert from which tcgen05 tiles pay


def experts(h, gate_up, down, top_idx, top_w, shared, shared_gate, y, act=None) -> None:
    """``act``: the experts' gated activation as (kind, limit, alpha) (``layer_ops.GLU_KINDS``); None: silu(g) * u."""
    T, d = h.shape
    ff = gate_up.shape[1] // 2
    E, top = gate_up.shape[0], top_idx.shape[1]
    # streaming reads an expert once per pair that chose it, the grouped products once per tile of its pairs: with no
    # more pairs than experts streaming reads no more than they do
    if (h.dtype == torch.bfloat16 and T >= GROUPED_FROM and T * top > E and d % 8 == 0 and ff % 8 == 0
            and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0):
        if T * top >= TC_PAIRS_PER_EXPERT * E and gate_up.data_ptr() % 16 == 0 and down.data_ptr() % 16 == 0:
            L.moe_experts_tc(h, gate_up, down, top_idx, top_w, shared, shared_gate, y, act)
        else:
            L.moe_experts_grouped(h, gate_up, down, top_idx, top_w, shared, shared_gate, y, act)
        return
    # the streaming kernels index (token, choice) pairs by a grid dimension of at most 65,535
    step = max(1, 65535 // top_idx.shape[1])
    for a in range(0, T, step):
        b = min(T, a + step)
        L.moe_experts_streamed(h[a:b], gate_up, down, top_idx[a:b], top_w[a:b],
                               None if shared is None else shared[a:b], None if shared_gate is None else shared_gate[a:b],
                               y[a:b], act)


def plain_experts(h, up, down, top_idx, top_w, weight_input: bool, shared, y) -> None:
    """Ungated experts down(relu(up x)^2), up [E, ff, d], down [E, d, ff]: y[t] = sum_c expert_c(w_c h[t]) where the
    weight multiplies the expert's input (``weight_input``), else sum_c w_c expert_c(h[t]); ``shared`` float32 [T, d]
    or None is added.  More pairs than experts on the bf16 path: grouped tcgen05 products; else every pair streams its
    expert."""
    from . import Partials
    T, d = h.shape
    E, ff, _ = up.shape
    top = top_idx.shape[1]
    if (h.dtype == torch.bfloat16 and T >= GROUPED_FROM and T * top > E and d % 8 == 0 and ff % 8 == 0
            and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0 and up.data_ptr() % 16 == 0 and down.data_ptr() % 16 == 0):
        if isinstance(shared, Partials):
            shared = shared.materialize(torch.float32)
        L.moe_plain_tc(h, up, down, top_idx, top_w, weight_input, shared, y)
        return
    step = max(1, 65535 // top)
    if T <= step:                      # one launch: the shared expert's partial sums are added up inside it
        L.moe_plain_streamed(h, up, down, top_idx, top_w, weight_input, shared, y)
        return
    if isinstance(shared, Partials):
        shared = shared.materialize(torch.float32)
    for a in range(0, T, step):
        b = min(T, a + step)
        L.moe_plain_streamed(h[a:b], up, down, top_idx[a:b], top_w[a:b], weight_input,
                             None if shared is None else shared[a:b], y[a:b])
